from .target import AVALIABLE_TARGETS, determine_target  # noqa: F401
