"""Target names (cf. tilelang/utils/target.py:10-18 of the reference, which lists
auto/cuda/hip/webgpu/c/llvm/tpu).  This build has exactly one backend."""
from __future__ import annotations

import os

AVALIABLE_TARGETS = {"auto", "b200"}        # spelling of the constant kept from the reference
_ALIASES = {"cuda": "b200", "sm_100a": "b200"}


def determine_target(target="auto") -> str:
    """Resolve a target string to "b200".  "tpu" (the reference's BM1690 target) is accepted only
    when TL_B200_ACCEPT_TPU_TARGET=1, so unmodified demo scripts can run against this backend."""
    t = str(target)
    t = _ALIASES.get(t, t)
    if t == "tpu" and os.environ.get("TL_B200_ACCEPT_TPU_TARGET", "0") == "1":
        t = "b200"
    if t not in AVALIABLE_TARGETS:
        raise AssertionError(f"Target {target} is not supported: this build only has the b200 (sm_100a) "
                             f"backend; choose from {sorted(AVALIABLE_TARGETS)}")
    return "b200"
