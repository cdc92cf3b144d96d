"""ctypes binding of libtl_b200.so.

The reference loads one generated `main.so` per program and binds
`tilelang_tpu_run(void**) -> int` (tilelang/jit/adapter/cython/adapter.py:213-216).  This
module binds the pre-built kernel library instead; the prototypes below restate
include/tl_b200.h.  There is no fallback: if the library is missing, loading raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

_PKG_ROOT = Path(__file__).resolve().parent.parent
DEFAULT_LIB = _PKG_ROOT / "lib" / "libtl_b200.so"

TL_F32, TL_F16, TL_BF16, TL_E4M3, TL_I32, TL_U32, TL_I16 = range(7)
ABI_VERSION = 100          # TL_B200_VERSION of include/tl_b200.h

# name -> (restype, argtypes).  Kept in declaration order of include/tl_b200.h.
PROTOTYPES = {
    "tl_b200_init": (c_int, [c_int]),
    "tl_b200_version": (c_int, []),
    "tl_b200_last_error": (c_char_p, []),
    "tl_b200_launch_count": (c_int64, []),
    "tl_b200_device_status": (c_int, []),
    "tl_b200_selftest_bounded_wait": (c_int, [c_int64, c_void_p]),
    "tl_b200_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int, c_void_p]),
    "tl_b200_rope": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "tl_b200_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "tl_b200_reduce_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p]),
    "tl_b200_unary": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]),
    "tl_b200_binary": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_float, c_int, c_void_p]),
    "tl_b200_gather_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p]),
    "tl_b200_topk": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int64, c_int, c_void_p]),
    "tl_b200_gemm_fp8_blockscale": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                            c_int64, c_int, c_void_p]),
    "tl_b200_flash_attn_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                       c_int64, c_float, c_int, c_int, c_int, c_int, c_void_p]),
    "tl_b200_mla_decode_dense": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                         c_int64, c_int64, c_int64, c_float, c_int, c_void_p]),
    "tl_b200_mla_decode_paged_workspace_bytes": (c_int64, [c_int64]),
    "tl_b200_mla_decode_paged_split_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64]),
    "tl_b200_mla_decode_paged": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                         c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_int, c_void_p,
                                         c_int64, c_void_p]),
    "tl_b200_mla_decode_paged_gqa": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                             c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_void_p]),
    "tl_b200_mla_decode_paged_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                                 c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_void_p]),
    "tl_b200_rope_add": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "tl_b200_copy2d": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p]),
    "tl_b200_fill": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_float, c_int, c_void_p]),
    "tl_b200_gemm": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_void_p]),
    "tl_b200_gemm_tiled": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p]),
    "tl_b200_mlp_gate_up": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p]),
    "tl_b200_tile_program_registers": (c_int, [c_int64]),
    "tl_b200_tile_program": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int64, c_void_p]),
    "tl_b200_run": (c_int, [c_int, ctypes.POINTER(c_void_p), ctypes.POINTER(c_int64), c_void_p]),
}

# kernel ids of tl_b200_run (values of the TL_B200_K_* macros)
KERNEL_IDS = {name: i + 1 for i, name in enumerate(
    ["rmsnorm", "rope", "swiglu", "reduce_rows", "unary", "binary", "rope_add", "copy2d", "fill", "gather_rows", "topk",
     "gemm", "mlp_gate_up", "gemm_fp8_blockscale", "flash_attn_fwd", "mla_decode_dense", "mla_decode_paged"])}


def float_bits(v: float) -> int:
    """A float argument of tl_b200_run: its IEEE-754 single-precision bit pattern."""
    import struct
    return struct.unpack("<I", struct.pack("<f", float(v)))[0]


def run(kernel: str, pointers, meta, stream) -> int:
    """Call `tl_b200_run`: the pointer arguments and the non-pointer arguments of the typed entry point."""
    args = (c_void_p * len(pointers))(*[c_void_p(p) for p in pointers])
    m = (c_int64 * len(meta))(*[int(x) for x in meta])
    return load().tl_b200_run(KERNEL_IDS[kernel], args, m, stream)


class NativeLibraryError(RuntimeError):
    pass


_lib = None


def lib_path() -> Path:
    return Path(os.environ.get("TL_B200_LIB", str(DEFAULT_LIB)))


def load() -> ctypes.CDLL:
    """dlopen the kernel library and attach prototypes.  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not path.exists():
        raise NativeLibraryError(
            f"{path} not found: build it with `python __graft_entry__.py` (or "
            f"`python tilelang-tpu_b200/tilelang/_build.py`); there is no CPU fallback")
    lib = ctypes.CDLL(str(path))
    for name, (restype, argtypes) in PROTOTYPES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise NativeLibraryError(f"{path} does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    msg = load().tl_b200_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(status: int, what: str) -> int:
    """Raise on a non-zero status, carrying the library's message (cf. the reference's
    cython wrapper raising on a failed call, cython_wrapper.pyx:160-163)."""
    if status != 0:
        raise RuntimeError(f"{what} failed with status {status}: {last_error()}")
    return status
