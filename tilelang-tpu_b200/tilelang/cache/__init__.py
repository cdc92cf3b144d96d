"""Kernel cache (role of tilelang/cache/kernel_cache.py:100-186, whose lookup is commented out in
the reference fork so every compile builds a new kernel).  Binding is cheap here, so the cache
is a small in-memory map from (program object, options) to the JITKernel."""
from __future__ import annotations

import threading

_lock = threading.Lock()
_cache: dict = {}


def _key(func, out_idx, target, mode):
    oi = tuple(out_idx) if isinstance(out_idx, (list, tuple)) else out_idx
    return (id(func), oi, str(target), str(mode))


def cached(func=None, out_idx=None, *args, target="auto", target_host=None, execution_backend="cython",
           verbose=False, pass_configs=None, mode="pcie"):
    from ..jit.kernel import JITKernel
    key = _key(func, out_idx, target, mode)
    with _lock:
        hit = _cache.get(key)
        if hit is not None and hit.prim_func is func:
            return hit
    kernel = JITKernel(func, out_idx=out_idx, execution_backend=execution_backend, target=target,
                       target_host=target_host, verbose=verbose, pass_configs=pass_configs, mode=mode)
    with _lock:
        _cache[key] = kernel
    return kernel


def clear_cache():
    with _lock:
        _cache.clear()
