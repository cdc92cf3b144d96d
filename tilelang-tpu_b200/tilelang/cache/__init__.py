"""Kernel cache and tile-choice table.

Role of tilelang/cache/kernel_cache.py:100-186 in the reference (whose lookup is commented out in the fork, so
every compile there builds a new kernel) and of the result store of its tuner.  Two things are kept:

* the bound kernels of this process, keyed by the CONTENT of the program (its recorded op stream, parameters,
  `out_idx`, target and mode) - two builders that produce the same program share one JITKernel;
* on disk (`$TILELANG_B200_CACHE_DIR`, default `~/.cache/tilelang_b200`), one small JSON record per program key
  with the kernel it was bound to, and `tile_table.json`, the shape -> tile choices that `tilelang.autotuner`
  measured.  Binding is cheap, so a record is not needed to run; it is what a later process checks its own
  binding against (a library update that binds a program differently is reported, not silently accepted), and
  the tile table is what makes a tuning run worth doing once.
"""
from __future__ import annotations

import hashlib
import json
import os
import threading
from pathlib import Path
from typing import Optional

_lock = threading.Lock()
_cache: dict = {}
_tile_table: Optional[dict] = None
_enabled = True


def cache_dir() -> Path:
    return Path(os.environ.get("TILELANG_B200_CACHE_DIR", str(Path.home() / ".cache" / "tilelang_b200")))


def enable_cache(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def is_cache_enabled() -> bool:
    return _enabled and os.environ.get("TILELANG_B200_DISABLE_CACHE", "0") != "1"


def program_key(func, out_idx=None, target="auto", mode="pcie") -> str:
    """sha256 over the program's listing (parameters, grid, op stream), `out_idx`, target, mode and the library's ABI version."""
    from .. import _native
    oi = list(out_idx) if isinstance(out_idx, (list, tuple)) else out_idx
    data = {"program": func.script(), "attrs": {k: repr(v) for k, v in sorted(func.attrs.items()) if k != "global_symbol"},
            "out_idx": oi, "target": str(target), "mode": str(mode), "abi": _native.ABI_VERSION}
    return hashlib.sha256(json.dumps(data, sort_keys=True).encode()).hexdigest()


def _record_path(key: str) -> Path:
    return cache_dir() / "programs" / f"{key}.json"


def _write_json(path: Path, obj) -> None:
    try:
        path.parent.mkdir(parents=True, exist_ok=True)
        tmp = path.with_suffix(f".tmp{os.getpid()}")
        tmp.write_text(json.dumps(obj, indent=1, sort_keys=True, default=str))
        os.replace(tmp, path)                      # atomic: concurrent processes never see half a file
    except OSError:
        pass                                       # a read-only home must not stop a program from running


def load_record(key: str) -> Optional[dict]:
    try:
        return json.loads(_record_path(key).read_text())
    except (OSError, ValueError):
        return None


def cached(func=None, out_idx=None, *args, target="auto", target_host=None, execution_backend="cython",
           verbose=False, pass_configs=None, mode="pcie"):
    from ..jit.kernel import JITKernel

    def build():
        return JITKernel(func, out_idx=out_idx, execution_backend=execution_backend, target=target,
                         target_host=target_host, verbose=verbose, pass_configs=pass_configs, mode=mode)

    if not is_cache_enabled():
        return build()
    key = program_key(func, out_idx, target, mode)
    with _lock:
        hit = _cache.get(key)
    if hit is not None:
        return hit
    kernel = build()
    bound = kernel.adapter.bound
    record = {"program": bound.program, "entry_point": bound.entry_point, "facts": bound.facts, "name": func.name}
    previous = load_record(key)
    if previous is not None and (previous.get("program"), previous.get("entry_point")) != (bound.program, bound.entry_point):
        import warnings
        warnings.warn(f"program {func.name} was bound to {previous.get('entry_point')} by an earlier run and is bound to "
                      f"{bound.entry_point} now (key {key[:12]}); the stored record is replaced")
        previous = None
    if previous is None:
        _write_json(_record_path(key), record)
    kernel.cache_key = key
    with _lock:
        _cache[key] = kernel
    return kernel


def clear_cache(disk: bool = False):
    global _tile_table
    with _lock:
        _cache.clear()
        if disk:
            _tile_table = None
            import shutil
            shutil.rmtree(cache_dir(), ignore_errors=True)


# ------------------------------------------------------------------------------- tile table
def _table_path() -> Path:
    return cache_dir() / "tile_table.json"


def _table() -> dict:
    global _tile_table
    if _tile_table is None:
        try:
            _tile_table = json.loads(_table_path().read_text())
        except (OSError, ValueError):
            _tile_table = {}
    return _tile_table


def tile_key(kernel: str, **shape) -> str:
    return kernel + "|" + ",".join(f"{k}={shape[k]}" for k in sorted(shape))


def tile_choice(kernel: str, **shape) -> Optional[dict]:
    """The tuned choice for this kernel and shape, or None (the library's own rule applies)."""
    if not is_cache_enabled():
        return None
    with _lock:
        return _table().get(tile_key(kernel, **shape))


def set_tile_choice(kernel: str, choice: dict, **shape) -> None:
    with _lock:
        _table()[tile_key(kernel, **shape)] = dict(choice)
        _write_json(_table_path(), _table())
