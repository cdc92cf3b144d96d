"""The C-ABI library must load and export every symbol include/tl_b200.h declares (no compute)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "tl_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tl_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert "tl_b200_rmsnorm" in syms and "tl_b200_init" in syms


def test_library_exports_every_declared_symbol():
    from tilelang import _native
    path = _native.lib_path()
    if not path.exists():
        from tilelang import _build
        _build.build()
    lib = ctypes.CDLL(str(path))
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, f"not exported: {missing}"


def test_python_prototypes_cover_header():
    from tilelang import _native
    assert sorted(_native.PROTOTYPES) == declared_symbols()


def test_version_and_error_string_without_gpu():
    from tilelang import _native
    lib = _native.load()
    assert lib.tl_b200_version() == 100
    # argument validation happens before any CUDA call, so it is testable without a device
    rc = lib.tl_b200_rmsnorm(None, None, None, 4, 4, 1e-6, _native.TL_BF16, None)
    assert rc == -1 and "null" in _native.last_error()
    rc = lib.tl_b200_topk(None, None, None, 1, 8, 9, 1, 8, _native.TL_F32, None)
    assert rc == -1 and "exceeds length" in _native.last_error()
    rc = lib.tl_b200_rope(None, None, None, None, 4, 3, 1, _native.TL_BF16, None)
    assert rc == -1 and "even" in _native.last_error()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from tilelang import _native
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setenv("TL_B200_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(_native.NativeLibraryError):
        _native.load()
