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


def test_generic_entry_point_dispatches_and_validates_without_gpu():
    """`tl_b200_run(kernel_id, void** args, meta, stream)` keeps the `void**` shape of the reference's
    generated symbol; argument validation of the typed entry point behind it runs before any CUDA call."""
    from tilelang import _native
    import re as _re
    header = (ROOT / "include" / "tl_b200.h").read_text()
    ids = {m.group(1).lower(): int(m.group(2)) for m in _re.finditer(r"#define TL_B200_K_([A-Z0-9_]+) (\d+)", header)}
    assert ids == _native.KERNEL_IDS
    rc = _native.run("rmsnorm", [0, 0, 0], [4, 4, _native.float_bits(1e-6), _native.TL_BF16], None)
    assert rc == -1 and "null" in _native.last_error()
    rc = _native.run("rope", [0, 0, 0, 0], [4, 3, 1, _native.TL_BF16], None)
    assert rc == -1 and "even" in _native.last_error()
    lib = _native.load()
    rc = lib.tl_b200_run(99, (ctypes.c_void_p * 1)(), (ctypes.c_int64 * 1)(), None)
    assert rc == -1 and "unknown kernel id" in _native.last_error()


def test_device_status_error_path_on_the_host(monkeypatch):
    """`ops.check_device_status()` turns a non-zero status word into TL_B200_EDEVICE (-4); the word itself is
    faked here, the GPU test makes a real bounded wait run out."""
    from tilelang import _native, ops

    class FakeLib:
        def tl_b200_device_status(self):
            return 1

        def tl_b200_last_error(self):
            return b"a kernel gave up a bounded wait (device status 1)"

    monkeypatch.setattr(_native, "_lib", FakeLib())
    with pytest.raises(RuntimeError, match="TL_B200_EDEVICE.*bounded wait"):
        ops.check_device_status()
    monkeypatch.setattr(_native, "_lib", None)
    lib = _native.load()
    assert lib.tl_b200_device_status() == 0                      # no status word exists without a device
    assert lib.tl_b200_selftest_bounded_wait(0, None) == -1 and "budget" in _native.last_error()
