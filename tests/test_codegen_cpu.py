"""The generated-kernel path of the row-local executor without a GPU: the program's instruction list is printed as
CUDA C and NVRTC compiles it for sm_100a (nothing is launched here)."""
import pytest

import tilelang.language as T
from tilelang import programs as P
from tilelang.engine import codegen, fuser
from tilelang.language.ir import const_value


def _lower(func):
    c = fuser._Compiler(func).compile()
    grid = [int(const_value(g)) for g in func.grid]
    return c, grid + [1] * (3 - len(grid))


def test_every_instruction_becomes_one_statement():
    c, grid = _lower(P.rmsnorm(64, 4096, eps=1e-6))
    src = codegen.generate(c.ins, grid, c.bm, c.max_width)
    statements = [l for l in src.splitlines() if l.lstrip().startswith("/*") and "*/" in l]
    assert len(statements) == len(c.ins)
    assert "constexpr int TPR = 256, EPT = 16" in src                 # the split of the interpreter kernel for 4096 columns
    assert f"unit0 < {grid[0] * grid[1] * grid[2] * c.bm}ll" in src   # the launch grid and the rows of a block are constants
    # immediates are printed with their exact bits
    assert codegen._f(1.0) == "__uint_as_float(0x3f800000u)" and codegen._f(-0.0) == "__uint_as_float(0x80000000u)"


@pytest.mark.parametrize("make", [lambda: P.rmsnorm(64, 4096, eps=1e-6), lambda: P.rope(128, 8, 128), lambda: P.swiglu(64, 2048),
                                  lambda: P.rmsnorm(32, 200, blk_m=16, dtype="float16", eps=1e-6, weight=False)])
def test_generated_source_compiles_for_sm_100a(make, tmp_path, monkeypatch):
    monkeypatch.setenv("TILELANG_B200_CACHE_DIR", str(tmp_path))
    try:
        codegen._bindings()
    except codegen.Unavailable as why:
        pytest.skip(str(why))
    c, grid = _lower(make())
    src = codegen.generate(c.ins, grid, c.bm, c.max_width)
    cubin = codegen.compile_cubin(src)
    assert cubin[:4] == b"\x7fELF" and len(cubin) > 4096
    # the second request is served from the cache directory
    files = list(tmp_path.glob("gen_*.cubin"))
    assert len(files) == 1 and files[0].read_bytes() == cubin
    assert codegen.compile_cubin(src) == cubin


def test_a_program_that_does_not_compile_is_reported_with_the_log(tmp_path, monkeypatch):
    monkeypatch.setenv("TILELANG_B200_CACHE_DIR", str(tmp_path))
    try:
        codegen._bindings()
    except codegen.Unavailable as why:
        pytest.skip(str(why))
    with pytest.raises(RuntimeError, match="does not compile"):
        codegen.compile_cubin("extern \"C\" __global__ void tile_program() { this is not CUDA }")
