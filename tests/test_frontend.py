"""Host-side front end: tracing of `T.ppl_*` programs, program matching, compile/adapter
argument handling.  CPU only (binding a program needs no GPU; running it does)."""
import ast
import os
from pathlib import Path

import pytest
import torch

import tilelang
import tilelang.language as T
from tilelang.engine import UnsupportedProgram, bind

# root of a checkout of the reference project; the tests that trace its demo files are skipped without it
REFERENCE = Path(os.environ.get("TILELANG_TPU_REFERENCE", "reference-tree-not-given"))


# ------------------------------------------------------------------ programs written against the DSL
def rms_norm_program(M, N, blk_m, dtype="bfloat16", eps=1e-12):
    @T.prim_func
    def main_kernel_inner(A: T.Tensor((M, N), dtype), B: T.Tensor((M, N), dtype)):
        inv_n = T.float32(1.0 / N)
        with T.Kernel(T.ceildiv(M, blk_m), is_cpu=True) as (bx,):
            a16 = T.alloc_shared((blk_m, N), dtype)
            a32 = T.alloc_shared((blk_m, N), "float32")
            sq = T.alloc_shared((blk_m, N), "float32")
            acc = T.alloc_shared((blk_m, 1), "float32")
            T.ppl_copy(A[bx * blk_m, 0], a16)
            T.ppl_copy(a16, a32)
            T.ppl_mul(sq, a32, a32)
            T.ppl_reduce_sum(sq, acc, dim=1)
            T.ppl_mul_C(acc, acc, inv_n)
            T.ppl_add_C(acc, acc, T.float32(eps))
            T.ppl_rsqrt(acc, acc)
            T.ppl_mul(a32, a32, acc)
            T.ppl_copy(a32, a16)
            T.ppl_copy(a16, B[bx * blk_m, 0])
    return main_kernel_inner


def matmul_program(M, N, K, bm, bn, bk, dtype="float16", trans_b=False):
    b_shape = (N, K) if trans_b else (K, N)

    @T.prim_func
    def main_kernel_inner(A: T.Tensor((M, K), dtype), B: T.Tensor(b_shape, dtype), C: T.Tensor((M, N), dtype)):
        with T.Kernel(T.ceildiv(N, bn), T.ceildiv(M, bm), is_cpu=True) as (bx, by):
            a_t = T.alloc_shared((bm, bk), dtype)
            b_t = T.alloc_shared((bn, bk) if trans_b else (bk, bn), dtype)
            c_t = T.alloc_shared((bm, bn), "float32")
            c_o = T.alloc_shared((bm, bn), dtype)
            T.ppl_fill(c_t, T.float32(0))
            for k in T.Pipelined(T.ceildiv(K, bk), num_stages=1):
                T.ppl_copy(A[by * bm, k * bk], a_t)
                if trans_b:
                    T.ppl_copy(B[bx * bn, k * bk], b_t)
                else:
                    T.ppl_copy(B[k * bk, bx * bn], b_t)
                T.ppl_gemm(a_t, b_t, c_t, transpose_B=trans_b)
            T.ppl_copy(c_t, c_o)
            T.ppl_copy(c_o, C[by * bm, bx * bn])
    return main_kernel_inner


def mlp_program(rows, hidden, inter, block_rows, block_h=None, block_i=None, dtype="bfloat16"):
    """Gated MLP written with the tile ops in the order of the reference's program: gate GEMM, SiLU
    in fp32 (g / (exp(-g) + 1)), up GEMM, product, down GEMM; weights are (out_features, in_features)."""
    bh, bi = block_h or hidden, block_i or inter

    @T.prim_func
    def main_kernel_inner(Y: T.Tensor((rows, hidden), dtype), X: T.Tensor((rows, hidden), dtype),
                          Wg: T.Tensor((inter, hidden), dtype), Wu: T.Tensor((inter, hidden), dtype),
                          Wd: T.Tensor((hidden, inter), dtype)):
        with T.Kernel(T.ceildiv(rows, block_rows), T.ceildiv(hidden, bh), T.ceildiv(inter, bi), is_cpu=True) as (bx, by, bz):
            x_t = T.alloc_shared((block_rows, bh), dtype)
            wg_t = T.alloc_shared((bi, bh), dtype)
            wu_t = T.alloc_shared((bi, bh), dtype)
            wd_t = T.alloc_shared((bh, bi), dtype)
            gate16 = T.alloc_shared((block_rows, bi), dtype)
            up16 = T.alloc_shared((block_rows, bi), dtype)
            act16 = T.alloc_shared((block_rows, bi), dtype)
            y16 = T.alloc_shared((block_rows, bh), dtype)
            gate = T.alloc_shared((block_rows, bi), "float32")
            up = T.alloc_shared((block_rows, bi), "float32")
            neg = T.alloc_shared((block_rows, bi), "float32")
            one = T.alloc_shared((block_rows, bi), "float32")
            den = T.alloc_shared((block_rows, bi), "float32")
            silu = T.alloc_shared((block_rows, bi), "float32")
            act = T.alloc_shared((block_rows, bi), "float32")
            w0 = T.alloc_shared((block_rows, bi), "float32")
            w1 = T.alloc_shared((block_rows, bi), "float32")
            coeff = T.alloc_shared((64, 32), "float32")
            table = T.alloc_shared((64, 192), "float32")
            T.ppl_fill(one, T.float32(1.0))
            T.ppl_copy(X[bx * block_rows:(bx + 1) * block_rows, by * bh:(by + 1) * bh], x_t)
            T.ppl_copy(Wg[bz * bi:(bz + 1) * bi, by * bh:(by + 1) * bh], wg_t)
            T.ppl_copy(Wu[bz * bi:(bz + 1) * bi, by * bh:(by + 1) * bh], wu_t)
            T.ppl_copy(Wd[by * bh:(by + 1) * bh, bz * bi:(bz + 1) * bi], wd_t)
            T.ppl_gemm(x_t, wg_t, gate16, transpose_B=True)
            T.ppl_copy(gate16, gate)
            T.ppl_mul_C(neg, gate, T.float32(-1.0))
            T.ppl_exp2(neg, w0, w1, coeff, table)
            T.ppl_add(den, neg, one)
            T.ppl_div(silu, gate, den)
            T.ppl_gemm(x_t, wu_t, up16, transpose_B=True)
            T.ppl_copy(up16, up)
            T.ppl_mul(act, silu, up)
            T.ppl_copy(act, act16)
            T.ppl_gemm(act16, wd_t, y16, transpose_B=True)
            T.ppl_copy(y16, Y[bx * block_rows:(bx + 1) * block_rows, by * bh:(by + 1) * bh])
    return main_kernel_inner


def rms_norm_program_f32(M, N, blk_m, eps=1e-12):
    """The float32 form: no casting copies, the tiles are loaded and stored directly."""
    @T.prim_func
    def main_kernel_inner(A: T.Tensor((M, N), "float32"), B: T.Tensor((M, N), "float32")):
        with T.Kernel(T.ceildiv(M, blk_m), is_cpu=True) as (bx,):
            x = T.alloc_shared((blk_m, N), "float32")
            sq = T.alloc_shared((blk_m, N), "float32")
            ms = T.alloc_shared((blk_m, 1), "float32")
            T.ppl_copy(A[bx * blk_m, 0], x)
            T.ppl_mul(sq, x, x)
            T.ppl_reduce_sum(sq, ms, dim=1)
            T.ppl_mul_C(ms, ms, T.float32(1.0 / N))
            T.ppl_add_C(ms, ms, T.float32(eps))
            T.ppl_rsqrt(ms, ms)
            T.ppl_mul(x, x, ms)
            T.ppl_copy(x, B[bx * blk_m, 0])
    return main_kernel_inner


def swiglu_program_f32(C, W, bc, bw):
    @T.prim_func
    def main_kernel_inner(Out: T.Tensor((C, W), "float32"), G: T.Tensor((C, W), "float32"), U: T.Tensor((C, W), "float32")):
        with T.Kernel(T.ceildiv(C, bc), T.ceildiv(W, bw), is_cpu=True) as (bx, by):
            g = T.alloc_shared((bc, bw), "float32")
            u = T.alloc_shared((bc, bw), "float32")
            neg = T.alloc_shared((bc, bw), "float32")
            one = T.alloc_shared((bc, bw), "float32")
            den = T.alloc_shared((bc, bw), "float32")
            silu = T.alloc_shared((bc, bw), "float32")
            out = T.alloc_shared((bc, bw), "float32")
            T.ppl_fill(one, T.float32(1.0))
            T.ppl_copy(G[bx * bc, by * bw], g)
            T.ppl_copy(U[bx * bc, by * bw], u)
            T.ppl_mul_C(neg, g, T.float32(-1.0))
            T.ppl_exp2(neg, out, out, out, out)
            T.ppl_add(den, neg, one)
            T.ppl_div(silu, g, den)
            T.ppl_mul(out, u, silu)
            T.ppl_copy(out, Out[bx * bc, by * bw])
    return main_kernel_inner


def topk_program(length, K, descended=True):
    @T.prim_func
    def main_kernel_inner(Input: T.Tensor((length,), "float32"), Output: T.Tensor((length,), "float32"),
                          Indices: T.Tensor((length,), "int32")):
        with T.Kernel(1, 1, is_cpu=True) as (bx, by):
            T.ppl_topk(Output, Indices, Input, K, 1 if descended else 0, length)
    return main_kernel_inner


# ------------------------------------------------------------------ tracing
def test_trace_records_the_ppl_op_stream():
    f = rms_norm_program(128, 128, 32)
    assert [o.name for o in f.ops] == ["ppl.copy", "ppl.copy", "ppl.mul", "ppl.reduce_sum", "ppl.mul_C",
                                       "ppl.add_C", "ppl.rsqrt", "ppl.mul", "ppl.copy", "ppl.copy"]
    assert f.grid == (4,) and len(f.params) == 2 and f.params[0].shape == (128, 128)
    load = f.ops[0]
    src, dst = load.args
    assert src.buffer is f.params[0] and src.extents == (32, 128)       # extents merged from the tile
    assert repr(src.starts[0]) == "(bx * 32)" and src.starts[1] == 0
    assert "ppl.rsqrt" in f.script()


def test_trace_loops_slices_and_macros():
    shape = [2, 64, 4, 16]

    @T.macro
    def load(K, tile, k, by, bz):
        T.copy(K[bz, k * 8:(k + 1) * 8, by, :], tile)

    @T.prim_func
    def prog(K: T.Tensor(shape, "bfloat16"), O: T.Tensor(shape, "bfloat16")):
        with T.Kernel(8, 4, 2, is_cpu=True) as (bx, by, bz):
            tile = T.alloc_shared([8, 16], "bfloat16")
            n = T.min(T.ceildiv(64, 8), T.ceildiv((bx + 1) * 8, 8))
            for k in T.Pipelined(n, num_stages=2):
                load(K, tile, k, by, bz)
            T.copy(tile, O[bz, bx * 8:(bx + 1) * 8, by, :])

    names = [o.name for o in prog.ops]
    assert names == ["loop.begin", "ppl.copy", "loop.end", "ppl.copy"]
    region = prog.ops[1].args[0]
    assert region.extents == (1, 8, 1, 16)                 # point indices select one element
    loop = prog.ops[0]
    assert loop.attrs["num_stages"] == 2 and repr(loop.args[1]).startswith("min(")
    bx, by, bz = prog.block_vars
    assert loop.args[1].evaluate({bx: 2}) == 3 and loop.args[1].evaluate({bx: 7}) == 8


def test_intrinsic_argument_checks():
    with pytest.raises(AssertionError, match="gemm K shape check failed"):
        @T.prim_func
        def bad(A: T.Tensor((8, 8), "float16")):
            with T.Kernel(1, is_cpu=True) as (bx,):
                a = T.alloc_shared((8, 4), "float16")
                b = T.alloc_shared((8, 8), "float16")
                c = T.alloc_shared((8, 8), "float32")
                T.ppl_gemm(a, b, c)
    with pytest.raises(AssertionError, match="dim=1"):
        @T.prim_func
        def bad2(A: T.Tensor((8, 8), "float16")):
            with T.Kernel(1, is_cpu=True) as (bx,):
                a = T.alloc_shared((8, 8), "float16")
                o = T.alloc_shared((8, 1), "float16")
                T.ppl_reduce_sum(a, o, dim=0)
    with pytest.raises(RuntimeError, match="inside a @T.prim_func"):
        T.alloc_shared((4, 4), "float32")


# ------------------------------------------------------------------ matching
def test_bind_rmsnorm_extracts_eps_and_checks_the_mean_scale():
    b = bind(rms_norm_program(128, 128, 32, eps=1e-6))
    assert b.program == "rmsnorm" and b.entry_point == "tl_b200_rmsnorm"
    assert b.facts["eps"] == pytest.approx(1e-6) and b.facts["rows"] == 128

    @T.prim_func
    def wrong_scale(A: T.Tensor((64, 64), "bfloat16"), B: T.Tensor((64, 64), "bfloat16")):
        with T.Kernel(2, is_cpu=True) as (bx,):
            a16 = T.alloc_shared((32, 64), "bfloat16")
            a32 = T.alloc_shared((32, 64), "float32")
            sq = T.alloc_shared((32, 64), "float32")
            acc = T.alloc_shared((32, 1), "float32")
            T.ppl_copy(A[bx * 32, 0], a16)
            T.ppl_copy(a16, a32)
            T.ppl_mul(sq, a32, a32)
            T.ppl_reduce_sum(sq, acc, dim=1)
            T.ppl_mul_C(acc, acc, T.float32(0.5))
            T.ppl_add_C(acc, acc, T.float32(1e-6))
            T.ppl_rsqrt(acc, acc)
            T.ppl_mul(a32, a32, acc)
            T.ppl_copy(a32, a16)
            T.ppl_copy(a16, B[bx * 32, 0])
    with pytest.raises(UnsupportedProgram, match="not 1/N"):
        bind(wrong_scale)


def test_bind_matmul_both_layouts_and_tiling_rule():
    b = bind(matmul_program(64, 64, 64, 32, 32, 32))
    assert b.program == "matmul" and b.facts["transpose_B"] is False and b.facts["K"] == 64
    b = bind(matmul_program(128, 256, 64, 32, 64, 64, dtype="bfloat16", trans_b=True))
    assert b.facts["transpose_B"] is True and b.facts["N"] == 256
    # C = A B^T overwrites C per K iteration in the reference (codegen_ppl.cc:1276-1279): with more than
    # one K tile the program is not the full product, and the tile-op executor takes it
    assert bind(matmul_program(128, 256, 64, 32, 64, 32, dtype="bfloat16", trans_b=True)).program == "generic"
    with pytest.raises(UnsupportedProgram, match="no tail masking"):
        bind(matmul_program(100, 64, 64, 32, 32, 32))


def generic_program(M=64, N=96, bm=32, bn=32, dtype="bfloat16"):
    """Not one of the fused programs: out = exp(x) * rsqrt(mean(x * x) + 1) + 0.5, row block by row
    block (a block spans all columns), fp32 math on a 16-bit tensor."""
    @T.prim_func
    def main_kernel_inner(X: T.Tensor((M, N), dtype), Y: T.Tensor((M, N), dtype)):
        with T.Kernel(T.ceildiv(M, bm), is_cpu=True) as (bx,):
            x16 = T.alloc_shared((bm, N), dtype)
            x = T.alloc_shared((bm, N), "float32")
            sq = T.alloc_shared((bm, N), "float32")
            ss = T.alloc_shared((bm, 1), "float32")
            y = T.alloc_shared((bm, N), "float32")
            y16 = T.alloc_shared((bm, N), dtype)
            T.ppl_copy(X[bx * bm, 0], x16)
            T.ppl_copy(x16, x)
            T.ppl_mul(sq, x, x)
            T.ppl_reduce_sum(sq, ss, dim=1)
            T.ppl_mul_C(ss, ss, T.float32(1.0 / N))
            T.ppl_add_C(ss, ss, T.float32(1.0))
            T.ppl_rsqrt(ss, ss)
            T.ppl_copy(x, y)
            T.ppl_exp2(y, sq, sq, sq, sq)
            T.ppl_mul(y, y, ss)
            T.ppl_add_C(y, y, T.float32(0.5))
            T.ppl_copy(y, y16)
            T.ppl_copy(y16, Y[bx * bm, 0])
    return main_kernel_inner


def test_float32_program_forms_bind_to_the_fused_kernels():
    assert bind(rms_norm_program_f32(64, 128, 32, eps=1e-6)).facts == dict(rows=64, cols=128, eps=1e-6, dtype="float32", weight=False)
    assert bind(swiglu_program_f32(64, 128, 32, 64)).program == "swiglu"


def test_unmatched_program_binds_to_the_generic_executor():
    bound = bind(generic_program())
    assert bound.program == "generic" and bound.facts["grid"] == [2]


def test_program_the_executor_cannot_run_is_rejected_with_its_listing():
    @T.prim_func
    def odd(A: T.Tensor((8, 8), "float32"), B: T.Tensor((8, 8), "float32")):
        with T.Kernel(1, is_cpu=True) as (bx,):
            t = T.alloc_shared((2, 4, 8), "float32")
            T.ppl_fill(t, T.float32(0))
            T.ppl_rsqrt(t, t)
    with pytest.raises(UnsupportedProgram, match="has rank 3.*no CPU fallback"):
        tilelang.compile(odd, out_idx=-1, target="b200")


# ------------------------------------------------------------------ compile / adapter
def test_compile_signature_and_out_idx_legalisation():
    k = tilelang.compile(rms_norm_program(128, 128, 32), out_idx=-1, target="b200")
    assert k.adapter.result_idx == [1] and [p.shape for p in k.params] == [[128, 128], [128, 128]]
    assert k.params[0].dtype == torch.bfloat16
    assert "tl_b200_rmsnorm" in k.get_kernel_source()
    k2 = tilelang.compile(topk_program(1024, 8), out_idx=[1, 2], target="b200", mode="cmodel")
    assert k2.adapter.result_idx == [1, 2]
    with pytest.raises(ValueError):
        tilelang.compile(topk_program(64, 8), out_idx=[5], target="b200")
    with pytest.raises(AssertionError, match="not supported"):
        tilelang.compile(topk_program(64, 8), out_idx=[1, 2], target="tpu")
    with pytest.raises(AssertionError, match="Invalid mode"):
        tilelang.compile(topk_program(64, 8), out_idx=[1, 2], target="b200", mode="fpga")


def test_tpu_target_alias_is_opt_in(monkeypatch):
    monkeypatch.setenv("TL_B200_ACCEPT_TPU_TARGET", "1")
    k = tilelang.compile(topk_program(128, 4), out_idx=[1, 2], target="tpu")
    assert k.target == "b200"


def test_adapter_validates_arguments_before_launch():
    k = tilelang.compile(rms_norm_program(128, 128, 32), out_idx=-1, target="b200")
    a = torch.zeros(128, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="Expected 2 inputs"):
        k(a)
    with pytest.raises(ValueError, match="dtype"):
        k(a, a.float())
    with pytest.raises(ValueError, match="shape"):
        k(a, torch.zeros(64, 128, dtype=torch.bfloat16))


def test_compile_is_cached_per_program_object():
    f = topk_program(256, 4)
    assert tilelang.compile(f, out_idx=[1, 2], target="b200") is tilelang.compile(f, out_idx=[1, 2], target="b200")


def test_mlp_program_binds_only_in_its_single_tile_form():
    bound = bind(mlp_program(128, 256, 512, 64))
    assert bound.program == "mlp" and bound.facts == dict(M=128, hidden=256, intermediate=512, dtype="bfloat16")
    # tiles along the hidden or intermediate dimension overwrite each other in the program (no accumulator):
    # not the MLP any more; the generic executor runs it tile by tile as the reference would
    assert bind(mlp_program(16, 16, 16, 8, 8, 8)).program == "generic"
    with pytest.raises(UnsupportedProgram, match="no tail masking"):
        bind(mlp_program(100, 256, 512, 64))


# ------------------------------------------------------------------ the reference's own demo programs
def _reference_builder(rel_path: str, func_name: str):
    """Lift one program-builder function out of a reference demo script (the script itself builds
    a TPU kernel at import time, so it cannot be imported) and bind it to this package's T."""
    src = (REFERENCE / rel_path).read_text()
    tree = ast.parse(src)
    nodes = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == func_name]
    assert nodes, f"{func_name} not found in {rel_path}"
    env = {"tilelang": tilelang, "T": T, "torch": torch}
    T.copy = T.ppl_copy            # the demos do this at module level
    exec(compile(ast.Module(body=nodes, type_ignores=[]), str(REFERENCE / rel_path), "exec"), env)
    return env[func_name]


needs_reference = pytest.mark.skipif(not REFERENCE.exists(), reason="reference tree not present")

DEMOS = [
    ("tpu_demo/matmul/tpu_test_matmul_fp16.py", "matmul", (64, 64, 64, 32, 32, 32), "matmul"),
    ("tpu_demo/matmul/tpu_test_matmul_bf16.py", "matmul", (64, 64, 64, 32, 32, 32), "matmul"),
    ("tpu_demo/rms_norm/rms_norm_bf16.py", "rms_norm", (128, 128, 32), "rmsnorm"),
    ("tpu_demo/rms_norm/rmsnorm_splitk_bf16.py", "rms_norm_splitk", (512, 512, 32, 32), "rmsnorm_splitk"),
    ("tpu_demo/tpu_test_rope_bf16.py", "rope", (64, 16, 128, 64), "rope"),
    ("tpu_demo/tpu_test_swiglu_bf16.py", "swi_glu", (32, 32, 64, 64), "swiglu"),
    ("tpu_demo/tpu_test_reduce_sum.py", "reduce_sum", (64, 64, 32, 64), "reduce_sum"),
    ("tpu_demo/tpu_test_reduce_max.py", "reduce_max", (64, 64, 32, 64), "reduce_max"),
    ("tpu_demo/tpu_test_topk_fp32.py", "topk_kernel", (1024, 8), "topk"),
    ("tpu_demo/tpu_test_gather_fp32.py", "gather_kernel", (128, 64, 8), "gather"),
    ("tpu_demo/tpu_test_sigmoid_fp32.py", "sigmoid_kernel", (32, 32, 1024, 1024), "sigmoid"),
    ("tpu_demo/ppl/mlp/mlp_bf16.py", "deepseek_v3_mlp_bf16", (64, 256, 512, 128, 256, 512), "mlp"),
    ("tpu_demo/ppl/mlp/mlp_bf16.py", "deepseek_v3_mlp_bf16", (8, 8, 8, 16, 16, 16), "generic"),
    ("tpu_demo/ppl/mlp/mlp_fp32.py", "deepseek_v3_mlp_fp32", (8, 8, 8, 16, 16, 16), "generic"),
    ("tpu_demo/rms_norm/rmsnorm_fp32.py", "rms_norm", (128, 128, 32), "rmsnorm"),
    ("tpu_demo/rms_norm/rmsnorm_splitk_fp32.py", "rms_norm_splitk", (512, 512, 32, 32), "rmsnorm_splitk"),
    ("tpu_demo/tpu_test_swiglu_fp32.py", "swi_glu", (32, 32, 64, 64), "swiglu"),
    ("tpu_demo/matmul/tpu_test_matmul_fp32.py", "matmul", (64, 64, 64, 32, 32, 32), "generic"),
    ("tpu_demo/ppl/test/elementwise_c.py", "elementwise_c", (16, 4, 4, 2, "float32"), "generic"),
    ("tpu_demo/ppl/test/mul_N_1.py", "rms_norm", (128, 128, 32, "float32"), "generic"),
    ("tpu_demo/ppl/elementwise_add_kernel/elementwise_add.py", "elementwise_add",
     (128, 128, 32, 32, "float32", "float32", 128), "elementwise_add"),
]


@needs_reference
@pytest.mark.parametrize("path,builder,args,program", DEMOS, ids=[d[3] + "_" + Path(d[0]).stem for d in DEMOS])
def test_unmodified_reference_demo_programs_bind(path, builder, args, program):
    func = _reference_builder(path, builder)(*args)
    assert bind(func).program == program


@needs_reference
@pytest.mark.parametrize("causal", [False, True])
def test_reference_flash_attention_program_binds(causal):
    build = _reference_builder("tpu_demo/flashattn/tpu_test_flashattn_bf16.py", "flashattn")
    func = build(batch=1, heads=2, seq_len=256, dim=64, is_causal=causal)(64, 64, 1, 128)
    b = bind(func)
    assert b.program == "flash_attention_fwd"
    assert b.facts["causal"] == ("block" if causal else "none")
    assert b.facts["scale"] == pytest.approx(64 ** -0.5) and b.facts["block_M"] == 64


@needs_reference
def test_reference_mla_decode_program_binds():
    build = _reference_builder("tpu_demo/ppl/deepseek_mla/mla_decode.py", "flashattn")
    b = bind(build(4, 8, 1, 512, 32, 4, 4, 4))
    assert b.program == "mla_decode" and b.facts["pe_dim"] == 4 and b.facts["seqlen_kv"] == 512
    assert b.facts["scale"] == pytest.approx(36 ** -0.5)


# ------------------------------------------------------------------ programs of the benchmark configurations
def test_benchmark_programs_bind_to_the_fused_kernels():
    from tilelang import programs as P
    b = bind(P.rmsnorm(8192, 4096, eps=1e-6))
    assert b.program == "rmsnorm" and b.facts["weight"] is True and b.facts["eps"] == pytest.approx(1e-6)
    assert bind(P.rmsnorm(128, 128, weight=False)).facts["weight"] is False
    b = bind(P.rope(8192, 32, 128))
    assert b.program == "rope" and b.facts["shape"] == [8192, 32, 128] and b.facts["table"] == [8192, 128]
    assert bind(P.swiglu(8192, 14336)).program == "swiglu"
    assert bind(P.gemm_fp8_blockscale(256, 384, 512)).entry_point == "tl_b200_gemm_fp8_blockscale"
    k = tilelang.compile(P.mla_decode_paged(4, 128, 576, 512, 40, 64, 11), out_idx=-1, target="b200")
    assert [list(p.shape) for p in k.params][-1] == [4, 1, 128, 512] and k.adapter.result_idx == [5]
    assert k.params[1].dtype == torch.float8_e4m3fn


def test_weighted_rmsnorm_with_other_dataflow_is_not_bound_to_the_fused_kernel():
    """Same op order as the weighted RMSNorm, but the weight multiplies the SQUARES: not RMSNorm."""
    M, N, bm = 64, 128, 32

    @T.prim_func
    def not_rmsnorm(A: T.Tensor((M, N), "bfloat16"), W: T.Tensor((1, N), "bfloat16"), B: T.Tensor((M, N), "bfloat16")):
        with T.Kernel(M // bm, is_cpu=True) as (bx,):
            a16 = T.alloc_shared((bm, N), "bfloat16")
            a32 = T.alloc_shared((bm, N), "float32")
            sq = T.alloc_shared((bm, N), "float32")
            acc = T.alloc_shared((bm, 1), "float32")
            w16 = T.alloc_shared((1, N), "bfloat16")
            w32 = T.alloc_shared((1, N), "float32")
            T.ppl_copy(A[bx * bm, 0], a16)
            T.ppl_copy(a16, a32)
            T.ppl_mul(sq, a32, a32)
            T.ppl_copy(W[0, 0], w16)
            T.ppl_copy(w16, w32)
            T.ppl_mul(sq, sq, w32)
            T.ppl_reduce_sum(sq, acc, dim=1)
            T.ppl_mul_C(acc, acc, T.float32(1.0 / N))
            T.ppl_add_C(acc, acc, T.float32(1e-6))
            T.ppl_rsqrt(acc, acc)
            T.ppl_mul(a32, a32, acc)
            T.ppl_copy(a32, a16)
            T.ppl_copy(a16, B[bx * bm, 0])
    assert bind(not_rmsnorm).program == "generic"


def test_rope_program_with_mismatched_token_blocks_is_rejected():
    tokens, heads, width, bt = 128, 4, 64, 32

    @T.prim_func
    def shifted(X: T.Tensor((tokens, heads, width), "bfloat16"), Cos: T.Tensor((tokens, width), "bfloat16"),
                Sin: T.Tensor((tokens, width), "bfloat16"), Out: T.Tensor((tokens, heads, width), "bfloat16")):
        with T.Kernel(tokens // bt, heads, is_cpu=True) as (bx, by):
            x, c, s, xc, xs, nx, nxs, o = (T.alloc_shared((bt, width), "bfloat16") for _ in range(8))
            T.ppl_copy(X[bx * bt:(bx + 1) * bt, by, 0:width], x)
            T.ppl_copy(Cos[0, 0], c)                      # always the first token block: not the per-token table
            T.ppl_copy(Sin[bx * bt, 0], s)
            T.ppl_mul(xc, x, c)
            T.ppl_mul(xs, x, s)
            T.ppl_mul_C(nx, x, -1.0)
            T.ppl_mul(nxs, nx, s)
            T.ppl_rope_add(o, xc, nxs, xc, xs)
            T.ppl_copy(o, Out[bx * bt:(bx + 1) * bt, by, 0:width])
    with pytest.raises(UnsupportedProgram, match="same token block"):
        bind(shifted)


# ------------------------------------------------------------------ kernel cache and tile table
def test_cache_is_keyed_by_program_content_and_persists_its_record(tmp_path, monkeypatch):
    from tilelang import cache
    monkeypatch.setenv("TILELANG_B200_CACHE_DIR", str(tmp_path))
    cache.clear_cache()
    k1 = tilelang.compile(rms_norm_program(64, 128, 32, eps=1e-6), out_idx=-1, target="b200")
    k2 = tilelang.compile(rms_norm_program(64, 128, 32, eps=1e-6), out_idx=-1, target="b200")     # a second, equal program object
    assert k1 is k2
    k3 = tilelang.compile(rms_norm_program(64, 128, 32, eps=1e-5), out_idx=-1, target="b200")
    assert k3 is not k1 and k3.cache_key != k1.cache_key
    rec = cache.load_record(k1.cache_key)
    assert rec["program"] == "rmsnorm" and rec["entry_point"] == "tl_b200_rmsnorm" and rec["facts"]["eps"] == pytest.approx(1e-6)
    # a record that disagrees with today's binding (e.g. written by an older library) is reported and replaced
    (tmp_path / "programs" / f"{k1.cache_key}.json").write_text('{"program": "generic", "entry_point": "x", "facts": {}}')
    cache.clear_cache()
    with pytest.warns(UserWarning, match="bound to"):
        tilelang.compile(rms_norm_program(64, 128, 32, eps=1e-6), out_idx=-1, target="b200")
    assert cache.load_record(k1.cache_key)["program"] == "rmsnorm"
    cache.clear_cache()


def test_tile_table_round_trip(tmp_path, monkeypatch):
    from tilelang import cache
    monkeypatch.setenv("TILELANG_B200_CACHE_DIR", str(tmp_path))
    cache.clear_cache(disk=True)
    assert cache.tile_choice("gemm", m=128, n=256, k=64, dtype="torch.bfloat16", transpose_b=False) is None
    cache.set_tile_choice("gemm", {"tile_n": 128, "ms": 0.5}, m=128, n=256, k=64, dtype="torch.bfloat16", transpose_b=False)
    cache.clear_cache()
    cache._tile_table = None                       # a new process reads the file
    assert cache.tile_choice("gemm", m=128, n=256, k=64, dtype="torch.bfloat16", transpose_b=False)["tile_n"] == 128
    cache.clear_cache(disk=True)


def test_autotuner_interface_rejects_unrunnable_configs_on_cpu():
    from tilelang.autotuner import AutoTuner, product_configs
    cfgs = product_configs(blk_m=[32, 48])
    assert cfgs == [{"blk_m": 32}, {"blk_m": 48}]
    tuner = AutoTuner.from_kernel(lambda blk_m: rms_norm_program(64, 128, blk_m), cfgs).set_compile_args(out_idx=-1)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no configuration"):     # timing needs the GPU: there is no CPU path
            tuner.run(warmup=1, rep=1)


def test_matmul_with_other_addressing_goes_to_the_executor():
    """Same op order as the matmul program, but every block reads the FIRST row block of A: not C = A B."""
    M = N = K = 64

    @T.prim_func
    def not_matmul(A: T.Tensor((M, K), "float16"), B: T.Tensor((K, N), "float16"), C: T.Tensor((M, N), "float16")):
        with T.Kernel(N // 32, M // 32, is_cpu=True) as (bx, by):
            a_t = T.alloc_shared((32, 32), "float16")
            b_t = T.alloc_shared((32, 32), "float16")
            c_t = T.alloc_shared((32, 32), "float32")
            c_o = T.alloc_shared((32, 32), "float16")
            T.ppl_fill(c_t, T.float32(0))
            for k in T.Pipelined(K // 32, num_stages=1):
                T.ppl_copy(A[0, k * 32], a_t)
                T.ppl_copy(B[k * 32, bx * 32], b_t)
                T.ppl_gemm(a_t, b_t, c_t)
            T.ppl_copy(c_t, c_o)
            T.ppl_copy(c_o, C[by * 32, bx * 32])
    assert bind(not_matmul).program == "generic"
    assert bind(matmul_program(M, N, K, 32, 32, 32)).program == "matmul"
