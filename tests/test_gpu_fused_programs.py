"""Row-local tile programs as ONE kernel launch (engine/fuser.py -> tl_b200_tile_program): same answers as the
op-by-op executor and as the oracle, for 2-D tensors and for windows of rank-3 / rank-4 tensors."""
import pytest
import torch

import oracle.ops as O
import tilelang
import tilelang.language as T
from test_frontend import generic_program, rms_norm_program, rms_norm_program_f32, swiglu_program_f32
from tilelang import ops, programs as P
from tilelang.engine import bind, fuser, interpreter

pytestmark = pytest.mark.gpu
BF, HF, F32 = torch.bfloat16, torch.float16, torch.float32
TOL16 = dict(atol=2e-2, rtol=2e-2)


def gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def run_fused(func, tensors, dev):
    """The program as ONE launch: by the kernel generated for it and by the interpreter kernel, which must agree bit
    for bit (the same instruction list, the same arithmetic)."""
    run = fuser.build(func)
    assert run is not None, fuser.build.last_reason
    assert run.generated, fuser.build.last_reason             # NVRTC is part of the CUDA toolkit of this image
    d = [t.to(dev) for t in tensors]
    before = ops.launch_count()
    assert run(*d) == 0
    torch.cuda.synchronize()
    assert ops.launch_count() - before == 1                   # the whole program is one launch
    di = [t.to(dev) for t in tensors]
    before = ops.launch_count()
    assert run.interpreted(*di) == 0
    torch.cuda.synchronize()
    assert ops.launch_count() - before == 1
    for a, b in zip(d, di):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    return [t.cpu() for t in d]


def run_by_op(func, tensors, dev):
    d = [t.to(dev) for t in tensors]
    assert interpreter.build(func)(*d) == 0
    torch.cuda.synchronize()
    return [t.cpu() for t in d]


@pytest.mark.parametrize("M,N,bm", [(64, 96, 32), (64, 100, 16), (256, 4096, 32), (32, 8192, 8), (48, 520, 16)])
def test_generic_program_fused_equals_op_by_op(cuda_device, M, N, bm):
    func = generic_program(M, N, bm)
    bound = bind(func)
    assert bound.program == "generic" and bound.facts["fused"] is True
    x = torch.randn(M, N, generator=gen(M + N)).to(BF)
    y_f = run_fused(func, [x, torch.zeros_like(x)], cuda_device)[1]
    y_o = run_by_op(func, [x, torch.zeros_like(x)], cuda_device)[1]
    xf = x.float()
    ref = (torch.exp(xf) * torch.rsqrt((xf * xf).sum(1, keepdim=True) * (1.0 / N) + 1.0) + 0.5).to(BF)
    assert torch.allclose(y_f.float(), ref.float(), **TOL16)
    assert torch.allclose(y_f.float(), y_o.float(), atol=1e-2, rtol=1e-2)      # row sums are taken in another order


def test_rmsnorm_programs_through_the_fused_path(cuda_device):
    x = torch.randn(128, 256, generator=gen(2)).to(BF)
    y = run_fused(rms_norm_program(128, 256, 32), [x, torch.zeros_like(x)], cuda_device)[1]
    assert torch.allclose(y.float(), O.rmsnorm(x, eps=1e-12).float(), **TOL16)
    x32 = torch.randn(64, 128, generator=gen(3))
    y32 = run_fused(rms_norm_program_f32(64, 128, 32, eps=1e-6), [x32, torch.zeros_like(x32)], cuda_device)[1]
    assert torch.allclose(y32, O.rmsnorm(x32, eps=1e-6), atol=1e-5, rtol=1e-5)
    # the weighted form of the benchmark: a (1, N) tile broadcast down the rows
    w = (1 + 0.02 * torch.randn(1, 4096, generator=gen(4))).to(BF)
    xl = torch.randn(64, 4096, generator=gen(5)).to(BF)
    yl = run_fused(P.rmsnorm(64, 4096, eps=1e-6), [xl, w, torch.zeros_like(xl)], cuda_device)[2]
    assert torch.allclose(yl.float(), O.rmsnorm(xl, w.view(-1), eps=1e-6).float(), **TOL16)


def test_loops_are_unrolled_running_maximum(cuda_device):
    M, N, bn = 32, 128, 32

    @T.prim_func
    def main_kernel_inner(X: T.Tensor((M, N), "float32"), Y: T.Tensor((M, N), "float32")):
        with T.Kernel(1, is_cpu=True) as (bx,):
            x = T.alloc_shared((M, bn), "float32")
            m = T.alloc_shared((M, 1), "float32")
            T.ppl_fill(m, T.float32(-1e30))
            for k in T.Pipelined(N // bn, num_stages=1):
                T.ppl_copy(X[0:M, k * bn:(k + 1) * bn], x)
                T.ppl_reduce_max(x, m, dim=1, clear=False)
            for k in T.Pipelined(N // bn, num_stages=1):
                T.ppl_copy(X[0:M, k * bn:(k + 1) * bn], x)
                T.ppl_subtract(x, x, m)
                T.ppl_copy(x, Y[0:M, k * bn:(k + 1) * bn])

    x = torch.randn(M, N, generator=gen(6))
    y = run_fused(main_kernel_inner, [x, torch.zeros(M, N)], cuda_device)[1]
    assert torch.equal(y, x - x.max(dim=1, keepdim=True).values)


def test_rope_with_per_token_tables_rank3_is_bit_exact(cuda_device):
    """X (tokens, heads, W) addressed as [t0:t0+bt, head, :]: rows of a window are H*W elements apart."""
    tokens, heads, width = 64, 4, 128
    func = P.rope(tokens, heads, width, blk_t=16)
    g = gen(7)
    x = torch.randn(tokens, heads, width, generator=g).to(BF)
    cos, sin = O.make_rope_cos_sin(tokens, width)
    cos, sin = cos.to(BF), sin.to(BF)
    y = run_fused(func, [x, cos, sin, torch.zeros_like(x)], cuda_device)[3]
    assert torch.equal(y.view(torch.int16), O.rope(x, cos, sin).view(torch.int16))
    y2 = run_by_op(func, [x, cos, sin, torch.zeros_like(x)], cuda_device)[3]
    assert torch.equal(y2.view(torch.int16), y.view(torch.int16))


def softmax_program(B, S, H, D, bm, dtype="bfloat16"):
    """Row softmax over the last dimension of a bshd tensor, one (batch, head, row block) per grid block."""
    @T.prim_func
    def softmax_kernel(X: T.Tensor((B, S, H, D), dtype), Y: T.Tensor((B, S, H, D), dtype)):
        with T.Kernel(T.ceildiv(S, bm), H, B, is_cpu=True) as (bx, by, bz):
            x16 = T.alloc_shared((bm, D), dtype)
            x = T.alloc_shared((bm, D), "float32")
            m = T.alloc_shared((bm, 1), "float32")
            l = T.alloc_shared((bm, 1), "float32")
            work0 = T.alloc_shared((bm, D), "float32")
            work1 = T.alloc_shared((bm, D), "float32")
            coeff = T.alloc_shared((64, 32), "float32")
            table = T.alloc_shared((64, 192), "float32")
            T.ppl_copy(X[bz, bx * bm:(bx + 1) * bm, by, :], x16)
            T.ppl_copy(x16, x)
            T.ppl_reduce_max(x, m, dim=1, clear=True)
            T.ppl_subtract(x, x, m)
            T.ppl_exp2(x, work0, work1, coeff, table)
            T.ppl_reduce_sum(x, l, dim=1)
            T.ppl_div(x, x, l)
            T.ppl_copy(x, x16)
            T.ppl_copy(x16, Y[bz, bx * bm:(bx + 1) * bm, by, :])
    return softmax_kernel


@pytest.mark.parametrize("dtype,tdt", [("bfloat16", BF), ("float16", HF), ("float32", F32)])
def test_softmax_shaped_program_on_a_4d_tensor(cuda_device, dtype, tdt):
    B, S, H, D, bm = 2, 64, 3, 80, 16
    func = softmax_program(B, S, H, D, bm, dtype)
    kernel = tilelang.compile(func, out_idx=-1, target="b200")
    assert kernel.adapter.bound.facts["fused"] is True
    x = (torch.randn(B, S, H, D, generator=gen(8)) * 3).to(tdt)
    y = torch.zeros_like(x)
    assert kernel(x, y) == 0
    ref = torch.softmax(x.float(), dim=-1).to(tdt)
    tol = dict(atol=1e-6, rtol=1e-5) if tdt == F32 else TOL16
    assert torch.allclose(y.float(), ref.float(), **tol)
    y2 = run_by_op(func, [x, torch.zeros_like(x)], cuda_device)[1]           # rank-4 windows in the op-by-op executor too
    assert torch.allclose(y2.float(), ref.float(), **tol)


def test_swiglu_and_elementwise_programs(cuda_device):
    g = gen(9)
    gate, up = torch.randn(64, 128, generator=g), torch.randn(64, 128, generator=g)
    out = run_fused(swiglu_program_f32(64, 128, 32, 64), [torch.zeros(64, 128), gate, up], cuda_device)[0]
    assert torch.allclose(out, O.swiglu(gate, up), atol=1e-5, rtol=1e-5)
    gb, ub = torch.randn(32, 1024, generator=g).to(BF), torch.randn(32, 1024, generator=g).to(BF)
    ob = run_fused(P.swiglu(32, 1024, blk_c=16, blk_w=512), [gb, ub, torch.zeros_like(gb)], cuda_device)[2]
    assert torch.allclose(ob.float(), O.swiglu(gb, ub).float(), **TOL16)


def test_programs_with_a_gemm_are_left_to_the_op_by_op_executor():
    from test_frontend import matmul_program
    assert fuser.build(matmul_program(64, 64, 64, 32, 32, 32, dtype="float32")) is None
    assert "row-local" in fuser.build.last_reason
