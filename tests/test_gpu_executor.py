"""The generic tile-op executor: programs that no matcher knows run op by op on the GPU, and the
programs that do have a fused kernel give the same answers when they are forced through it."""
import pytest
import torch

import oracle.ops as O
import tilelang
from test_frontend import generic_program, matmul_program, mlp_program, rms_norm_program, topk_program
from tilelang.engine import bind, interpreter

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def run_generic(func, tensors, dev):
    d = [t.to(dev) for t in tensors]
    assert interpreter.build(func)(*d) == 0
    torch.cuda.synchronize()
    return [t.cpu() for t in d]


def test_unmatched_program_through_compile(cuda_device):
    M, N = 64, 96
    kernel = tilelang.compile(generic_program(M, N, 32), out_idx=-1, target="b200")
    x = torch.randn(M, N, generator=gen(1)).to(BF)
    y = torch.zeros(M, N, dtype=BF)
    assert kernel(x, y) == 0
    xf = x.float()
    ref = (torch.exp(xf) * torch.rsqrt((xf * xf).sum(1, keepdim=True) * (1.0 / N) + 1.0) + 0.5).to(BF)
    assert torch.allclose(y.float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_rmsnorm_program_same_as_the_fused_kernel(cuda_device):
    func = rms_norm_program(128, 256, 32)
    x = torch.randn(128, 256, generator=gen(2)).to(BF)
    y_gen = run_generic(func, [x, torch.zeros_like(x)], cuda_device)[1]
    y_fused = torch.zeros_like(x).to(cuda_device)
    assert bind(func).run(x.to(cuda_device), y_fused) == 0
    assert torch.allclose(y_gen.float(), y_fused.cpu().float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(y_gen.float(), O.rmsnorm(x, eps=1e-12).float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("trans_b,bk", [(False, 32), (True, 64)])
def test_matmul_program(cuda_device, trans_b, bk):
    """Without transpose_B the tile GEMM accumulates over the K loop; with it the result tile is
    overwritten, so that form is run with a single K block."""
    func = matmul_program(64, 96, 64, 32, 32, bk, dtype="float16", trans_b=trans_b)
    g = gen(3)
    a = torch.randn(64, 64, generator=g).half()
    b = (torch.randn(96, 64, generator=g) if trans_b else torch.randn(64, 96, generator=g)).half()
    c = run_generic(func, [a, b, torch.zeros(64, 96).half()], cuda_device)[2]
    assert torch.allclose(c, O.matmul(a, b, transpose_b=trans_b), atol=1e-2, rtol=1e-2)


def test_mlp_program(cuda_device):
    rows, hidden, inter = 64, 128, 256
    func = mlp_program(rows, hidden, inter, 32)
    g = gen(4)
    x = torch.randn(rows, hidden, generator=g).to(BF)
    wg = (torch.randn(inter, hidden, generator=g) / hidden ** 0.5).to(BF)
    wu = (torch.randn(inter, hidden, generator=g) / hidden ** 0.5).to(BF)
    wd = (torch.randn(hidden, inter, generator=g) / inter ** 0.5).to(BF)
    y = run_generic(func, [torch.zeros(rows, hidden, dtype=BF), x, wg, wu, wd], cuda_device)[0]
    assert torch.allclose(y.float(), O.mlp(x, wg, wu, wd).float(), atol=2e-2, rtol=2e-2)


def test_topk_program(cuda_device):
    func = topk_program(1024, 8)
    x = torch.randn(1024, generator=gen(5))
    _, vals, idx = run_generic(func, [x, torch.zeros(1024), torch.zeros(1024, dtype=torch.int32)], cuda_device)
    ref_v, ref_i = O.topk(x, 8)
    assert torch.equal(idx[:8].long(), ref_i.long()) and torch.equal(vals[:8], ref_v)


def test_running_maximum_and_column_broadcast(cuda_device):
    """reduce_max with clear=False keeps a running maximum across a loop; (M, 1) operands broadcast."""
    import tilelang.language as T
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
    y = run_generic(main_kernel_inner, [x, torch.zeros(M, N)], cuda_device)[1]
    assert torch.equal(y, x - x.max(dim=1, keepdim=True).values)


def test_rope_from_its_terms_is_bit_exact_with_the_fused_kernel(cuda_device):
    """x*cos, x*sin and -(x)*sin rounded to bf16 tiles, assembled by ppl_rope_add: the same rounding
    points as the fused RoPE kernel and the reference's check function."""
    import tilelang.language as T
    from tilelang import ops
    tokens, heads, dim, bt = 32, 4, 64, 8
    rows = tokens * heads

    @T.prim_func
    def main_kernel_inner(X: T.Tensor((rows, dim), "bfloat16"), C: T.Tensor((rows, dim), "bfloat16"),
                          S: T.Tensor((rows, dim), "bfloat16"), Y: T.Tensor((rows, dim), "bfloat16")):
        with T.Kernel(rows // bt, is_cpu=True) as (bx,):
            x = T.alloc_shared((bt, dim), "bfloat16")
            c = T.alloc_shared((bt, dim), "bfloat16")
            s = T.alloc_shared((bt, dim), "bfloat16")
            xc = T.alloc_shared((bt, dim), "bfloat16")
            xs = T.alloc_shared((bt, dim), "bfloat16")
            xn = T.alloc_shared((bt, dim), "bfloat16")
            y = T.alloc_shared((bt, dim), "bfloat16")
            T.ppl_copy(X[bx * bt, 0], x)
            T.ppl_copy(C[bx * bt, 0], c)
            T.ppl_copy(S[bx * bt, 0], s)
            T.ppl_mul(xc, x, c)
            T.ppl_mul(xs, x, s)
            T.ppl_mul_C(xn, x, T.float32(-1.0))
            T.ppl_mul(xn, xn, s)
            T.ppl_rope_add(y, xc, xn, xc, xs)
            T.ppl_copy(y, Y[bx * bt, 0])

    g = gen(7)
    x = torch.randn(rows, dim, generator=g).to(BF)
    cos, sin = O.make_rope_cos_sin(tokens, dim)
    cos_r, sin_r = cos.to(BF).repeat_interleave(heads, dim=0), sin.to(BF).repeat_interleave(heads, dim=0)
    y = run_generic(main_kernel_inner, [x, cos_r, sin_r, torch.zeros_like(x)], cuda_device)[3]
    fused = torch.empty_like(x).to(cuda_device)
    assert ops.rope(x.to(cuda_device), cos.to(BF).to(cuda_device), sin.to(BF).to(cuda_device), fused) == 0
    assert torch.equal(y.view(torch.int16), fused.cpu().view(torch.int16))
    assert torch.equal(y.view(torch.int16), O.rope(x, cos.to(BF), sin.to(BF)).view(torch.int16))
