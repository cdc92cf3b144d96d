"""Parity of the GEMM kernels (tcgen05 path and FMA path) against the oracle, through the C ABI."""
import pytest
import torch

import oracle.ops as O
from conftest import load_golden
from tilelang import ops

pytestmark = pytest.mark.gpu
BF, HF, F32 = torch.bfloat16, torch.float16, torch.float32
TOL16 = dict(atol=2e-2, rtol=2e-2)      # tolerance the benchmark spec states for 16-bit outputs


def gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def run(a, b, out_dtype, transpose_b, dev, tile_n=None):
    m = a.shape[0]
    n = b.shape[0] if transpose_b else b.shape[1]
    c = torch.full((m, n), float("nan"), dtype=out_dtype, device=dev)
    assert ops.gemm(a.to(dev), b.to(dev), c, transpose_b, tile_n=tile_n) == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return c.cpu()


def check(c, ref, scale):
    """|c - ref| <= atol*scale + rtol*|ref| where scale ~ sqrt(K) bounds the accumulated magnitude."""
    err = (c.double() - ref.double()).abs()
    bound = 2e-2 * scale + 2e-2 * ref.double().abs()
    assert (err <= bound).all(), f"max err {err.max().item()} (scale {scale})"


def test_matmul_golden(cuda_device):
    g = load_golden("matmul_fp16", dict(a=HF, b=HF, ref=HF))
    c = run(g["a"], g["b"], HF, False, cuda_device)
    assert torch.allclose(c.float(), g["ref"].float(), atol=1e-2, rtol=1e-2)     # the demo's tolerance
    g = load_golden("matmul_bf16", dict(a=BF, b=BF, ref=BF))
    c = run(g["a"], g["b"], BF, False, cuda_device)
    assert torch.allclose(c.float(), g["ref"].float(), atol=1e-1, rtol=2e-2)


@pytest.mark.parametrize("dtype", [BF, HF])
@pytest.mark.parametrize("transpose_b", [False, True])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 64, 128), (256, 512, 256), (64, 64, 64),
                                   (1024, 1024, 1024), (200, 136, 72), (129, 264, 200), (1, 8, 8),
                                   (384, 1288, 520), (2048, 4096, 512)])
def test_gemm_tensor_core_shapes(cuda_device, dtype, transpose_b, m, n, k):
    g = gen(m * 7 + n * 3 + k)
    a = torch.randn(m, k, generator=g).to(dtype)
    b = (torch.randn(n, k, generator=g) if transpose_b else torch.randn(k, n, generator=g)).to(dtype)
    ref32 = O.matmul(a, b, F32, transpose_b)
    c = run(a, b, dtype, transpose_b, cuda_device)
    assert torch.allclose(c.float(), ref32.to(dtype).float(), **TOL16)          # the stated tolerance
    check(c, ref32, k ** 0.5)
    # identity structure: exact integers survive fp32 accumulation bit-exactly
    c32 = run(a, b, F32, transpose_b, cuda_device)
    assert ((c32.double() - ref32.double()).abs() <= 1e-3 * k ** 0.5 + 1e-4 * ref32.double().abs()).all()


def test_gemm_exact_small_integers(cuda_device):
    # integer-valued inputs make every product and sum exact: results must be bit-identical
    g = gen(11)
    a = torch.randint(-4, 5, (256, 192), generator=g).to(BF)
    for tb in (False, True):
        b = torch.randint(-4, 5, (320, 192) if tb else (192, 320), generator=g).to(BF)
        ref = O.matmul(a, b, F32, tb)
        assert torch.equal(run(a, b, F32, tb, cuda_device), ref)
        assert torch.equal(run(a, b, BF, tb, cuda_device), ref.to(BF))


@pytest.mark.parametrize("dtype", [BF, HF, F32])
@pytest.mark.parametrize("transpose_b", [False, True])
@pytest.mark.parametrize("m,n,k", [(64, 64, 64), (33, 17, 5), (100, 70, 130), (7, 3, 1)])
def test_gemm_fma_path(cuda_device, dtype, transpose_b, m, n, k):
    # odd K / N force the non-TMA kernel for 16-bit types; float32 always uses it
    g = gen(m + n + k)
    a = torch.randn(m, k, generator=g).to(dtype)
    b = (torch.randn(n, k, generator=g) if transpose_b else torch.randn(k, n, generator=g)).to(dtype)
    ref = O.matmul(a, b, F32, transpose_b)
    c = run(a, b, dtype, transpose_b, cuda_device)
    if dtype == F32:
        assert ((c.double() - ref.double()).abs() <= 1e-5 * (a.double().abs() @ (b.double().abs().t() if transpose_b else b.double().abs()))).all()
    else:
        check(c, ref, k ** 0.5)


def test_gemm_anchor_config(cuda_device):
    """fp16 1024^3, N(0,1) inputs from seed 0, fp32 accumulate, fp16 output."""
    g = gen(0)
    a = torch.randn(1024, 1024, generator=g).half()
    b = torch.randn(1024, 1024, generator=g).half()
    ref = O.matmul(a, b)
    c = run(a, b, HF, False, cuda_device)
    assert torch.allclose(c.float(), ref.float(), **TOL16)                       # the stated tolerance: atol = rtol = 2e-2
    check(c, ref.float(), 32.0)


def test_gemm_llama70b_ffn_config(cuda_device):
    """bf16 M8192 K8192 N28672, A and B = 0.05 N(0,1) from seed 2: the oracle on 64 rows spread over every
    128-row tile band, all 28672 columns (so every column shard of every sharding), at the stated tolerance."""
    g = gen(2)
    m, k, n = 8192, 8192, 28672
    a = (torch.randn(m, k, generator=g) * 0.05).to(BF)
    b = (torch.randn(k, n, generator=g) * 0.05).to(BF)
    c = torch.full((m, n), float("nan"), dtype=BF, device=cuda_device)
    assert ops.gemm(a.to(cuda_device), b.to(cuda_device), c) == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    rows = torch.arange(64) * 128 + torch.randint(0, 128, (64,), generator=g)      # one row in each of the 64 row tiles
    ref = O.matmul(a[rows], b, BF)
    got = c[rows.to(cuda_device)].cpu()
    assert torch.allclose(got.float(), ref.float(), **TOL16)
    assert torch.isfinite(c.float()).all()


def test_gemm_linearity_at_large_size(cuda_device):
    """Size-independent property at a shape the CPU oracle cannot afford: A(B1+B2) = AB1 + AB2
    for integer-valued inputs (exact), plus a sampled oracle check."""
    g = gen(5)
    m, n, k = 4096, 7168, 2048
    a = torch.randint(-2, 3, (m, k), generator=g).to(BF).to(cuda_device)
    b1 = torch.randint(-2, 3, (k, n), generator=g).to(BF).to(cuda_device)
    b2 = torch.randint(-2, 3, (k, n), generator=g).to(BF).to(cuda_device)
    c1 = torch.empty(m, n, dtype=F32, device=cuda_device)
    c2 = torch.empty_like(c1)
    c12 = torch.empty_like(c1)
    ops.gemm(a, b1, c1)
    ops.gemm(a, b2, c2)
    ops.gemm(a, b1 + b2, c12)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(c12, c1 + c2)
    rows = torch.randint(0, m, (16,), generator=g)
    ref = O.matmul(a[rows].cpu(), b1.cpu(), F32)
    assert torch.equal(c1[rows].cpu(), ref)


def test_gemm_argument_errors(cuda_device):
    a = torch.zeros(8, 16, dtype=BF, device=cuda_device)
    with pytest.raises(ValueError, match="K shape"):
        ops.gemm(a, torch.zeros(8, 8, dtype=BF, device=cuda_device), torch.zeros(8, 8, dtype=BF, device=cuda_device))
    with pytest.raises(ValueError):
        ops.gemm(a, torch.zeros(16, 8, dtype=HF, device=cuda_device), torch.zeros(8, 8, dtype=BF, device=cuda_device))


@pytest.mark.parametrize("transpose_b", [False, True])
@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (256, 512, 384), (200, 144, 80), (1, 16, 16), (1024, 1024, 1024),
                                   (384, 1296, 528)])
def test_gemm_e4m3_operands(cuda_device, transpose_b, m, n, k):
    """The plain FP8 operand form of ppl_gemm (src/target/codegen_ppl.cc:775-790): e4m3 A and B, fp32 accumulate.
    Products of e4m3 values are exact in fp32, so only the summation order separates kernel and oracle."""
    F8 = torch.float8_e4m3fn
    g = gen(m + 5 * n + 11 * k)
    a = torch.randn(m, k, generator=g).to(F8)
    b = (torch.randn(n, k, generator=g) if transpose_b else torch.randn(k, n, generator=g)).to(F8)
    ref = O.matmul(a.float(), b.float(), F32, transpose_b)
    c = run(a, b, F32, transpose_b, cuda_device)
    assert ((c.double() - ref.double()).abs() <= 1e-4 * k ** 0.5 + 1e-5 * ref.double().abs()).all()
    c16 = run(a, b, BF, transpose_b, cuda_device)
    assert torch.allclose(c16.float(), ref.to(BF).float(), **TOL16)
    # small integers: every partial sum is exact, the result must be bit-identical
    ai = torch.randint(-3, 4, (m, k), generator=g).float().to(F8)
    bi = torch.randint(-3, 4, (n, k) if transpose_b else (k, n), generator=g).float().to(F8)
    assert torch.equal(run(ai, bi, F32, transpose_b, cuda_device), O.matmul(ai.float(), bi.float(), F32, transpose_b))


PAIR = 512          # tile_n value of the CTA-pair kernel: 256 x 256 tiles of C, each on two SMs (cta_group::2)


@pytest.mark.parametrize("transpose_b", [False, True])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (256, 256, 1024), (512, 768, 256), (200, 136, 72), (129, 264, 200),
                                   (1, 8, 8), (384, 1288, 520), (2048, 4096, 512), (5000, 2304, 640)])
def test_gemm_cta_pair_tiles(cuda_device, transpose_b, m, n, k):
    """The CTA-pair kernel against the oracle on full, ragged and tiny shapes (rows and columns past the edge are
    zero-filled by the loads and masked by the stores), and bit-exact on small integers in every operand type."""
    g = gen(m * 5 + n * 3 + k + 1)
    for dtype in (BF, HF):
        a = torch.randn(m, k, generator=g).to(dtype)
        b = (torch.randn(n, k, generator=g) if transpose_b else torch.randn(k, n, generator=g)).to(dtype)
        ref32 = O.matmul(a, b, F32, transpose_b)
        c = run(a, b, dtype, transpose_b, cuda_device, PAIR)
        assert torch.allclose(c.float(), ref32.to(dtype).float(), **TOL16)
        c32 = run(a, b, F32, transpose_b, cuda_device, PAIR)
        assert ((c32.double() - ref32.double()).abs() <= 1e-3 * k ** 0.5 + 1e-4 * ref32.double().abs()).all()
    ai = torch.randint(-4, 5, (m, k), generator=g).to(BF)
    bi = torch.randint(-4, 5, (n, k) if transpose_b else (k, n), generator=g).to(BF)
    refi = O.matmul(ai, bi, F32, transpose_b)
    assert torch.equal(run(ai, bi, F32, transpose_b, cuda_device, PAIR), refi)
    # the pair kernel and the one-CTA kernel add the same products in the same order per output element
    assert torch.equal(run(a, b, F32, transpose_b, cuda_device, PAIR), run(a, b, F32, transpose_b, cuda_device, 256))


@pytest.mark.parametrize("transpose_b", [False, True])
@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (512, 768, 384), (200, 144, 80), (1024, 1024, 1024), (384, 1296, 528)])
def test_gemm_cta_pair_tiles_e4m3(cuda_device, transpose_b, m, n, k):
    F8 = torch.float8_e4m3fn
    g = gen(m + 3 * n + 7 * k)
    a = torch.randn(m, k, generator=g).to(F8)
    b = (torch.randn(n, k, generator=g) if transpose_b else torch.randn(k, n, generator=g)).to(F8)
    ref = O.matmul(a.float(), b.float(), F32, transpose_b)
    c = run(a, b, F32, transpose_b, cuda_device, PAIR)
    assert ((c.double() - ref.double()).abs() <= 1e-4 * k ** 0.5 + 1e-5 * ref.double().abs()).all()
    assert torch.allclose(run(a, b, BF, transpose_b, cuda_device, PAIR).float(), ref.to(BF).float(), **TOL16)
    ai = torch.randint(-3, 4, (m, k), generator=g).float().to(F8)
    bi = torch.randint(-3, 4, (n, k) if transpose_b else (k, n), generator=g).float().to(F8)
    assert torch.equal(run(ai, bi, F32, transpose_b, cuda_device, PAIR), O.matmul(ai.float(), bi.float(), F32, transpose_b))
