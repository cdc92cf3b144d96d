"""Parity of the block-scaled FP8 GEMM against the oracle (explicit de-quantised product)."""
import pytest
import torch

import oracle.ops as O
from conftest import load_golden
from tilelang import ops

pytestmark = pytest.mark.gpu
F8 = torch.float8_e4m3fn


def gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def run(a8, b8, sa, sb, out_dtype, dev):
    c = torch.full((a8.shape[0], b8.shape[0]), float("nan"), dtype=out_dtype, device=dev)
    assert ops.gemm_fp8_blockscale(a8.to(dev), b8.to(dev), sa.to(dev), sb.to(dev), c) == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return c.cpu()


def quantised(m, n, k, seed, amp=0.05):
    g = gen(seed)
    a8, sa = O.per_token_cast_to_fp8(torch.randn(m, k, generator=g) * amp)
    b8, sb = O.per_block_cast_to_fp8(torch.randn(n, k, generator=g) * amp)
    return a8, b8, sa.contiguous(), sb.contiguous()


def test_golden_quantised_operands(cuda_device):
    g = load_golden("fp8_quant", dict(a8=F8, b8=F8))
    ref = O.gemm_fp8_blockscale(g["a8"], g["b8"], g["sa"], g["sb"], torch.float32)
    out = run(g["a8"], g["b8"], g["sa"], g["sb"], torch.float32, cuda_device)
    assert torch.allclose(out, ref, atol=1e-4, rtol=1e-4)
    out16 = run(g["a8"], g["b8"], g["sa"], g["sb"], torch.bfloat16, cuda_device)
    assert torch.allclose(out16.float(), ref, atol=2e-2, rtol=2e-2)


# the shapes of the second line give every pair of SMs a 256 x 128 tile and so run on CTA pairs, with ragged edges in
# both directions (300 rows: the odd CTA of the last row block has no row at all)
@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 384, 512), (200, 136, 256), (1, 8, 128), (130, 1000, 384),
                                   (1024, 2048, 1024),
                                   (2000, 1300, 256), (2304, 1280, 384), (300, 9600, 128), (4096, 4096, 512)])
def test_shapes(cuda_device, m, n, k):
    a8, b8, sa, sb = quantised(m, n, k, m + n + k)
    ref = O.gemm_fp8_blockscale(a8, b8, sa, sb, torch.float32)
    out = run(a8, b8, sa, sb, torch.float32, cuda_device)
    # fp32 accumulation of exact fp8 products: only the summation order differs
    assert torch.allclose(out, ref, atol=1e-4 * k ** 0.5, rtol=1e-4)
    out16 = run(a8, b8, sa, sb, torch.bfloat16, cuda_device)
    assert torch.allclose(out16.float(), ref, atol=2e-2, rtol=2e-2)


def test_scales_are_applied_per_k_block_and_per_n_block(cuda_device):
    """With all-ones bytes the result is exactly sum_kb 128 * sa[m,kb] * sb[nb,kb]."""
    m, n, k = 128, 256, 512
    one = torch.ones(1).to(F8)
    a8 = one.expand(m, k).contiguous()
    b8 = one.expand(n, k).contiguous()
    g = gen(3)
    sa = torch.randint(1, 5, (m, k // 128), generator=g).float()
    sb = torch.randint(1, 5, (n // 128, k // 128), generator=g).float()
    out = run(a8, b8, sa, sb, torch.float32, cuda_device)
    ref = 128.0 * (sa @ sb.t()).repeat_interleave(128, dim=1)
    assert torch.equal(out, ref)


def test_repeated_row_scale_satisfies_the_per_block_wording(cuda_device):
    """One scale per 128x128 block of A (repeated over its 128 rows) is a special case."""
    m, n, k = 256, 256, 256
    g = gen(4)
    a = torch.randn(m, k, generator=g) * 0.05
    a8, sa_blk = O.per_block_cast_to_fp8(a)
    sa = sa_blk.repeat_interleave(128, dim=0).contiguous()
    b8, sb = O.per_block_cast_to_fp8(torch.randn(n, k, generator=g) * 0.05)
    ref = O.gemm_fp8_blockscale(a8, b8, sa, sb, torch.float32)
    assert torch.allclose(run(a8, b8, sa, sb.contiguous(), torch.float32, cuda_device), ref, atol=1e-4, rtol=1e-4)


def test_argument_errors(cuda_device):
    a8, b8, sa, sb = quantised(128, 128, 128, 1)
    with pytest.raises(ValueError):
        ops.gemm_fp8_blockscale(a8.to(cuda_device), b8.to(cuda_device), sa.to(cuda_device), sb.to(cuda_device),
                                torch.zeros(128, 128, dtype=torch.float16, device=cuda_device))
    with pytest.raises(ValueError):
        ops.gemm_fp8_blockscale(a8.to(cuda_device)[:, :64].contiguous(), b8.to(cuda_device)[:, :64].contiguous(),
                                sa.to(cuda_device), sb.to(cuda_device),
                                torch.zeros(128, 128, dtype=torch.bfloat16, device=cuda_device))


def calc_diff(x, y):
    """1 - cosine-style similarity: the measure the block-scaled GEMM example asserts on
    (examples/deepseek_deepgemm/example_deepgemm_fp8_2xAcc.py:142-146, `diff < 1e-3`)."""
    x, y = x.double(), y.double()
    return float(1 - 2 * (x * y).sum() / (x * x + y * y).sum())


def test_against_the_reference_functions_own_result(cuda_device):
    """tests/golden/fp8_gemm_ref.npz holds the output of the reference's `ref_deepgemm_fp8` (:115-139, per-block
    torch._scaled_mm on a CUDA device, every 128-wide partial rounded to bf16 before the fp32 sum) on operands cut
    by its own quantisers: oracle and kernel must meet it within the example's own criterion."""
    from conftest import GOLDEN
    if not (GOLDEN / "fp8_gemm_ref.npz").exists():
        pytest.skip("fixture not generated (needs a CUDA device and the reference tree)")
    g = load_golden("fp8_gemm_ref", dict(a8=F8, b8=F8, ref=torch.bfloat16))
    out = run(g["a8"], g["b8"], g["sa"].contiguous(), g["sb"].contiguous(), torch.bfloat16, cuda_device)
    assert calc_diff(out, g["ref"]) < 1e-3
    assert torch.allclose(out.float(), g["ref"].float(), atol=2e-2, rtol=2e-2)


def test_llama70b_ffn_config(cuda_device):
    """e4m3 M8192 K8192 N28672 (0.05 N(0,1), seed 2) cut by the example's quantisers: the oracle on 64 rows
    spread over every 128-row tile band and all columns, at the stated tolerance."""
    g = gen(2)
    m, k, n = 8192, 8192, 28672
    a8, sa = O.per_token_cast_to_fp8(torch.randn(m, k, generator=g) * 0.05)
    b = torch.randn(k, n, generator=g) * 0.05                    # drawn as [K, N] like the bf16 configuration
    b8, sb = O.per_block_cast_to_fp8(b.t().contiguous())
    del b
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    assert ops.gemm_fp8_blockscale(a8.to(cuda_device), b8.to(cuda_device), sa.contiguous().to(cuda_device),
                                   sb.contiguous().to(cuda_device), out) == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    rows = torch.arange(64) * 128 + torch.randint(0, 128, (64,), generator=g)
    ref = O.gemm_fp8_blockscale(a8[rows], b8, sa[rows], sb, torch.float32)
    got = out[rows.to(cuda_device)].cpu().float()
    assert torch.allclose(got, ref, atol=2e-2, rtol=2e-2)
    assert calc_diff(got, ref) < 1e-3
    assert torch.isfinite(out.float()).all()
