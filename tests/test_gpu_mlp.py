"""Parity of the fused gate/up projection + SiLU-product kernel (front half of the MLP program,
tpu_demo/ppl/mlp/mlp_bf16.py) against the oracle and against the unfused kernels, through the C ABI."""
import pytest
import torch

import oracle.ops as O
from tilelang import ops

pytestmark = pytest.mark.gpu
BF, HF, F32 = torch.bfloat16, torch.float16, torch.float32


def make(m, n, k, dtype, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(m, k, generator=g).to(dtype)
    wg = (torch.randn(n, k, generator=g) / k ** 0.5).to(dtype)      # gate and up come out ~ N(0, 1)
    wu = (torch.randn(n, k, generator=g) / k ** 0.5).to(dtype)
    return x, wg, wu


def fused(x, wg, wu, dev):
    out = torch.full((x.shape[0], wg.shape[0]), float("nan"), dtype=x.dtype, device=dev)
    assert ops.mlp_gate_up(x.to(dev), wg.to(dev), wu.to(dev), out) == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return out.cpu()


def unfused(x, wg, wu, dev):
    m, n = x.shape[0], wg.shape[0]
    xd = x.to(dev)
    gate = torch.empty(m, n, dtype=x.dtype, device=dev)
    up = torch.empty(m, n, dtype=x.dtype, device=dev)
    out = torch.empty(m, n, dtype=x.dtype, device=dev)
    assert ops.gemm(xd, wg.to(dev), gate, True) == 0 and ops.gemm(xd, wu.to(dev), up, True) == 0
    assert ops.swiglu(gate, up, out) == 0
    torch.cuda.synchronize()
    return out.cpu()


@pytest.mark.parametrize("dtype", [BF, HF])
# the shapes of the last line give every pair of SMs a 256-row tile and run on CTA pairs, ragged in both directions
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 384, 512), (64, 64, 64), (1024, 1024, 1024), (200, 136, 72),
                                   (129, 264, 200), (1, 8, 8), (384, 1288, 520),
                                   (2000, 1300, 256), (300, 9600, 72), (2304, 1280, 520)])
def test_tensor_core_shapes(cuda_device, dtype, m, n, k):
    x, wg, wu = make(m, n, k, dtype, m * 7 + n * 3 + k)
    out = fused(x, wg, wu, cuda_device)
    ref = O.mlp_gate_up(x, wg, wu)
    # a unit in the last place of a rounded gate or up value moves the product by about 2^-8 (bf16)
    assert torch.allclose(out.float(), ref.float(), atol=2e-2, rtol=2e-2)
    # same accumulation order and the same SiLU expression as the separate kernels: identical bits
    assert torch.equal(out.view(torch.int16), unfused(x, wg, wu, cuda_device).view(torch.int16))


@pytest.mark.parametrize("dtype,m,n,k", [(F32, 96, 80, 56), (BF, 33, 47, 13), (HF, 17, 9, 5), (F32, 1, 1, 1)])
def test_fma_path_shapes(cuda_device, dtype, m, n, k):
    """fp32 and shapes whose rows are not 16-byte multiples."""
    x, wg, wu = make(m, n, k, dtype, 11 * m + n + k)
    out = fused(x, wg, wu, cuda_device)
    ref = O.mlp_gate_up(x, wg, wu)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == F32 else dict(atol=2e-2, rtol=2e-2)
    assert torch.allclose(out.float(), ref.float(), **tol)


def test_whole_mlp_matches_the_program(cuda_device):
    """gate/up + SiLU-product, then the down projection as a plain GEMM with trans_b."""
    m, hidden, inter = 256, 512, 1024
    x, wg, wu = make(m, inter, hidden, BF, 5)
    g = torch.Generator(device="cpu").manual_seed(6)
    wd = (torch.randn(hidden, inter, generator=g) / inter ** 0.5).to(BF)
    act = torch.empty(m, inter, dtype=BF, device=cuda_device)
    y = torch.empty(m, hidden, dtype=BF, device=cuda_device)
    assert ops.mlp_gate_up(x.to(cuda_device), wg.to(cuda_device), wu.to(cuda_device), act) == 0
    assert ops.gemm(act, wd.to(cuda_device), y, True) == 0
    torch.cuda.synchronize()
    assert torch.allclose(y.cpu().float(), O.mlp(x, wg, wu, wd).float(), atol=2e-2, rtol=2e-2)


def test_zero_gate_and_linearity_in_up(cuda_device):
    """Size-independent properties at a Llama-3-8B-like shape: a zero gate weight gives exact zeros
    (silu(0) = 0); scaling the up weight by 2 doubles every output exactly (a power of two commutes
    with every rounding)."""
    m, n, k = 2048, 14336, 4096
    x, wg, wu = make(m, n, k, BF, 9)
    assert (fused(x, torch.zeros_like(wg), wu, cuda_device) == 0).all()
    a = fused(x, wg, wu, cuda_device)
    b = fused(x, wg, (wu.float() * 2).to(BF), cuda_device)
    assert torch.equal((a.float() * 2).to(BF).view(torch.int16), b.view(torch.int16))
    rows = [0, 777, 2047]
    assert torch.allclose(a[rows].float(), O.mlp_gate_up(x[rows], wg, wu).float(), atol=2e-2, rtol=2e-2)


def test_argument_errors(cuda_device):
    x, wg, wu = make(8, 8, 8, BF, 1)
    out = torch.empty(8, 8, dtype=BF, device=cuda_device)
    with pytest.raises(ValueError, match="K shape"):
        ops.mlp_gate_up(x.to(cuda_device), wg[:, :4].contiguous().to(cuda_device), wu[:, :4].contiguous().to(cuda_device), out)
    with pytest.raises(ValueError, match="dtype"):
        ops.mlp_gate_up(x.to(cuda_device), wg.half().to(cuda_device), wu.to(cuda_device), out)
    assert ops.mlp_gate_up(x[:0].to(cuda_device), wg.to(cuda_device), wu.to(cuda_device), out[:0]) == 0
