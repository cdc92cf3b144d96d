"""Bit-exact parity of gather and top-k (index-valued programs) through the C ABI."""
import pytest
import torch

import oracle.ops as O
from conftest import load_golden
from tilelang import ops

pytestmark = pytest.mark.gpu


def gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def test_gather_golden(cuda_device):
    g = load_golden("gather_fp32")
    out = torch.zeros(8, 64, device=cuda_device)
    ops.gather_rows(g["param"].to(cuda_device), g["index"].view(torch.uint32).to(cuda_device), out)
    assert torch.equal(out.cpu(), g["ref"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,hidden,n", [(128, 64, 8), (1000, 4096, 333), (7, 3, 20), (50, 1, 50), (32768, 512, 8192)])
def test_gather_shapes(cuda_device, dtype, rows, hidden, n):
    g = gen(rows + hidden + n)
    param = torch.randn(rows, hidden, generator=g).to(dtype)
    idx = torch.randint(0, rows, (n, 1), generator=g, dtype=torch.int32)
    ref = O.gather_rows(param, idx)
    out = torch.zeros(n, hidden, dtype=dtype, device=cuda_device)
    ops.gather_rows(param.to(cuda_device), idx.to(cuda_device), out)
    assert torch.equal(out.cpu().view(torch.uint8), ref.view(torch.uint8))


@pytest.mark.parametrize("width", [8, 136, 520])         # 520 fp32 = 130 vectors: the warp-per-row form, ragged
def test_gather_out_of_range_index_writes_zeros(cuda_device, width):
    param = torch.ones(4, width, device=cuda_device)
    idx = torch.tensor([[0], [4], [3], [2 ** 31 - 1]], dtype=torch.int32, device=cuda_device)
    out = torch.full((4, width), 7.0, device=cuda_device)
    ops.gather_rows(param, idx, out)
    assert out.cpu().tolist() == [[1.0] * width, [0.0] * width, [1.0] * width, [0.0] * width]


def test_gather_empty(cuda_device):
    param = torch.ones(4, 8, device=cuda_device)
    assert ops.gather_rows(param, torch.empty(0, 1, dtype=torch.int32, device=cuda_device),
                           torch.empty(0, 8, device=cuda_device)) == 0


def test_topk_golden(cuda_device):
    g = load_golden("topk_fp32")
    vals = torch.zeros(1024, device=cuda_device)
    idx = torch.zeros(1024, dtype=torch.int32, device=cuda_device)
    ops.topk(g["src"].to(cuda_device), vals, idx, 8, True)
    assert torch.equal(idx[:8].cpu(), g["ref_idx"])
    assert torch.equal(vals[:8].cpu(), g["ref_vals"])
    assert (vals[8:] == 0).all()           # only the first K entries are written


@pytest.mark.parametrize("desc", [True, False])
@pytest.mark.parametrize("rows,length,k", [(1, 1024, 8), (8192, 256, 8), (5, 37, 37), (3, 1000, 16),
                                           (2, 5000, 10), (1, 70000, 4), (4, 1, 1), (9, 257, 3), (3, 3000, 40),
                                           (2, 2048, 8), (2, 4096, 33), (1, 6000, 70)])
def test_topk_fp32_shapes(cuda_device, rows, length, k, desc):
    # a random permutation of distinct values: tie-free, so positions are pinned
    g = gen(rows * 3 + length + k)
    src = torch.stack([torch.randperm(length, generator=g).float() - length / 2 for _ in range(min(rows, 64))])
    if rows > 64:
        src = src.repeat(rows // 64, 1)
    src = (src * 0.37).contiguous()
    rv, ri = O.topk(src, k, desc)
    vals = torch.zeros(src.shape[0], k, device=cuda_device)
    idx = torch.zeros(src.shape[0], k, dtype=torch.int32, device=cuda_device)
    ops.topk(src.to(cuda_device), vals, idx, k, desc)
    assert torch.equal(idx.cpu(), ri.reshape(-1, k))
    assert torch.equal(vals.cpu(), rv.reshape(-1, k))
    # same positions as torch.topk on tie-free input (the reference's check function)
    tv, ti = torch.topk(src, k, largest=desc, sorted=True)
    assert torch.equal(idx.cpu().long(), ti)


@pytest.mark.parametrize("dtype", [torch.int32, torch.float32])
def test_topk_ties_lower_index_first(cuda_device, dtype):
    src = torch.tensor([[1, 3, 3, -2, 3, 0, 3, -2]], dtype=dtype)
    for length_pad in (0, 2000):
        s = torch.cat([src, torch.full((1, length_pad), -9, dtype=dtype)], dim=1).contiguous()
        for desc in (True, False):
            k = 5 if desc else 2       # ascending: only the two -2 entries are pinned (pad is lower)
            if not desc and length_pad:
                continue
            rv, ri = O.topk(s, k, desc)
            vals = torch.zeros(1, k, dtype=dtype, device=cuda_device)
            idx = torch.zeros(1, k, dtype=torch.int32, device=cuda_device)
            ops.topk(s.to(cuda_device), vals, idx, k, desc)
            assert torch.equal(idx.cpu(), ri) and torch.equal(vals.cpu(), rv)


@pytest.mark.parametrize("desc", [True, False])
@pytest.mark.parametrize("dtype", [torch.int32, torch.float32])
@pytest.mark.parametrize("rows,length,k,levels", [(64, 1024, 8, 3), (33, 1000, 32, 5), (16, 2048, 16, 2), (8, 1537, 8, 1),
                                                  (40, 255, 32, 40), (7, 31, 20, 4), (16, 1024, 32, 2000)])
def test_topk_many_equal_values(cuda_device, dtype, rows, length, k, levels, desc):
    """Few distinct values: the candidate set of the threshold selection overflows its 32 slots (the round-by-round
    path runs), and every tie must still come out lower position first; 2000 levels gives a mix of both paths."""
    g = gen(rows + length * 7 + k + levels)
    src = torch.randint(-levels, levels + 1, (rows, length), generator=g).to(dtype)
    rv, ri = O.topk(src, k, desc)
    vals = torch.zeros(rows, k, dtype=dtype, device=cuda_device)
    idx = torch.zeros(rows, k, dtype=torch.int32, device=cuda_device)
    ops.topk(src.to(cuda_device), vals, idx, k, desc)
    assert torch.equal(idx.cpu(), ri.reshape(rows, k))
    assert torch.equal(vals.cpu(), rv.reshape(rows, k))


@pytest.mark.parametrize("desc", [True, False])
@pytest.mark.parametrize("rows,length,k,levels", [(600, 4096, 8, 0), (600, 2501, 32, 0), (640, 4096, 8, 3), (600, 3001, 5, 50),
                                                  (592, 16384, 16, 100000), (600, 8192, 32, 0)])
def test_topk_many_long_rows(cuda_device, rows, length, k, levels, desc):
    """Enough rows of 2049..16384 elements for the one-warp-per-row streaming kernel; levels 0 = distinct values."""
    g = gen(rows + length + k + levels)
    if levels:
        src = torch.randint(-levels, levels + 1, (rows, length), generator=g).float()
    else:
        src = torch.stack([torch.randperm(length, generator=g).float() for _ in range(8)]).repeat(rows // 8, 1) * 0.25 - 100.0
    src = src.contiguous()
    ref = torch.sort(src, dim=1, descending=desc, stable=True)
    rv, ri = O.topk(src[:16], k, desc)
    assert torch.equal(ri.reshape(16, k).long(), ref.indices[:16, :k])       # the oracle's order = a stable sort's
    vals = torch.zeros(rows, k, device=cuda_device)
    idx = torch.zeros(rows, k, dtype=torch.int32, device=cuda_device)
    ops.topk(src.to(cuda_device), vals, idx, k, desc)
    assert torch.equal(idx.cpu().long(), ref.indices[:, :k])
    assert torch.equal(vals.cpu(), ref.values[:, :k])


def test_topk_row_base_not_16_byte_aligned(cuda_device):
    """A view that starts 4 bytes into an allocation takes the scalar-load form of the kernel."""
    g = gen(77)
    base = torch.randn(4 * 1024 + 1, generator=g)
    src = base[1:].view(4, 1024)
    rv, ri = O.topk(src.contiguous(), 8, True)
    dev = base.to(cuda_device)[1:].view(4, 1024)
    vals = torch.zeros(4, 8, device=cuda_device)
    idx = torch.zeros(4, 8, dtype=torch.int32, device=cuda_device)
    ops.topk(dev, vals, idx, 8, True)
    assert torch.equal(idx.cpu(), ri.reshape(4, 8)) and torch.equal(vals.cpu(), rv.reshape(4, 8))


def test_topk_negative_and_special_floats(cuda_device):
    src = torch.tensor([[-1.5, float("-inf"), 2.0, float("inf"), -0.25, 1e-38, -1e-38, 3.5]])
    rv, ri = O.topk(src, 8, True)
    vals = torch.zeros(1, 8, device=cuda_device)
    idx = torch.zeros(1, 8, dtype=torch.int32, device=cuda_device)
    ops.topk(src.to(cuda_device), vals, idx, 8, True)
    assert torch.equal(idx.cpu(), ri) and torch.equal(vals.cpu(), rv)


def test_topk_argument_errors(cuda_device):
    src = torch.zeros(16, device=cuda_device)
    with pytest.raises(RuntimeError, match="exceeds length"):
        ops.topk(src, torch.zeros(32, device=cuda_device), torch.zeros(32, dtype=torch.int32, device=cuda_device), 17)
    with pytest.raises(ValueError):
        ops.topk(src.half(), torch.zeros(16, device=cuda_device).half(),
                 torch.zeros(16, dtype=torch.int32, device=cuda_device), 2)
