"""Parity of paged MLA decode (tcgen05 FP8 kernel and FMA kernel) against the oracle."""
import pytest
import torch

import oracle.ops as O
from conftest import load_golden
from tilelang import ops, workloads

pytestmark = pytest.mark.gpu
BF, HF, F8 = torch.bfloat16, torch.float16, torch.float8_e4m3fn


def run(w, dev, heads=None, balanced=True):
    q = w["q"].to(dev)
    b, h = q.shape[0], q.shape[-2]
    out = torch.full((b, h, w["dv"]), float("nan"), dtype=q.dtype, device=dev)
    scale = w["kv_scale"].to(dev) if w["kv_scale"] is not None else None
    assert ops.mla_decode_paged(q, w["kv_cache"].to(dev), scale, w["block_table"].to(dev),
                                w["cache_seqlens"].to(dev), out, softmax_scale=w["softmax_scale"],
                                balanced=balanced) == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return out.cpu()


def oracle(w, rows=None):
    q = w["q"].reshape(w["q"].shape[0], w["q"].shape[-2], w["q"].shape[-1])
    sel = slice(None) if rows is None else rows
    return O.mla_decode_paged(q[sel], w["kv_cache"], w["kv_scale"], w["block_table"][sel], w["cache_seqlens"][sel],
                              w["dv"])


# The tensor-core path feeds the query and the softmax weights to the FP8 tensor core as two e4m3
# terms each (value + residual), which keeps ~8 mantissa bits: the stated 2e-2 holds with margin
# and the error in norm stays below one percent.
def assert_close(out, ref, rel_norm=0.01, tol=2e-2):
    assert torch.allclose(out.float(), ref.float(), atol=tol, rtol=tol), (out.float() - ref.float()).abs().max()
    # FP8 attention (query cut to e4m3 with one scale per head) is a few percent accurate in norm;
    # random-data outputs are small, so the absolute tolerance alone would say little
    err = (out.float() - ref.float()).norm() / ref.float().norm().clamp_min(1e-12)
    assert err < rel_norm, f"relative error {err.item():.4f}"


def test_golden_paged_fp16_cache(cuda_device):
    g = load_golden("mla_paged_fp16", dict(q=HF, blocked_k=HF, ref=HF))
    w = dict(q=g["q"], kv_cache=g["blocked_k"][:, :, 0].contiguous(), kv_scale=None, block_table=g["block_table"],
             cache_seqlens=g["cache_seqlens"], dv=int(g["dv"]), softmax_scale=96 ** -0.5)
    out = run(w, cuda_device)
    assert torch.allclose(out.float(), g["ref"][:, 0].float(), atol=1e-2, rtol=1e-2)   # the example's tolerance


@pytest.mark.parametrize("dtype", [BF, HF])
def test_fma_kernel_small_fp8(cuda_device, dtype):
    w = workloads.mla_fp8_paged(batch=3, heads=8, d=64, dv=32, page_size=16, min_len=1, max_len=100, seed=5, dtype=dtype)
    assert_close(run(w, cuda_device), oracle(w))


@pytest.mark.parametrize("heads,page,lens", [(128, 64, (1, 64, 65, 500, 1000, 2048)), (16, 64, (300, 77)),
                                             (128, 128, (129, 1024, 640)), (100, 64, (2000,))])
def test_tensor_core_kernel(cuda_device, heads, page, lens):
    w = workloads.mla_fp8_paged(batch=len(lens), heads=heads, page_size=page, min_len=1, max_len=max(lens), seed=7)
    w["cache_seqlens"] = torch.tensor(lens, dtype=torch.int32)
    assert_close(run(w, cuda_device), oracle(w))


def test_tensor_core_kernel_fp16_queries_and_empty_sequence(cuda_device):
    w = workloads.mla_fp8_paged(batch=3, heads=128, min_len=100, max_len=700, seed=8, dtype=HF)
    w["cache_seqlens"][1] = 0
    out = run(w, cuda_device)
    ref = oracle(w, rows=[0, 2])
    assert_close(out[[0, 2]], ref)
    assert (out[1] == 0).all()


def paged_16bit(batch, heads, lens, page, dtype, seed, d=576):
    g = torch.Generator().manual_seed(seed)
    lens = torch.tensor(lens, dtype=torch.int32)
    pages = (lens + page - 1) // page
    total = int(pages.sum()) + 3
    perm = torch.randperm(total, generator=g).to(torch.int32)
    table = torch.zeros(batch, int(pages.max()) + 1, dtype=torch.int32)
    cur = 0
    for i in range(batch):
        table[i, :int(pages[i])] = perm[cur:cur + int(pages[i])]
        cur += int(pages[i])
    cache = torch.randn(total, page, d, generator=g).to(dtype)
    q = torch.randn(batch, heads, d, generator=g).to(dtype)
    return dict(q=q, kv_cache=cache, kv_scale=None, block_table=table, cache_seqlens=lens, dv=512, softmax_scale=d ** -0.5)


@pytest.mark.parametrize("dtype", [BF, HF])
@pytest.mark.parametrize("heads,page,lens", [(128, 64, (1, 64, 65, 500, 1000, 2048)), (16, 64, (300, 77, 0)),
                                             (128, 128, (129, 1024, 640)), (100, 64, (1500,))])
def test_16bit_cache_on_tensor_cores(cuda_device, dtype, heads, page, lens):
    """bf16 / fp16 latent caches at the DeepSeek shape (d 576, dv 512) run the tcgen05 kernel of mla_f16.cu (layout of
    examples/deepseek_mla/example_mla_decode_paged.py:20-97): oracle parity at the stated tolerance, every length class
    (one token, exactly one tile, a ragged tail, an empty sequence)."""
    w = paged_16bit(len(lens), heads, lens, page, dtype, seed=heads + page)
    out = run(w, cuda_device)
    ref = oracle(w)
    live = [i for i, n in enumerate(lens) if n > 0]
    assert torch.allclose(out[live].float(), ref[live].float(), atol=2e-2, rtol=2e-2)
    for i, n in enumerate(lens):
        if n == 0:
            assert (out[i] == 0).all()
    a = run(w, cuda_device)
    assert torch.equal(a.view(torch.int16), out.view(torch.int16))              # run-to-run determinism
    # with the large scratch every sequence is cut into several shares of its key tiles that are merged by their
    # log-sum-exp (split-KV); with the minimal scratch one CTA pair walks a whole sequence: same answer
    whole = run(w, cuda_device, balanced=False)
    assert torch.allclose(whole[live].float(), ref[live].float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(whole.float(), out.float(), atol=4e-3, rtol=2e-2)


@pytest.mark.parametrize("s_q,h_q,h_kv,d,dv,page", [(1, 128, 1, 576, 512, 64), (2, 64, 2, 576, 512, 64), (4, 32, 1, 576, 512, 64),
                                                    (3, 16, 2, 576, 512, 128), (2, 8, 2, 64, 32, 16), (3, 4, 1, 96, 64, 16)])
def test_several_query_tokens_and_kv_heads(cuda_device, s_q, h_q, h_kv, d, dv, page):
    """s_q > 1 and h_kv > 1 (examples/deepseek_mla/example_mla_decode_paged.py:99-256, checked there against
    `run_torch_mla`): the DeepSeek-shaped cases run on tensor cores with the (query token, head) pairs of a kv head as
    the rows of the MMAs, the others on the FMA kernel."""
    g = torch.Generator().manual_seed(s_q * 100 + h_q)
    lens = torch.tensor([300, 65, s_q, 1000][:3 if d != 576 else 4], dtype=torch.int32).clamp(max=20 * page)
    b = lens.numel()
    pages = (lens + page - 1) // page
    total = int(pages.sum()) + 2
    perm = torch.randperm(total, generator=g).to(torch.int32)
    table = torch.zeros(b, int(pages.max()), dtype=torch.int32)
    cur = 0
    for i in range(b):
        table[i, :int(pages[i])] = perm[cur:cur + int(pages[i])]
        cur += int(pages[i])
    cache = torch.randn(total, page, h_kv, d, generator=g).to(BF)
    q = torch.randn(b, s_q, h_q, d, generator=g).to(BF)
    out = torch.full((b, s_q, h_q, dv), float("nan"), dtype=BF, device=cuda_device)
    assert ops.mla_decode_paged_gqa(q.to(cuda_device), cache.to(cuda_device), table.to(cuda_device), lens.to(cuda_device), out) == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    ref = O.mla_decode_paged_gqa(q, cache, table, lens, dv)
    assert torch.allclose(out.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_peaked_attention_rows(cuda_device):
    """A query aligned with one cached token: softmax is nearly one-hot, so the output must
    reproduce that token's value row (checks the scale folding and the two-term P split)."""
    w = workloads.mla_fp8_paged(batch=2, heads=128, min_len=300, max_len=400, seed=9)
    cache, scale, table = w["kv_cache"], w["kv_scale"], w["block_table"]
    for b, t in ((0, 17), (1, 250)):
        page, slot = int(table[b, t // 64]), t % 64
        k = cache[page, slot].float() * scale[page, slot]
        w["q"][b, 0, :, :] = (k * 3.0).to(BF)
    out = run(w, cuda_device)
    assert_close(out, oracle(w))


def test_balanced_kernel_matches_the_per_sequence_kernel(cuda_device):
    """The persistent kernel cuts sequences at range boundaries and merges the pieces; the
    per-sequence kernel (small workspace) never cuts.  Same answers either way, for a batch far
    smaller than the GPU, one near its size and one with empty and one-token sequences."""
    for kw in (dict(batch=3, min_len=1500, max_len=4000, seed=12), dict(batch=40, min_len=1, max_len=700, seed=13),
               dict(batch=150, min_len=0, max_len=130, seed=14)):
        w = workloads.mla_fp8_paged(heads=128, **kw)
        if kw["seed"] == 14:
            w["cache_seqlens"][::7] = 0
            w["cache_seqlens"][1::7] = 1
        out_a = run(w, cuda_device)
        out_b = run(w, cuda_device, balanced=False)
        assert torch.allclose(out_a.float(), out_b.float(), atol=2e-3, rtol=1e-2)      # bf16: a few units in the last place
        assert_close(out_a, oracle(w))


def test_run_to_run_determinism(cuda_device):
    w = workloads.mla_fp8_paged(batch=4, heads=128, min_len=500, max_len=1500, seed=10)
    a = run(w, cuda_device)
    assert torch.equal(run(w, cuda_device).view(torch.int16), a.view(torch.int16))


def test_benchmark_config(cuda_device):
    """Batch 128, 128 heads, lengths uniform in [1024, 8192]: oracle on a sample of sequences and a
    size-independent property on all (outputs lie inside the range of the de-quantised V rows)."""
    w = workloads.mla_fp8_paged()
    out = run(w, cuda_device)
    assert torch.isfinite(out.float()).all()
    lens = w["cache_seqlens"]
    rows = sorted({int(lens.argmin()), int(lens.argmax()), 0, 127} | set(range(5, 128, 10)))    # 16+ sequences
    assert len(rows) >= 16
    assert_close(out[rows], oracle(w, rows=rows))
    vmax = (w["kv_cache"].float().abs().amax(dim=(1, 2)) * w["kv_scale"].amax(dim=1)).max()
    assert out.float().abs().max() <= vmax


def test_argument_errors(cuda_device):
    w = workloads.mla_fp8_paged(batch=2, heads=8, d=64, dv=32, page_size=16, min_len=1, max_len=40, seed=1)
    q = w["q"].to(cuda_device)
    out = torch.zeros(2, 8, 32, dtype=BF, device=cuda_device)
    with pytest.raises(ValueError, match="kv_scale"):
        ops.mla_decode_paged(q, w["kv_cache"].to(cuda_device), None, w["block_table"].to(cuda_device),
                             w["cache_seqlens"].to(cuda_device), out)
    with pytest.raises(ValueError, match="int32"):
        ops.mla_decode_paged(q, w["kv_cache"].to(cuda_device), w["kv_scale"].to(cuda_device),
                             w["block_table"].to(cuda_device).long(), w["cache_seqlens"].to(cuda_device), out)
