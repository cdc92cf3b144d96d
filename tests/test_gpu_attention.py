"""Parity of attention forward (tcgen05 kernel and FMA kernel) and dense MLA decode."""
import math

import pytest
import torch

import oracle.ops as O
from conftest import load_golden
from tilelang import ops

pytestmark = pytest.mark.gpu
BF, HF, F32 = torch.bfloat16, torch.float16, torch.float32
TOL16 = dict(atol=2e-2, rtol=2e-2)


def gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def block_causal_ref(q, k, v, bm, bn):
    """What the reference TPU program computes with is_causal=True: query row r sees the keys
    [0, ceil((r // bm + 1) * bm / bn) * bn) — a shortened loop with no mask inside the last tile."""
    b, s, h, d = q.shape
    rows = torch.arange(s)
    limit = ((rows // bm + 1) * bm + bn - 1) // bn * bn
    mask = torch.arange(s)[None, :] >= limit[:, None]
    scores = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) / math.sqrt(d)
    scores = scores.masked_fill(mask[None, None], float("-inf"))
    w = torch.softmax(scores, dim=-1)
    return torch.einsum("bhqk,bkhd->bqhd", w, v.float()).to(q.dtype)


def run(q, k, v, dev, **kw):
    o = torch.full_like(q, float("nan"), device=dev)
    assert ops.flash_attn_fwd(q.to(dev), k.to(dev), v.to(dev), o, **kw) == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return o.cpu()


def test_golden_small_shape_fma_kernel(cuda_device):
    d = dict(q=BF, k=BF, v=BF, ref_full=BF, ref_causal=BF)
    g = load_golden("flash_attn_bf16", d)
    full = run(g["q"], g["k"], g["v"], cuda_device, causal=False)
    causal = run(g["q"], g["k"], g["v"], cuda_device, causal=True)
    assert torch.allclose(full.float(), g["ref_full"].float(), **TOL16)
    assert torch.allclose(causal.float(), g["ref_causal"].float(), **TOL16)


@pytest.mark.parametrize("dtype", [BF, HF, F32])
def test_reference_demo_shape(cuda_device, dtype):
    g = gen(1)
    q, k, v = (torch.randn(1, 4, 2, 8, generator=g).to(dtype) for _ in range(3))
    out = run(q, k, v, cuda_device, causal=False)
    ref = O.flash_attn_fwd(q, k, v, causal=False)
    if dtype == F32:
        assert torch.allclose(out, ref, atol=1e-5, rtol=1e-5)
    else:
        assert torch.allclose(out.float(), ref.float(), atol=5e-2, rtol=5e-2)       # the demo's tolerance
        assert torch.allclose(out.float(), ref.float(), **TOL16)


@pytest.mark.parametrize("dtype", [BF, HF])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("b,s,h,d", [(1, 256, 2, 128), (2, 512, 3, 64), (1, 320, 2, 128), (1, 1000, 1, 128),
                                     (2, 128, 4, 64), (1, 64, 1, 128), (1, 1536, 2, 128)])
def test_tensor_core_kernel(cuda_device, dtype, causal, b, s, h, d):
    g = gen(b * 5 + s + h * 3 + d)
    q, k, v = (torch.randn(b, s, h, d, generator=g).to(dtype) for _ in range(3))
    ref = O.flash_attn_fwd(q, k, v, causal=causal)
    out = run(q, k, v, cuda_device, causal=causal)
    assert torch.allclose(out.float(), ref.float(), **TOL16), (out.float() - ref.float()).abs().max()


def test_cross_attention_lengths(cuda_device):
    g = gen(3)
    q = torch.randn(2, 200, 2, 128, generator=g).to(BF)
    k = torch.randn(2, 777, 2, 128, generator=g).to(BF)
    v = torch.randn(2, 777, 2, 128, generator=g).to(BF)
    out = run(q, k, v, cuda_device, causal=False)
    assert torch.allclose(out.float(), O.flash_attn_fwd(q, k, v, causal=False).float(), **TOL16)


@pytest.mark.parametrize("bm,bn", [(64, 64), (128, 32), (32, 128)])
def test_block_causal_mode_of_the_reference_program(cuda_device, bm, bn):
    g = gen(bm + bn)
    q, k, v = (torch.randn(1, 512, 2, 128, generator=g).to(BF) for _ in range(3))
    out = run(q, k, v, cuda_device, causal="block", block_m=bm, block_n=bn)
    assert torch.allclose(out.float(), block_causal_ref(q, k, v, bm, bn).float(), **TOL16)
    small = tuple(torch.randn(1, 8, 2, 8, generator=g).to(BF) for _ in range(3))     # FMA kernel
    out = run(*small, cuda_device, causal="block", block_m=2, block_n=2)
    assert torch.allclose(out.float(), block_causal_ref(*small, 2, 2).float(), **TOL16)


def test_large_scores_exercise_the_rescale_path(cuda_device):
    # keys whose scores grow along the sequence force the running maximum up by more than 2^8
    g = gen(9)
    s, d = 1024, 128
    q = torch.ones(1, s, 1, d).to(BF)
    k = (torch.arange(s).float()[:, None] / s * 4.0 * torch.ones(1, d)).view(1, s, 1, d).to(BF)
    v = torch.randn(1, s, 1, d, generator=g).to(BF)
    for causal in (False, True):
        out = run(q, k, v, cuda_device, causal=causal)
        assert torch.allclose(out.float(), O.flash_attn_fwd(q, k, v, causal=causal).float(), **TOL16)


def test_benchmark_config_properties(cuda_device):
    """B4 H32 S4096 D128 causal bf16: oracle on a slice of heads, plus size-independent
    properties on everything (row 0 copies v[0]; outputs are convex combinations of V rows)."""
    g = gen(4)
    b, s, h, d = 4, 4096, 32, 128
    q, k, v = (torch.randn(b, s, h, d, generator=g).to(BF) for _ in range(3))
    out = run(q, k, v, cuda_device, causal=True)
    assert torch.equal(out[:, 0], v[:, 0])
    vmax = v.float().cummax(dim=1).values
    vmin = v.float().cummin(dim=1).values
    assert (out.float() <= vmax + 2e-2).all() and (out.float() >= vmin - 2e-2).all()
    # the oracle on one whole head of every batch entry ...
    for bi, hi in enumerate((5, 0, 31, 18)):
        sel = (slice(bi, bi + 1), slice(None), slice(hi, hi + 1))
        ref = O.flash_attn_fwd(q[sel], k[sel], v[sel], causal=True, head_chunk=1)
        assert torch.allclose(out[sel].float(), ref.float(), **TOL16), (bi, hi)
    # ... and on the first and the last 256 query rows of EVERY (batch, head): the shortest and the
    # longest rows of work of each one (first CTA scheduled last, last CTA scheduled first)
    ref = O.flash_attn_fwd(q[:, :256], k[:, :256], v[:, :256], causal=True)
    assert torch.allclose(out[:, :256].float(), ref.float(), **TOL16)
    ref = O.flash_attn_fwd(q[:, s - 256:], k, v, causal=True, q_offset=s - 256)
    assert torch.allclose(out[:, s - 256:].float(), ref.float(), **TOL16)


def test_run_to_run_determinism(cuda_device):
    g = gen(6)
    q, k, v = (torch.randn(2, 512, 4, 128, generator=g).to(BF) for _ in range(3))
    a = run(q, k, v, cuda_device, causal=True)
    for _ in range(3):
        assert torch.equal(run(q, k, v, cuda_device, causal=True).view(torch.int16), a.view(torch.int16))


def test_mla_dense_golden_and_fp16(cuda_device):
    g = load_golden("mla_dense_fp32")
    q, qpe = g["q"].transpose(1, 2).contiguous(), g["qpe"].transpose(1, 2).contiguous()
    out = torch.zeros_like(q, device=cuda_device)
    ops.mla_decode_dense(q.to(cuda_device), qpe.to(cuda_device), g["kv"].to(cuda_device), g["kpe"].to(cuda_device), out)
    assert torch.allclose(out.cpu(), g["ref"].transpose(1, 2), atol=1e-5, rtol=1e-4)
    qh, qph, kvh, kph = (t.half() for t in (q, qpe, g["kv"], g["kpe"]))
    outh = torch.zeros_like(qh, device=cuda_device)
    ops.mla_decode_dense(qh.to(cuda_device), qph.to(cuda_device), kvh.to(cuda_device), kph.to(cuda_device), outh)
    ref = O.mla_decode_dense(qh, qph, kvh, kph)
    assert torch.allclose(outh.cpu().float(), ref.float(), atol=5e-2, rtol=5e-2)    # tolerance of check_mla_decode.py
    assert torch.allclose(outh.cpu().float(), ref.float(), **TOL16)


@pytest.mark.parametrize("dtype", [BF, torch.float16])
@pytest.mark.parametrize("batch,heads,seq", [(4, 128, 777), (2, 64, 64), (1, 128, 4096), (3, 20, 130)])
def test_mla_dense_program_at_the_deepseek_shape_runs_on_tensor_cores(cuda_device, dtype, batch, heads, seq):
    """The reference's MLA program (tpu_demo/ppl/deepseek_mla/mla_decode.py:9-121: Q, Q_pe, KV, K_pe as four tensors,
    dense cache) with latent 512 + rope 64: the tcgen05 kernel, the cache addressed without a page table."""
    g = gen(batch * 7 + heads)
    q = torch.randn(batch, heads, 1, 512, generator=g).to(dtype)
    qpe = torch.randn(batch, heads, 1, 64, generator=g).to(dtype)
    kv = torch.randn(batch, seq, 1, 512, generator=g).to(dtype)
    kpe = torch.randn(batch, seq, 1, 64, generator=g).to(dtype)
    out = torch.full_like(q, float("nan"), device=cuda_device)
    assert ops.mla_decode_dense(q.to(cuda_device), qpe.to(cuda_device), kv.to(cuda_device), kpe.to(cuda_device), out) == 0
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.allclose(out.cpu().float(), O.mla_decode_dense(q, qpe, kv, kpe).float(), **TOL16)


def test_argument_errors(cuda_device):
    q = torch.zeros(1, 128, 2, 64, dtype=BF, device=cuda_device)
    with pytest.raises(ValueError):
        ops.flash_attn_fwd(q, q[:, :, :1], q[:, :, :1], q)
    with pytest.raises(RuntimeError, match="seq_q == seq_kv"):
        ops.flash_attn_fwd(q, torch.zeros(1, 64, 2, 64, dtype=BF, device=cuda_device),
                           torch.zeros(1, 64, 2, 64, dtype=BF, device=cuda_device), q, causal=True)
    with pytest.raises(RuntimeError, match="block sizes"):
        ops.flash_attn_fwd(q, q, q, q, causal="block")
