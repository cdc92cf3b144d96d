"""CPU restatement of the reference's operator semantics.  TEST INFRASTRUCTURE ONLY.

Nothing shipped may import this package: it is used by tests/, by the smoke check and by the
CPU-baseline legs of bench.py as the checker, never as the thing measured or shipped.

What it restates.  The arithmetic of the reference's `T.ppl_*` path lives in SOPHGO's closed
BM1690 runtime ("PPL version <= 1.4.195", README.md:40), which is not part of the reference tree
and cannot be installed offline.  The reference validates every program against a torch/numpy
function written in the demo script itself; those functions are what this module follows, one
function per program, each citing the lines it restates.  Pin status: the restatements are
checked against vectors produced by executing the reference's own functions (extracted from the
demo files, see tests/golden/make_golden.py); the numerics of the closed `tpu_bdc_*` routines
themselves stay unpinned beyond the demos' stated tolerances.

All functions take and return CPU torch tensors.  Floating-point programs are evaluated in
fp32 on the already-quantised inputs and rounded once to the output dtype, except where the
reference program itself rounds intermediates (RoPE works in the tile dtype throughout).
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F


# ---------------------------------------------------------------------------- matmul
def matmul(a: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype | None = None,
           transpose_b: bool = False) -> torch.Tensor:
    """C = A @ B with fp32 accumulation, rounded to out_dtype.

    Follows tpu_demo/matmul/tpu_test_matmul_fp16.py:45 (`torch.matmul(a, b).half()`) with the
    fp32 accumulate tile of the program itself (C_shared is float32, :20) and of `ppl.gemm`
    (src/target/codegen_ppl.cc:1261-1274).
    """
    out_dtype = out_dtype or a.dtype
    bf = b.float().t() if transpose_b else b.float()
    return (a.float() @ bf).to(out_dtype)


# ---------------------------------------------------------------------------- FP8 GEMM
def per_token_cast_to_fp8(x: torch.Tensor):
    """1x128 activation quantiser, examples/deepseek_deepgemm/example_deepgemm_fp8_2xAcc.py:93-99."""
    assert x.dim() == 2 and x.size(1) % 128 == 0
    m, n = x.shape
    xv = x.view(m, -1, 128)
    amax = xv.abs().float().amax(dim=2).view(m, -1).clamp(1e-4)
    q = (xv * (448.0 / amax.unsqueeze(2))).to(torch.float8_e4m3fn).view(m, n)
    return q, (amax / 448.0).view(m, -1)


def per_block_cast_to_fp8(x: torch.Tensor):
    """128x128 weight quantiser, example_deepgemm_fp8_2xAcc.py:102-112."""
    assert x.dim() == 2
    m, n = x.shape
    mp, np_ = -(-m // 128) * 128, -(-n // 128) * 128
    xp = torch.zeros(mp, np_, dtype=x.dtype)
    xp[:m, :n] = x
    xv = xp.view(-1, 128, np_ // 128, 128)
    amax = xv.abs().float().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
    q = (xv * (448.0 / amax)).to(torch.float8_e4m3fn)
    return q.view_as(xp)[:m, :n].contiguous(), (amax / 448.0).view(xv.size(0), xv.size(2))


def gemm_fp8_blockscale(a8: torch.Tensor, b8: torch.Tensor, sa: torch.Tensor, sb: torch.Tensor,
                        out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """C[M,N] = sum_kb (A8[:,kb]*sa[:,kb]) @ (B8[:,kb]*sb[nb,kb])^T, fp32 accumulate.

    A8 (M,K) e4m3 with sa (M, K/128); B8 (N,K) e4m3 with sb (ceil(N/128), K/128).  Restates the
    kernel of example_deepgemm_fp8_2xAcc.py:66-81 (per-K-block fp32 partial product promoted with
    `scales_a[m,k] * scales_b[n_block,k]`), which is what `ref_deepgemm_fp8` (:115-139) checks
    through torch._scaled_mm on CUDA; this CPU form keeps every partial product in fp32.
    """
    m, k = a8.shape
    n = b8.shape[0]
    kb = k // 128
    af = a8.float().view(m, kb, 128) * sa.float().view(m, kb, 1)
    sb_full = sb.float().repeat_interleave(128, dim=0)[:n]            # (N, K/128)
    bf = b8.float().view(n, kb, 128) * sb_full.view(n, kb, 1)
    return (af.view(m, k) @ bf.view(n, k).t()).to(out_dtype)


# ---------------------------------------------------------------------------- RMSNorm
def rmsnorm(x: torch.Tensor, weight: torch.Tensor | None = None, eps: float = 1e-12) -> torch.Tensor:
    """tpu_demo/rms_norm/rms_norm_bf16.py:51-54 (fp32 math, one cast); numpy form in
    tpu_demo/ppl/rms_norm/rmsnorm/check_rmsnorm.py:5-7.  `weight` and eps=1e-6 are the
    Llama-shaped extension of the benchmark configuration."""
    xf = x.float()
    r = xf / torch.sqrt(torch.mean(xf * xf, dim=1, keepdim=True) + eps)
    if weight is not None:
        r = r * weight.float()
    return r.to(x.dtype)


# ---------------------------------------------------------------------------- RoPE
def make_rope_cos_sin(rows: int, width: int, base: float = 10000.0, pos_start: int = 0,
                      dtype: torch.dtype = torch.bfloat16):
    """Pair-duplicated cos/sin tables, tpu_demo/tpu_test_rope_bf16.py:53-74 (note the reference
    builds frequencies and angles in the table dtype itself)."""
    assert width % 2 == 0
    half = width // 2
    k = torch.arange(half, dtype=dtype)
    inv_freq = (base ** (-2 * k / width)).to(dtype)
    pos = torch.arange(pos_start, pos_start + rows, dtype=dtype).unsqueeze(1)
    theta = pos * inv_freq
    c, s = torch.cos(theta), torch.sin(theta)
    cos = torch.empty(rows, width, dtype=dtype)
    sin = torch.empty(rows, width, dtype=dtype)
    cos[:, 0::2] = c
    cos[:, 1::2] = c
    sin[:, 0::2] = s
    sin[:, 1::2] = s
    return cos.contiguous(), sin.contiguous()


def make_rope_cos_sin_f32(rows: int, width: int, base: float, dtype: torch.dtype = torch.bfloat16):
    """Same layout, but angles computed in fp32 before the cast: positions above 256 are not
    representable in bf16, so long-sequence tables (8192 positions, theta 500000) are built in
    fp32 and rounded once."""
    half = width // 2
    k = torch.arange(half, dtype=torch.float32)
    inv_freq = base ** (-2.0 * k / width)
    theta = torch.arange(rows, dtype=torch.float32).unsqueeze(1) * inv_freq
    c = torch.cos(theta).repeat_interleave(2, dim=1)
    s = torch.sin(theta).repeat_interleave(2, dim=1)
    return c.to(dtype).contiguous(), s.to(dtype).contiguous()


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Interleaved-pair rotation in the tile dtype: every product and the sum are rounded to
    x.dtype, as in `rope_ref_torch` (tpu_demo/tpu_test_rope_bf16.py:76-92) and in the program
    itself (ppl_mul / ppl_mul_C / ppl_rope_add on bf16 tiles, :31-46).  Lane pairing follows
    ppl_rope_add (src/target/codegen_ppl.cc:1809-1848): out[2i] = (x*cos)[2i] + (-x*sin)[2i+1],
    out[2i+1] = (x*cos)[2i+1] + (x*sin)[2i].  x: (..., W); cos/sin: (T, W), each table row
    serving rows/T consecutive rows of x."""
    width = x.shape[-1]
    x2 = x.reshape(-1, width)
    rep = x2.shape[0] // cos.shape[0]
    c = cos.repeat_interleave(rep, dim=0) if rep > 1 else cos
    s = sin.repeat_interleave(rep, dim=0) if rep > 1 else sin
    x_cos = x2 * c
    x_sin = x2 * s
    x_neg_sin = (x2 * -1.0) * s
    out = torch.empty_like(x2)
    out[:, 0::2] = x_cos[:, 0::2] + x_neg_sin[:, 1::2]
    out[:, 1::2] = x_cos[:, 1::2] + x_sin[:, 0::2]
    return out.reshape(x.shape)


# ---------------------------------------------------------------------------- SwiGLU
def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """`b * F.silu(a)` (tpu_demo/tpu_test_swiglu_bf16.py:68) evaluated in fp32 as the program
    does (:36-51, accum_dtype float32), one cast at the end."""
    return (up.float() * F.silu(gate.float())).to(gate.dtype)


# ---------------------------------------------------------------------------- gated MLP
def mlp_gate_up(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) with the roundings of the MLP program
    (tpu_demo/ppl/mlp/mlp_bf16.py:103-125): both `ppl_gemm`s deliver tiles of the input dtype
    (:103, :113), SiLU = g / (exp(-g) + 1) and the product run in fp32 (:44-54, :118), and the
    product is cast back (:121).  The reference has no check function for this program; this is
    the composition of `matmul` and `swiglu`, which are pinned to theirs."""
    return swiglu(matmul(x, w_gate, transpose_b=True), matmul(x, w_up, transpose_b=True))


def mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """The whole tile program: down projection of `mlp_gate_up` (mlp_bf16.py:123-128), w_down (hidden, inter)."""
    return matmul(mlp_gate_up(x, w_gate, w_up), w_down, transpose_b=True)


# ---------------------------------------------------------------------------- reductions / elementwise
def reduce_sum(x: torch.Tensor) -> torch.Tensor:
    """tpu_demo/tpu_test_reduce_sum.py:36 — row sum, keepdim; fp32 accumulate, cast back.  Integer tiles
    (int32 / uint32 / int16, accepted by the code generator at src/target/codegen_ppl.cc:1570-1592): the exact
    sum cut to the tile's width (two's complement wrap-around)."""
    if x.dtype in (torch.int32, torch.uint32, torch.int16):
        signed = x.view(torch.int32) if x.dtype == torch.uint32 else x
        total = signed.to(torch.int64).sum(dim=1, keepdim=True)
        if x.dtype == torch.int16:
            return ((total + 2 ** 15) % 2 ** 16 - 2 ** 15).to(torch.int16)
        wrapped = ((total + 2 ** 31) % 2 ** 32 - 2 ** 31).to(torch.int32)
        return wrapped.view(torch.uint32) if x.dtype == torch.uint32 else wrapped
    return x.float().sum(dim=1, keepdim=True).to(x.dtype)


def reduce_max(x: torch.Tensor) -> torch.Tensor:
    """tpu_demo/tpu_test_reduce_max.py:34."""
    return torch.max(x, dim=1, keepdim=True).values


def sigmoid(x: torch.Tensor) -> torch.Tensor:
    """tpu_demo/tpu_test_sigmoid_fp32.py:51."""
    return torch.sigmoid(x.float()).to(x.dtype)


# ---------------------------------------------------------------------------- gather / top-k
def gather_rows(param: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """tpu_demo/tpu_test_gather_fp32.py:39 — `param[idx]`; numpy keeps it a pure byte move."""
    idx = index.view(torch.int32).reshape(-1).numpy().astype(np.int64)
    flat = param.contiguous().view(torch.uint8).reshape(param.shape[0], -1).numpy()
    out = torch.from_numpy(flat[idx].copy())
    return out.view(param.dtype).reshape(len(idx), param.shape[1])


def topk(src: torch.Tensor, k: int, descending: bool = True):
    """Sorted top-k values and int32 positions of each row (tpu_demo/tpu_test_topk_fp32.py:39,
    `torch.topk(largest=True, sorted=True)`).  The reference leaves tie order open (it validates
    positions by value look-up, :52-53); this restatement fixes it: equal values are ordered by
    lower position first, via a stable argsort."""
    a = src.reshape(-1, src.shape[-1]).numpy()
    wide = a.astype(np.float64) if a.dtype.kind == "f" else a.astype(np.int64)   # exact widening
    key = -wide if descending else wide
    order = np.argsort(key, axis=1, kind="stable")[:, :k]
    vals = np.take_along_axis(a, order, axis=1)
    shape = src.shape[:-1] + (k,)
    return (torch.from_numpy(vals.copy()).reshape(shape),
            torch.from_numpy(order.astype(np.int32)).reshape(shape))


# ---------------------------------------------------------------------------- attention
def flash_attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool,
                   head_chunk: int = 4, q_offset: int = 0) -> torch.Tensor:
    """softmax(Q K^T / sqrt(d) [+ tril mask]) V on bshd tensors, fp32, cast to q.dtype.

    Follows `ref_program` of tpu_demo/flashattn/tpu_test_flashattn_bf16.py:171-182 (identical to
    examples/flash_attention/example_mha_fwd_bshd.py:173-184); evaluated a few heads at a time
    so the score matrix of long sequences stays small.  `q_offset` lets a test check a block of query
    rows of a long sequence: row i of `q` then stands at position q_offset + i of the sequence (the
    mask of the full problem restricted to those rows; 0 is the reference function itself).
    """
    b, sq, h, d = q.shape
    sk = k.shape[1]
    out = torch.empty(b, sq, h, d, dtype=q.dtype)
    mask = torch.tril(torch.ones(sq, sk), diagonal=q_offset) == 0 if causal else None
    for h0 in range(0, h, head_chunk):
        hs = slice(h0, min(h, h0 + head_chunk))
        scores = torch.einsum("bqhd,bkhd->bhqk", q[:, :, hs].float(), k[:, :, hs].float())
        scores = scores / math.sqrt(d)
        if causal:
            scores = scores.masked_fill(mask, float("-inf"))
        w = F.softmax(scores, dim=-1)
        out[:, :, hs] = torch.einsum("bhqk,bkhd->bqhd", w, v[:, :, hs].float()).to(q.dtype)
    return out


def mla_decode_dense(q: torch.Tensor, q_pe: torch.Tensor, kv: torch.Tensor, k_pe: torch.Tensor) -> torch.Tensor:
    """Dense-cache MLA decode of the TPU program (tpu_demo/ppl/deepseek_mla/mla_decode.py:9-121):
    Q[b,h,1,dim], Q_pe[b,h,1,pe], KV[b,s,1,dim], K_pe[b,s,1,pe] -> Out[b,h,1,dim];
    scores = (Q.KV^T + Q_pe.K_pe^T) / sqrt(dim+pe), V = KV.  Reference check:
    tpu_demo/ppl/deepseek_mla/check_mla_decode.py:50-75."""
    dim, pe = q.shape[-1], q_pe.shape[-1]
    scale = (1.0 / (dim + pe)) ** 0.5
    qf, qpf = q.float()[:, :, 0], q_pe.float()[:, :, 0]          # (b,h,dim)
    kvf, kpf = kv.float()[:, :, 0], k_pe.float()[:, :, 0]        # (b,s,dim)
    s = (torch.einsum("bhd,bsd->bhs", qf, kvf) + torch.einsum("bhd,bsd->bhs", qpf, kpf)) * scale
    w = F.softmax(s, dim=-1)
    return torch.einsum("bhs,bsd->bhd", w, kvf).unsqueeze(2).to(q.dtype)


def mla_decode_paged(q: torch.Tensor, kv_pages: torch.Tensor, kv_scale: torch.Tensor | None,
                     block_table: torch.Tensor, cache_seqlens: torch.Tensor, dv: int,
                     out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """Paged MLA decode, one query token per sequence.

    q (b, h, d); kv_pages (num_pages, page, d) in any float dtype incl. e4m3; kv_scale
    (num_pages, page) fp32 per-token scale or None; block_table (b, max_pages) int32;
    cache_seqlens (b,) int32.  K = dequantised latent, V = its first dv columns, softmax scale
    1/sqrt(d).  Follows `run_torch_mla` / `scaled_dot_product_attention` of
    examples/deepseek_mla/example_mla_decode_paged.py:259-308 (h_kv = 1, s_q = 1, so its causal
    mask keeps every cached token) applied to the de-quantised cache `fp8.float() * scale[token]`.
    """
    b, h, d = q.shape
    page = kv_pages.shape[1]
    out = torch.empty(b, h, dv, dtype=out_dtype or q.dtype)
    for i in range(b):
        n = int(cache_seqlens[i])
        npg = -(-n // page)
        ids = block_table[i, :npg].long()
        kf = kv_pages[ids].float().reshape(npg * page, d)
        if kv_scale is not None:
            kf = kf * kv_scale[ids].float().reshape(npg * page, 1)
        kf = kf[:n]
        w = (q[i].float() @ kf.t()) / math.sqrt(d)
        w = torch.softmax(w, dim=-1, dtype=torch.float32)
        out[i] = (w @ kf[:, :dv]).to(out.dtype)
    return out


def mla_decode_paged_gqa(q: torch.Tensor, kv_pages: torch.Tensor, block_table: torch.Tensor, cache_seqlens: torch.Tensor,
                         dv: int) -> torch.Tensor:
    """Paged decode with several query tokens per sequence and several kv heads: q (b, s_q, h_q, d), kv_pages
    (num_pages, page, h_kv, d), out (b, s_q, h_q, dv).  Follows `run_torch_mla` / `scaled_dot_product_attention` of
    examples/deepseek_mla/example_mla_decode_paged.py:259-308 with causal=True: kv heads repeated h_q / h_kv times,
    scale 1/sqrt(d), mask tril(diagonal = s_k - s_q) (query token i sees keys up to len - s_q + i), V = first dv
    columns; the keys of a sequence are gathered through its page list."""
    b, s_q, h_q, d = q.shape
    page, h_kv = kv_pages.shape[1], kv_pages.shape[2]
    out = torch.zeros(b, s_q, h_q, dv, dtype=q.dtype)
    for i in range(b):
        n = int(cache_seqlens[i])
        if n == 0:
            continue
        npg = -(-n // page)
        k = kv_pages[block_table[i, :npg].long()].float().reshape(npg * page, h_kv, d)[:n]       # (n, h_kv, d)
        k = k.transpose(0, 1).repeat_interleave(h_q // h_kv, dim=0)                              # (h_q, n, d)
        w = q[i].float().transpose(0, 1) @ k.transpose(-2, -1) / math.sqrt(d)                    # (h_q, s_q, n)
        keep = torch.ones(s_q, n, dtype=torch.bool).tril(diagonal=n - s_q)
        w = w.masked_fill(~keep, float("-inf"))
        w = torch.softmax(w, dim=-1, dtype=torch.float32)
        w = torch.nan_to_num(w)                        # a query token that sees no key at all gives zeros
        out[i] = (w @ k[..., :dv]).transpose(0, 1).to(q.dtype)
    return out
