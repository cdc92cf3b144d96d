"""Seeded synthetic inputs for the benchmark configurations.

The reference's demos draw their inputs with `torch.randn` (e.g.
tpu_demo/rms_norm/rms_norm_bf16.py:42); there is no dataset on this path.  Inputs are generated
on the CPU in fp32 from a seeded generator and cast, so a CPU checker and the GPU see the same
bits.  Role comparable to the reference's tensor supply (tilelang/utils/tensor.py).
"""
from __future__ import annotations

import torch


def _gen(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed)


def rope_tables(positions: int, width: int, theta: float, dtype=torch.bfloat16):
    """Pair-duplicated cos/sin tables (layout of make_rope_cos_sin,
    tpu_demo/tpu_test_rope_bf16.py:53-74) with angles evaluated in fp32 and rounded once."""
    half = width // 2
    k = torch.arange(half, dtype=torch.float32)
    inv_freq = theta ** (-2.0 * k / width)
    ang = torch.arange(positions, dtype=torch.float32).unsqueeze(1) * inv_freq
    cos = torch.cos(ang).repeat_interleave(2, dim=1).to(dtype).contiguous()
    sin = torch.sin(ang).repeat_interleave(2, dim=1).to(dtype).contiguous()
    return cos, sin


def llama8b_memory_ops(tokens: int = 8192, hidden: int = 4096, q_heads: int = 32, kv_heads: int = 8,
                       head_dim: int = 128, ffn: int = 14336, theta: float = 500000.0, seed: int = 1,
                       dtype=torch.bfloat16) -> dict:
    """Llama-3-8B memory-bound operators at `tokens` tokens: RMSNorm over `hidden` (weight
    1+0.02*N(0,1), eps 1e-6), RoPE on Q[tokens,q_heads,head_dim] and K[tokens,kv_heads,head_dim]
    (positions 0..tokens-1), SwiGLU on [tokens, ffn]."""
    g = _gen(seed)
    w = {}
    w["x"] = torch.randn(tokens, hidden, generator=g).to(dtype)
    w["weight"] = (1.0 + 0.02 * torch.randn(hidden, generator=g)).to(dtype)
    w["eps"] = 1e-6
    w["q"] = torch.randn(tokens, q_heads, head_dim, generator=g).to(dtype)
    w["k"] = torch.randn(tokens, kv_heads, head_dim, generator=g).to(dtype)
    w["cos"], w["sin"] = rope_tables(tokens, head_dim, theta, dtype)
    w["gate"] = torch.randn(tokens, ffn, generator=g).to(dtype)
    w["up"] = torch.randn(tokens, ffn, generator=g).to(dtype)
    return w


def llama8b_algorithmic_bytes(tokens: int = 8192, hidden: int = 4096, q_heads: int = 32, kv_heads: int = 8,
                              head_dim: int = 128, ffn: int = 14336, elem: int = 2) -> dict:
    """Bytes each operator must move at least once (inputs read once, outputs written once)."""
    return {
        "rmsnorm": 2 * tokens * hidden * elem + hidden * elem,
        "rope": 2 * tokens * (q_heads + kv_heads) * head_dim * elem + 2 * tokens * head_dim * elem,
        "swiglu": 3 * tokens * ffn * elem,
    }


def quantise_tokens_e4m3(x: torch.Tensor):
    """One fp32 scale per token over all its columns: scale = amax / 448 (clamped), bytes = e4m3(x / scale)."""
    amax = x.abs().amax(dim=-1, keepdim=True).clamp(min=1e-4)
    scale = amax / 448.0
    return (x / scale).to(torch.float8_e4m3fn), scale.squeeze(-1).float()


def mla_fp8_paged(batch: int = 128, heads: int = 128, d: int = 576, dv: int = 512, page_size: int = 64,
                  min_len: int = 1024, max_len: int = 8192, seed: int = 3, spare_pages: int = 8,
                  dtype=torch.bfloat16) -> dict:
    """FP8 MLA paged decode at DeepSeek-V3 shape: one query token per sequence, latent KV cache in
    e4m3 with one fp32 scale per token, pages of `page_size` tokens assigned by a random
    permutation, sequence lengths uniform in [min_len, max_len]."""
    g = _gen(seed)
    lens = torch.randint(min_len, max_len + 1, (batch,), generator=g, dtype=torch.int32)
    pages_per_seq = (lens + page_size - 1) // page_size
    total_pages = int(pages_per_seq.sum()) + spare_pages
    max_pages = (max_len + page_size - 1) // page_size
    perm = torch.randperm(total_pages, generator=g).to(torch.int32)
    table = torch.zeros(batch, max_pages, dtype=torch.int32)
    cursor = 0
    for b in range(batch):
        n = int(pages_per_seq[b])
        table[b, :n] = perm[cursor:cursor + n]
        cursor += n
    cache = torch.empty(total_pages, page_size, d, dtype=torch.float8_e4m3fn)
    scale = torch.empty(total_pages, page_size, dtype=torch.float32)
    step = 512
    for p0 in range(0, total_pages, step):                      # bounded fp32 staging
        p1 = min(total_pages, p0 + step)
        c8, sc = quantise_tokens_e4m3(torch.randn(p1 - p0, page_size, d, generator=g))
        cache[p0:p1] = c8
        scale[p0:p1] = sc
    q = torch.randn(batch, 1, heads, d, generator=g).to(dtype)
    return {"q": q, "kv_cache": cache, "kv_scale": scale, "block_table": table, "cache_seqlens": lens, "dv": dv,
            "softmax_scale": d ** -0.5, "total_tokens": int(lens.sum())}
