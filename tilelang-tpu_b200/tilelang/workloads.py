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
