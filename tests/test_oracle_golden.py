"""Pins oracle/ops.py to vectors produced by executing the reference's own check functions
(tests/golden/make_golden.py).  CPU only."""
import torch

import oracle.ops as O
from conftest import load_golden

BF, HF, F8 = torch.bfloat16, torch.float16, torch.float8_e4m3fn


def bit_equal(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.dtype == b.dtype and a.shape == b.shape and torch.equal(
        a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8))


def test_matmul_fp16():
    g = load_golden("matmul_fp16", dict(a=HF, b=HF, ref=HF))
    assert bit_equal(O.matmul(g["a"], g["b"]), g["ref"])


def test_matmul_bf16():
    g = load_golden("matmul_bf16", dict(a=BF, b=BF, ref=BF))
    assert bit_equal(O.matmul(g["a"], g["b"]), g["ref"])


def test_rmsnorm_bf16():
    g = load_golden("rmsnorm_bf16", dict(a=BF, ref=BF))
    assert g["eps"] == 1e-12
    assert bit_equal(O.rmsnorm(g["a"], eps=g["eps"]), g["ref"])


def test_rope_tables_and_rotation_bf16():
    g = load_golden("rope_bf16", dict(x=BF, cos=BF, sin=BF, ref=BF))
    cos, sin = O.make_rope_cos_sin(128, 64, dtype=BF)
    assert bit_equal(cos, g["cos"]) and bit_equal(sin, g["sin"])
    assert bit_equal(O.rope(g["x"], g["cos"], g["sin"]), g["ref"])


def test_rope_fp32():
    g = load_golden("rope_fp32")
    cos, sin = O.make_rope_cos_sin(128, 64, dtype=torch.float32)
    assert bit_equal(cos, g["cos"]) and bit_equal(sin, g["sin"])
    assert bit_equal(O.rope(g["x"], g["cos"], g["sin"]), g["ref"])


def test_swiglu_bf16():
    # The reference check evaluates `b * F.silu(a)` on bf16 tensors (two roundings); the program
    # and the oracle keep fp32 until one final cast.  They agree within the demo's tolerance.
    g = load_golden("swiglu_bf16", dict(a=BF, b=BF, ref=BF))
    out = O.swiglu(g["a"], g["b"])
    assert torch.allclose(out.float(), g["ref"].float(), atol=1e-2, rtol=1e-2)


def test_reductions_fp16():
    g = load_golden("reduce_sum_fp16", dict(x=HF, ref=HF))
    assert torch.allclose(O.reduce_sum(g["x"]).float(), g["ref"].float(), atol=1e-2, rtol=1e-2)
    g = load_golden("reduce_max_fp16", dict(x=HF, ref=HF))
    assert bit_equal(O.reduce_max(g["x"]), g["ref"])


def test_topk_fp32():
    g = load_golden("topk_fp32")
    vals, idx = O.topk(g["src"], 8, descending=True)
    assert bit_equal(vals, g["ref_vals"])
    assert torch.equal(idx, g["ref_idx"])


def test_topk_tie_rule_and_ascending():
    src = torch.tensor([[1.0, 3.0, 3.0, -2.0, 3.0, 0.5]])
    vals, idx = O.topk(src, 4, descending=True)
    assert idx.tolist() == [[1, 2, 4, 0]]
    vals, idx = O.topk(src, 2, descending=False)
    assert idx.tolist() == [[3, 5]] and vals.tolist() == [[-2.0, 0.5]]
    isrc = torch.tensor([5, -7, 5, 2], dtype=torch.int32)
    vals, idx = O.topk(isrc, 3, descending=True)
    assert idx.tolist() == [0, 2, 3] and vals.tolist() == [5, 5, 2]


def test_gather_fp32():
    g = load_golden("gather_fp32")
    assert bit_equal(O.gather_rows(g["param"], g["index"]), g["ref"])


def test_sigmoid_fp32():
    g = load_golden("sigmoid_fp32")
    assert bit_equal(O.sigmoid(g["a"]), g["ref"])


def test_flash_attn_bf16():
    d = dict(q=BF, k=BF, v=BF, ref_full=BF, ref_causal=BF)
    g = load_golden("flash_attn_bf16", d)
    full = O.flash_attn_fwd(g["q"], g["k"], g["v"], causal=False, head_chunk=2)
    causal = O.flash_attn_fwd(g["q"], g["k"], g["v"], causal=True, head_chunk=2)
    # identical formula; chunking over heads may change fp32 summation order by an ulp
    assert torch.allclose(full.float(), g["ref_full"].float(), atol=1e-2, rtol=1e-2)
    assert torch.allclose(causal.float(), g["ref_causal"].float(), atol=1e-2, rtol=1e-2)
    assert (full.float() - g["ref_full"].float()).abs().max() <= 2 ** -7


def test_mla_dense_fp32():
    g = load_golden("mla_dense_fp32")
    # oracle layout is the TPU program's: Q[b,h,1,d]; the check script's is [b,1,h,d]
    out = O.mla_decode_dense(g["q"].transpose(1, 2).contiguous(), g["qpe"].transpose(1, 2).contiguous(),
                             g["kv"], g["kpe"])
    ref = g["ref"].transpose(1, 2)
    assert torch.allclose(out, ref, atol=1e-5, rtol=1e-4)


def test_mla_paged_fp16():
    g = load_golden("mla_paged_fp16", dict(q=HF, blocked_k=HF, ref=HF))
    q = g["q"][:, 0]                                    # (b, h, d)
    pages = g["blocked_k"][:, :, 0]                     # (num_pages, page, d)
    out = O.mla_decode_paged(q, pages, None, g["block_table"], g["cache_seqlens"], int(g["dv"]))
    assert torch.allclose(out.float(), g["ref"][:, 0].float(), atol=2e-3, rtol=2e-3)


def test_fp8_quantisers():
    g = load_golden("fp8_quant", dict(a8=F8, b8=F8))
    a8, sa = O.per_token_cast_to_fp8(g["xa"])
    b8, sb = O.per_block_cast_to_fp8(g["xb"])
    assert bit_equal(a8, g["a8"]) and bit_equal(sa, g["sa"])
    assert bit_equal(b8, g["b8"]) and bit_equal(sb, g["sb"])


def test_fp8_gemm_matches_dequantised_product():
    g = load_golden("fp8_quant", dict(a8=F8, b8=F8))
    c = O.gemm_fp8_blockscale(g["a8"], g["b8"], g["sa"], g["sb"], torch.float32)
    ref = g["xa"] @ g["xb"].t()
    # e4m3 keeps 3 mantissa bits: the quantised product tracks the fp32 one to a few percent
    assert (c - ref).norm() / ref.norm() < 0.05


def test_fp8_gemm_oracle_meets_the_reference_functions_result():
    """`ref_deepgemm_fp8` (examples/deepseek_deepgemm/example_deepgemm_fp8_2xAcc.py:115-139) needs
    torch._scaled_mm with row-wise scales, which only a CUDA device runs; its output on seeded operands was
    recorded there (tests/golden/make_golden.py --only-fp8-gemm).  The oracle keeps every partial in fp32, the
    reference function rounds each 128-wide partial to bf16: they agree within the example's own `diff < 1e-3`."""
    import oracle.ops as O
    from conftest import GOLDEN, load_golden
    import pytest
    import torch
    if not (GOLDEN / "fp8_gemm_ref.npz").exists():
        pytest.skip("fixture not generated (needs a CUDA device and the reference tree)")
    g = load_golden("fp8_gemm_ref", dict(a8=torch.float8_e4m3fn, b8=torch.float8_e4m3fn, ref=torch.bfloat16))
    mine = O.gemm_fp8_blockscale(g["a8"], g["b8"], g["sa"], g["sb"], torch.float32).double()
    ref = g["ref"].double()
    assert float(1 - 2 * (mine * ref).sum() / (mine * mine + ref * ref).sum()) < 1e-3
    assert torch.allclose(mine.float(), ref.float(), atol=2e-2, rtol=2e-2)
