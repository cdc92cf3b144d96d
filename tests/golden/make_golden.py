"""Generate tests/golden/*.npz by EXECUTING the reference's own check functions.

The reference's demo scripts cannot be imported (they build TPU kernels at import time and need
the SOPHGO toolchain), but each of them carries the torch/numpy function or statements it
validates its kernel against.  This script lifts exactly those definitions / statements out of
the files with `ast` (no reference source is copied into this repository), runs them on seeded
inputs in this process, and stores inputs and outputs.  tests/test_oracle_golden.py then pins
oracle/ops.py to these vectors.

Run from the repository root, with the reference tree available:
    python tests/golden/make_golden.py /path/to/reference
16-bit tensors are stored as uint16 bit patterns, e4m3 as uint8.
"""
from __future__ import annotations

import ast
import math
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

import os
_args = [a for a in sys.argv[1:] if not a.startswith("--")]
if not _args and "TILELANG_TPU_REFERENCE" not in os.environ:
    raise SystemExit("usage: make_golden.py /path/to/reference   (or set TILELANG_TPU_REFERENCE)")
REF = Path(_args[0] if _args else os.environ["TILELANG_TPU_REFERENCE"])
OUT_OVERRIDE = os.environ.get("TILELANG_TPU_GOLDEN_OUT")
OUT = Path(OUT_OVERRIDE) if OUT_OVERRIDE else Path(__file__).resolve().parent


def lift(path: str, funcs=(), assigns=(), env=None):
    """Exec the named top-level function defs and the top-level assignments to `assigns`
    (in file order) from a reference file, inside `env`; returns env."""
    src = (REF / path).read_text()
    tree = ast.parse(src)
    env = dict(env or {})
    env.setdefault("torch", torch)
    env.setdefault("F", F)
    env.setdefault("math", math)
    env.setdefault("np", np)
    from typing import Tuple
    env.setdefault("Tuple", Tuple)
    picked = []
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in funcs:
            picked.append(node)
        elif isinstance(node, ast.Assign) and any(
                isinstance(n, ast.Name) and n.id in assigns
                for t in node.targets for n in ast.walk(t)):
            picked.append(node)
    found = {n.name for n in picked if isinstance(n, ast.FunctionDef)}
    missing = set(funcs) - found
    if missing:
        raise RuntimeError(f"{path}: did not find {missing}")
    code = compile(ast.Module(body=picked, type_ignores=[]), str(REF / path), "exec")
    exec(code, env)
    return env


def bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.uint16).numpy()
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def save(name: str, **arrays):
    np.savez_compressed(OUT / f"{name}.npz", **{k: bits(v) if isinstance(v, torch.Tensor) else v
                                                for k, v in arrays.items()})
    print("wrote", name, {k: tuple(np.shape(v)) for k, v in arrays.items()})


def gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def main():
    # ---- matmul: `ref = torch.matmul(a, b).half()` (tpu_test_matmul_fp16.py) --------------
    g = gen(100)
    a = torch.randn(64, 64, generator=g).half()
    b = torch.randn(64, 64, generator=g).half()
    env = lift("tpu_demo/matmul/tpu_test_matmul_fp16.py", assigns=("ref",), env={"a": a, "b": b})
    save("matmul_fp16", a=a, b=b, ref=env["ref"])
    a = torch.randn(64, 64, generator=g).bfloat16()
    b = torch.randn(64, 64, generator=g).bfloat16()
    env = lift("tpu_demo/matmul/tpu_test_matmul_bf16.py", assigns=("ref",), env={"a": a, "b": b})
    save("matmul_bf16", a=a, b=b, ref=env["ref"])

    # ---- rmsnorm: module-level statements of rms_norm_bf16.py ----------------------------
    a = torch.randn(128, 128, generator=gen(101)).bfloat16()
    env = lift("tpu_demo/rms_norm/rms_norm_bf16.py", assigns=("eps", "a_fp32", "ref_fp32", "ref"),
               env={"a": a})
    save("rmsnorm_bf16", a=a, ref=env["ref"], eps=np.float64(env["eps"]))

    # ---- rope: make_rope_cos_sin + rope_ref_torch ------------------------------------------
    env = lift("tpu_demo/tpu_test_rope_bf16.py", funcs=("make_rope_cos_sin", "rope_ref_torch"))
    x = torch.randn(128, 64, generator=gen(102)).bfloat16()
    cos, sin = env["make_rope_cos_sin"](128, 64, device="cpu", dtype=torch.bfloat16)
    ref = env["rope_ref_torch"](x, cos, sin).bfloat16()
    save("rope_bf16", x=x, cos=cos, sin=sin, ref=ref)
    x32 = torch.randn(128, 64, generator=gen(103))
    cos32, sin32 = env["make_rope_cos_sin"](128, 64, device="cpu", dtype=torch.float32)
    save("rope_fp32", x=x32, cos=cos32, sin=sin32, ref=env["rope_ref_torch"](x32, cos32, sin32))

    # ---- swiglu: `ref = b * F.silu(a)` -----------------------------------------------------
    g = gen(104)
    a = torch.randn(64, 64, generator=g, dtype=torch.float32).bfloat16()
    b = torch.randn(64, 64, generator=g, dtype=torch.float32).bfloat16()
    env = lift("tpu_demo/tpu_test_swiglu_bf16.py", assigns=("ref",), env={"a": a, "b": b})
    save("swiglu_bf16", a=a, b=b, ref=env["ref"])

    # ---- reductions ------------------------------------------------------------------------
    x = torch.randn(64, 64, generator=gen(105)).half()
    env = lift("tpu_demo/tpu_test_reduce_sum.py", assigns=("y_torch",), env={"x": x})
    save("reduce_sum_fp16", x=x, ref=env["y_torch"])
    env = lift("tpu_demo/tpu_test_reduce_max.py", assigns=("y_torch",), env={"x": x})
    save("reduce_max_fp16", x=x, ref=env["y_torch"])

    # ---- top-k / gather ---------------------------------------------------------------------
    src = torch.randn(1024, generator=gen(106)).float()
    env = lift("tpu_demo/tpu_test_topk_fp32.py", assigns=("ref_vals", "ref_idx"), env={"src": src, "K": 8})
    save("topk_fp32", src=src, ref_vals=env["ref_vals"], ref_idx=env["ref_idx"].to(torch.int32))
    g = gen(107)
    param = torch.randn(128, 64, generator=g).float()
    idx_vals = torch.randint(0, 128, (8, 1), generator=g, dtype=torch.int32)
    env = lift("tpu_demo/tpu_test_gather_fp32.py", assigns=("ref",), env={"param": param, "idx_vals": idx_vals})
    save("gather_fp32", param=param, index=idx_vals, ref=env["ref"])

    # ---- sigmoid ----------------------------------------------------------------------------
    a = torch.randn(64, 64, generator=gen(108)).float()
    save("sigmoid_fp32", a=a, ref=torch.sigmoid(a).float())   # tpu_test_sigmoid_fp32.py:51, inside main()

    # ---- flash attention: ref_program, causal and not ---------------------------------------
    env = lift("tpu_demo/flashattn/tpu_test_flashattn_bf16.py", funcs=("ref_program",))
    g = gen(109)
    q = torch.randn(2, 96, 3, 32, generator=g).bfloat16()
    k = torch.randn(2, 96, 3, 32, generator=g).bfloat16()
    v = torch.randn(2, 96, 3, 32, generator=g).bfloat16()
    save("flash_attn_bf16", q=q, k=k, v=v, ref_full=env["ref_program"](q, k, v, False),
         ref_causal=env["ref_program"](q, k, v, True))

    # ---- dense MLA decode: ref_program of check_mla_decode.py -------------------------------
    dim, pe_dim = 32, 4
    env = lift("tpu_demo/ppl/deepseek_mla/check_mla_decode.py", funcs=("ref_program",),
               env={"dim": dim, "pe_dim": pe_dim})
    g = gen(110)
    q = torch.randn(4, 1, 8, dim, generator=g)
    qpe = torch.randn(4, 1, 8, pe_dim, generator=g)
    kv = torch.randn(4, 512, 1, dim, generator=g)
    kpe = torch.randn(4, 512, 1, pe_dim, generator=g)
    # the reference's einsum 'bhqk,bkhd->bqhd' needs matching head counts: expand the single kv head
    ref = env["ref_program"](q, qpe, kv.expand(-1, -1, 8, -1), kpe.expand(-1, -1, 8, -1), False)
    save("mla_dense_fp32", q=q, qpe=qpe, kv=kv, kpe=kpe, ref=ref)

    # ---- paged MLA decode: run_torch_mla ----------------------------------------------------
    env = lift("examples/deepseek_mla/example_mla_decode_paged.py",
               funcs=("scaled_dot_product_attention", "run_torch_mla"))
    b, h_q, h_kv, d, dv, page = 3, 16, 1, 96, 64, 16
    g = gen(111)
    cache_seqlens = torch.tensor([40, 64, 23], dtype=torch.int32)
    max_seqlen_pad = 64
    qq = torch.randn(b, 1, h_q, d, generator=g).half()
    block_table = torch.arange(b * max_seqlen_pad // page, dtype=torch.int32).view(b, max_seqlen_pad // page)
    blocked_k = torch.randn(block_table.numel(), page, h_kv, d, generator=g).half()
    ref = env["run_torch_mla"](qq, block_table, blocked_k, max_seqlen_pad, page, b, 1, cache_seqlens,
                               h_q, h_kv, d, dv, True, torch.float16)
    save("mla_paged_fp16", q=qq, block_table=block_table, blocked_k=blocked_k,
         cache_seqlens=cache_seqlens, ref=ref, dv=np.int64(dv))

    # ---- FP8 quantisers of the block-scaled GEMM example --------------------------------------
    env = lift("examples/deepseek_deepgemm/example_deepgemm_fp8_2xAcc.py",
               funcs=("ceildiv", "per_token_cast_to_fp8", "per_block_cast_to_fp8"))
    g = gen(112)
    xa = torch.randn(128, 256, generator=g) * 0.05
    xb = torch.randn(192, 256, generator=g) * 0.05
    a8, sa = env["per_token_cast_to_fp8"](xa)
    b8, sb = env["per_block_cast_to_fp8"](xb)
    save("fp8_quant", xa=xa, xb=xb, a8=a8, sa=sa, b8=b8, sb=sb)
    fp8_gemm_reference(env)


def fp8_gemm_reference(env=None):
    """`ref_deepgemm_fp8` (example_deepgemm_fp8_2xAcc.py:115-139) calls torch._scaled_mm with row-wise
    scales on "cuda", which torch's CPU backend does not implement: this fixture is written only when
    the script runs on a machine with a CUDA device (`--only-fp8-gemm` skips everything else)."""
    if not torch.cuda.is_available():
        print("fp8_gemm_ref.npz not refreshed: ref_deepgemm_fp8 needs torch._scaled_mm on a CUDA device")
        return
    env = lift("examples/deepseek_deepgemm/example_deepgemm_fp8_2xAcc.py",
               funcs=("ceildiv", "per_token_cast_to_fp8", "per_block_cast_to_fp8", "ref_deepgemm_fp8"))
    g = gen(113)
    m, n, k = 256, 384, 1024
    xa = (torch.randn(m, k, generator=g) * 0.05).cuda()
    xb = (torch.randn(n, k, generator=g) * 0.05).cuda()
    a8, sa = env["per_token_cast_to_fp8"](xa)
    b8, sb = env["per_block_cast_to_fp8"](xb)
    ref = env["ref_deepgemm_fp8"](a8, b8, sa, sb, torch.bfloat16)
    save("fp8_gemm_ref", a8=a8.cpu(), sa=sa.cpu(), b8=b8.cpu(), sb=sb.cpu(), ref=ref.cpu())


if __name__ == "__main__":
    if "--only-fp8-gemm" in sys.argv:
        sys.argv.remove("--only-fp8-gemm")
        fp8_gemm_reference()
    else:
        main()
