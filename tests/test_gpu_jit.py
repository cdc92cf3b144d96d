"""`tilelang.compile(...)` end to end on the GPU: the reference's call convention (all
parameters passed, outputs in place, int status) with host tensors and with device tensors."""
import pytest
import torch

import oracle.ops as O
import tilelang
import tilelang.language as T
from test_frontend import (matmul_program, mlp_program, rms_norm_program, rms_norm_program_f32, swiglu_program_f32,
                           topk_program)

pytestmark = pytest.mark.gpu


def gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def test_rmsnorm_program_host_tensors_like_the_demo(cuda_device):
    kernel = tilelang.compile(rms_norm_program(128, 128, 32), out_idx=-1, target="b200")
    a = torch.randn(128, 128, generator=gen(1)).bfloat16()
    b = torch.zeros(128, 128).bfloat16()
    res = kernel(a, b)                      # host tensors, result written into b
    assert res == 0
    ref = O.rmsnorm(a, eps=1e-12)
    assert torch.allclose(b.float(), ref.float(), atol=5e-2, rtol=5e-2)      # the demo's tolerance
    assert torch.allclose(b.float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_rmsnorm_program_device_tensors_and_pinned_host(cuda_device):
    kernel = tilelang.compile(rms_norm_program(256, 512, 32, eps=1e-6), out_idx=-1, target="b200")
    a = torch.randn(256, 512, generator=gen(2)).bfloat16()
    ref = O.rmsnorm(a, eps=1e-6)
    bd = torch.zeros(256, 512, dtype=torch.bfloat16, device=cuda_device)
    assert kernel(a.to(cuda_device), bd) == 0
    assert torch.allclose(bd.cpu().float(), ref.float(), atol=2e-2, rtol=2e-2)
    bp = torch.zeros(256, 512, dtype=torch.bfloat16).pin_memory()
    assert kernel(a.pin_memory(), bp) == 0
    assert torch.equal(bp, bd.cpu())


@pytest.mark.parametrize("trans_b,bk", [(False, 32), (True, 64), (True, 32)])
def test_matmul_program(cuda_device, trans_b, bk):
    kernel = tilelang.compile(matmul_program(64, 64, 64, 32, 32, bk, trans_b=trans_b), out_idx=-1, target="b200")
    g = gen(3)
    a = torch.randn(64, 64, generator=g).half()
    b = torch.randn(64, 64, generator=g).half()
    c = torch.zeros(64, 64).half()
    assert kernel(a, b, c) == 0
    if trans_b and bk < 64:
        # `C = A B^T` overwrites C on every K iteration in the reference's generated code
        # (src/target/codegen_ppl.cc:1276-1279): what is left is the product over the last K tile
        assert kernel.adapter.bound.program == "generic"
        ref = O.matmul(a[:, -bk:].contiguous(), b[:, -bk:].contiguous(), transpose_b=True)
    else:
        assert kernel.adapter.bound.program == "matmul"
        ref = O.matmul(a, b, transpose_b=trans_b)
    assert torch.allclose(c, ref, atol=1e-2, rtol=1e-2)                      # the demo's tolerance


def test_matmul_anchor_program_1024(cuda_device):
    kernel = tilelang.compile(matmul_program(1024, 1024, 1024, 128, 128, 64), out_idx=-1, target="b200")
    g = gen(0)
    a = torch.randn(1024, 1024, generator=g).half()
    b = torch.randn(1024, 1024, generator=g).half()
    c = torch.zeros(1024, 1024).half()
    assert kernel(a, b, c) == 0
    ref = O.matmul(a, b)
    assert torch.allclose(c.float(), ref.float(), atol=2e-2, rtol=2e-2)          # the stated tolerance


def test_topk_program_two_outputs(cuda_device):
    kernel = tilelang.compile(topk_program(1024, 8), out_idx=[1, 2], target="b200")
    src = torch.randn(1024, generator=gen(4))
    out = torch.zeros(1024)
    idx = torch.zeros(1024, dtype=torch.int32)
    assert kernel(src, out, idx) == 0
    rv, ri = torch.topk(src, 8, largest=True, sorted=True)
    assert torch.equal(idx[:8].long(), ri) and torch.equal(out[:8], rv)
    assert torch.allclose(src[idx[:8].long()], rv, atol=1e-5)               # the demo's look-up check


def test_gather_program_uint32_index(cuda_device):
    @T.prim_func
    def main_kernel_inner(Param: T.Tensor((128, 64), "float32"), Index: T.Tensor((8, 1), "uint32"),
                          Output: T.Tensor((8, 64), "float32")):
        with T.Kernel(1, 1, is_cpu=True) as (bx, by):
            T.ppl_gather(Output, Param, Index, 128)

    kernel = tilelang.compile(main_kernel_inner, out_idx=-1, target="b200")
    g = gen(5)
    param = torch.randn(128, 64, generator=g)
    idx_vals = torch.randint(0, 128, (8, 1), generator=g, dtype=torch.int32)
    out = torch.zeros(8, 64)
    assert kernel(param, idx_vals.view(torch.uint32), out) == 0
    assert torch.equal(out, param[idx_vals.view(-1)])


def test_profiler_consistency_and_bench(cuda_device):
    kernel = tilelang.compile(rms_norm_program(512, 1024, 32), out_idx=-1, target="b200")
    prof = kernel.get_profiler()
    prof.assert_consistent(repeat=3)
    assert prof.do_bench(rep=3) > 0


def test_mlp_program(cuda_device):
    """Output first in the parameter list, as in the reference's MLP program."""
    rows, hidden, inter = 128, 256, 512
    kernel = tilelang.compile(mlp_program(rows, hidden, inter, 64), out_idx=0, target="b200")
    g = gen(8)
    x = torch.randn(rows, hidden, generator=g).bfloat16()
    wg = (torch.randn(inter, hidden, generator=g) / hidden ** 0.5).bfloat16()
    wu = (torch.randn(inter, hidden, generator=g) / hidden ** 0.5).bfloat16()
    wd = (torch.randn(hidden, inter, generator=g) / inter ** 0.5).bfloat16()
    y = torch.zeros(rows, hidden).bfloat16()
    assert kernel(y, x, wg, wu, wd) == 0
    assert torch.allclose(y.float(), O.mlp(x, wg, wu, wd).float(), atol=2e-2, rtol=2e-2)


def test_float32_program_forms(cuda_device):
    g = gen(9)
    x = torch.randn(64, 128, generator=g)
    y = torch.zeros(64, 128)
    assert tilelang.compile(rms_norm_program_f32(64, 128, 32, eps=1e-6), out_idx=-1, target="b200")(x, y) == 0
    assert torch.allclose(y, O.rmsnorm(x, eps=1e-6), atol=1e-5, rtol=1e-5)
    gate, up = torch.randn(64, 128, generator=g), torch.randn(64, 128, generator=g)
    out = torch.zeros(64, 128)
    assert tilelang.compile(swiglu_program_f32(64, 128, 32, 64), out_idx=0, target="b200")(out, gate, up) == 0
    assert torch.allclose(out, O.swiglu(gate, up), atol=1e-5, rtol=1e-5)


# ------------------------------------------------------------------ benchmark programs through the plug-in call
def test_llama_programs_through_the_adapter_equal_the_operator_calls(cuda_device):
    """The programs the end-to-end benchmark compiles (weighted RMSNorm, RoPE with per-token tables shared by
    the heads, SwiGLU), called with pinned host tensors: same bits as `tilelang.ops` on device tensors."""
    from tilelang import ops, programs as P, workloads
    w = workloads.llama8b_memory_ops(tokens=256, seed=11)
    dev = cuda_device
    k_norm = tilelang.compile(P.rmsnorm(256, 4096, eps=w["eps"]), out_idx=-1, target="b200")
    k_rq = tilelang.compile(P.rope(256, 32, 128), out_idx=-1, target="b200")
    k_rk = tilelang.compile(P.rope(256, 8, 128), out_idx=-1, target="b200")
    k_sw = tilelang.compile(P.swiglu(256, 14336), out_idx=-1, target="b200")
    assert [k.adapter.bound.program for k in (k_norm, k_rq, k_rk, k_sw)] == ["rmsnorm", "rope", "rope", "swiglu"]
    pin = lambda t: t.contiguous().pin_memory()                                       # noqa: E731
    hy, hq, hk, hs = (pin(torch.full_like(w[n], float("nan"))) for n in ("x", "q", "k", "gate"))
    for _ in range(3):                    # three calls in flight exercise both buffer sets of every adapter
        assert k_norm(pin(w["x"]), pin(w["weight"].view(1, -1)), hy) == 0
        assert k_rq(pin(w["q"]), pin(w["cos"]), pin(w["sin"]), hq) == 0
        assert k_rk(pin(w["k"]), pin(w["cos"]), pin(w["sin"]), hk) == 0
        assert k_sw(pin(w["gate"]), pin(w["up"]), hs) == 0
    for k in (k_norm, k_rq, k_rk, k_sw):
        k.adapter.synchronize()
    d = {n: v.to(dev) for n, v in w.items() if isinstance(v, torch.Tensor)}
    y, qo, ko, so = (torch.empty_like(d[n]) for n in ("x", "q", "k", "gate"))
    ops.rmsnorm(d["x"], y, d["weight"], eps=w["eps"])
    ops.rope(d["q"], d["cos"], d["sin"], qo)
    ops.rope(d["k"], d["cos"], d["sin"], ko)
    ops.swiglu(d["gate"], d["up"], so)
    for host, devt in ((hy, y), (hq, qo), (hk, ko), (hs, so)):
        assert torch.equal(host.view(torch.int16), devt.cpu().view(torch.int16))
    assert torch.allclose(hy.float(), O.rmsnorm(w["x"], w["weight"], eps=w["eps"]).float(), atol=2e-2, rtol=2e-2)
    assert torch.equal(hq.view(torch.int16), O.rope(w["q"], w["cos"], w["sin"]).view(torch.int16))


def test_a_call_that_reads_what_an_earlier_call_still_writes_waits_for_it(cuda_device):
    """Asynchronous (pinned) calls chained through a host tensor: the second program's upload of `mid` is ordered
    after the first program's download into it, across two adapters."""
    k1 = tilelang.compile(rms_norm_program(256, 512, 32, eps=1e-6), out_idx=-1, target="b200")
    k2 = tilelang.compile(rms_norm_program(256, 512, 64, eps=1e-6), out_idx=-1, target="b200")     # another program: another adapter
    assert k1 is not k2 and k1.adapter is not k2.adapter
    a = torch.randn(256, 512, generator=gen(12)).bfloat16().pin_memory()
    mid = torch.zeros(256, 512, dtype=torch.bfloat16).pin_memory()
    out = torch.zeros(256, 512, dtype=torch.bfloat16).pin_memory()
    assert k1(a, mid) == 0 and k2(mid, out) == 0
    k2.adapter.synchronize()
    ref = O.rmsnorm(O.rmsnorm(a, eps=1e-6), eps=1e-6)
    assert torch.allclose(out.float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_library_programs_fp8_gemm_and_paged_mla(cuda_device):
    """The two benchmark operators without a `ppl_*` form go through the same compile / call convention."""
    from tilelang import ops, programs as P, workloads
    dev = cuda_device
    g = gen(13)
    m, n, k = 256, 384, 512
    a8, sa = O.per_token_cast_to_fp8(torch.randn(m, k, generator=g) * 0.05)
    b8, sb = O.per_block_cast_to_fp8(torch.randn(n, k, generator=g) * 0.05)
    c = torch.zeros(m, n, dtype=torch.bfloat16)
    kern = tilelang.compile(P.gemm_fp8_blockscale(m, n, k), out_idx=-1, target="b200")
    assert kern(a8, b8, sa, sb, c) == 0
    cd = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    ops.gemm_fp8_blockscale(a8.to(dev), b8.to(dev), sa.to(dev), sb.to(dev), cd)
    assert torch.equal(c.view(torch.int16), cd.cpu().view(torch.int16))
    assert torch.allclose(c.float(), O.gemm_fp8_blockscale(a8, b8, sa, sb).float(), atol=2e-2, rtol=2e-2)

    cfg = workloads.mla_fp8_paged(batch=4, heads=128, min_len=100, max_len=700, seed=14)
    pages, page = cfg["kv_cache"].shape[0], cfg["kv_cache"].shape[1]
    prog = P.mla_decode_paged(4, 128, 576, 512, pages, page, cfg["block_table"].shape[1])
    kern = tilelang.compile(prog, out_idx=-1, target="b200")
    out = torch.zeros(4, 1, 128, 512, dtype=torch.bfloat16)
    assert kern(cfg["q"], cfg["kv_cache"].view(pages, page, 1, 576), cfg["kv_scale"], cfg["block_table"],
                cfg["cache_seqlens"], out) == 0
    ref = O.mla_decode_paged(cfg["q"][:, 0], cfg["kv_cache"], cfg["kv_scale"], cfg["block_table"], cfg["cache_seqlens"], 512)
    assert torch.allclose(out[:, 0].float(), ref.float(), atol=2e-2, rtol=2e-2)


def test_library_program_full_mlp(cuda_device):
    """The gated MLP at full size (gate / up GEMM with the SiLU-product as epilogue, then the down GEMM) through the
    compile / call convention, against the oracle's composition of the pinned matmul and swiglu; one shape on one
    CTA per tile, one that gives every pair of SMs a tile (CTA pairs in both launches)."""
    from tilelang import ops, programs as P
    for (m, hidden, inter) in ((256, 384, 512), (2048, 1280, 1536)):
        g = gen(m + hidden)
        x = (torch.randn(m, hidden, generator=g) * 0.5).bfloat16()
        wg, wu = [(torch.randn(inter, hidden, generator=g) * 0.05).bfloat16() for _ in range(2)]
        wd = (torch.randn(hidden, inter, generator=g) * 0.05).bfloat16()
        out = torch.zeros(m, hidden, dtype=torch.bfloat16)
        kern = tilelang.compile(P.mlp(m, hidden, inter), out_idx=0, target="b200")
        assert kern(out, x, wg, wu, wd) == 0
        ref = O.mlp(x, wg, wu, wd)
        assert torch.allclose(out.float(), ref.float(), atol=2e-2, rtol=2e-2)
        # the same two launches by hand give the same bits
        dev = cuda_device
        h = torch.empty(m, inter, dtype=torch.bfloat16, device=dev)
        od = torch.empty(m, hidden, dtype=torch.bfloat16, device=dev)
        ops.mlp_gate_up(x.to(dev), wg.to(dev), wu.to(dev), h)
        ops.gemm(h, wd.to(dev), od, transpose_b=True)
        assert torch.equal(out.view(torch.int16), od.cpu().view(torch.int16))
        assert torch.allclose(h.cpu().float(), O.mlp_gate_up(x, wg, wu).float(), atol=2e-2, rtol=2e-2)


def test_autotuner_and_tile_table(cuda_device, tmp_path, monkeypatch):
    """The tuner times program configurations on the GPU; `tune_gemm` fills the shape -> tile table that
    `ops.gemm` reads, and the result does not depend on the tile."""
    from tilelang import cache, ops
    from tilelang.autotuner import AutoTuner, product_configs, tune_gemm
    monkeypatch.setenv("TILELANG_B200_CACHE_DIR", str(tmp_path))
    cache.clear_cache(disk=True)
    res = AutoTuner.from_kernel(lambda blk_m: rms_norm_program(256, 512, blk_m, eps=1e-6),
                                product_configs(blk_m=[32, 64, 48])).set_compile_args(
        out_idx=-1, ref_prog=lambda a: O.rmsnorm(a.cpu(), eps=1e-6), rtol=2e-2, atol=2e-2).run(warmup=2, rep=3)
    assert res.config["blk_m"] in (32, 64) and res.latency > 0
    assert [t for t in res.trials if "error" in t][0]["config"] == {"blk_m": 48}       # 48 does not divide 256
    choice = tune_gemm(512, 1024, 256, torch.bfloat16, warmup=1, rep=2)
    assert choice["tile_n"] in (64, 128, 256, 512)          # 512: 256 x 256 tiles on CTA pairs
    assert cache.tile_choice("gemm", m=512, n=1024, k=256, dtype="torch.bfloat16", transpose_b=False)["tile_n"] == choice["tile_n"]
    g = gen(21)
    a = torch.randn(512, 256, generator=g).bfloat16().to(cuda_device)
    b = torch.randn(256, 1024, generator=g).bfloat16().to(cuda_device)
    outs = []
    for t in (0, 64, 128, 256, 512, None):
        c = torch.zeros(512, 1024, dtype=torch.bfloat16, device=cuda_device)
        ops.gemm(a, b, c, tile_n=t)
        outs.append(c)
    assert all(torch.equal(outs[0].view(torch.int16), o.view(torch.int16)) for o in outs[1:])
    cache.clear_cache(disk=True)
