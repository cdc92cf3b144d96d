"""Per-kernel throughput of the tensor-core programs at the benchmark shapes, sharded over the
ranks of one node the way `tilelang/parallel.py` describes (GEMM by N columns, attention by heads, MLA
decode by sequences).  Every kernel writes its block straight into its slot of a rank-major receive
buffer (`parallel.ShardedOutput`), and the ONE in-place all-gather of the outputs is timed separately
(`ms_with_output_gather`); the gathered result is consumed through a zero-copy split view (columns,
heads) or put in order by one row-gather launch (MLA decode, whose sequences are dealt out by length).

Inputs are synthetic and generated on the device (these runs measure speed; parity lives in
tests/).  Work formulas are the reference's own: GEMM 2*M*N*K
(examples/deepseek_deepgemm/example_deepgemm_fp8_2xAcc.py:180), attention 4*B*H*S^2*D, halved
when causal (examples/flash_attention/example_mha_fwd_bshd.py:197-200), MLA decode
2*sum(L)*H*(d+dv) (examples/deepseek_mla/example_mla_decode_paged.py:380).
"""
from __future__ import annotations

import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT / "tilelang-tpu_b200"), str(ROOT)):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from tilelang import ops, parallel  # noqa: E402


_last_call = {}          # the timed callable of the most recent entry (run_all times it again, sustained)


def _time(fn, world, reps=5, warmup=3):
    """ms per call: CUDA events on the current stream, barrier on both sides, max over ranks."""
    _last_call.setdefault("fn", fn)
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / reps], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _sustained(fn, ms_burst, world, rank, seconds=0.6):
    """The same call back to back for about `seconds` (long enough for the power limiter to settle), with the SM clock
    and throttle reasons sampled meanwhile on rank 0: ms per call, max over ranks."""
    import bench                                   # ClockSampler lives beside the headline measurement
    reps = max(10, min(20000, int(seconds * 1e3 / max(ms_burst, 1e-3))))
    sampler = bench.ClockSampler(torch.cuda.current_device()) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.15)
        sampler.mark_begin()
    ms = _time(fn, world, reps=reps, warmup=1)
    clocks = None
    if sampler:
        sampler.mark_end()
        clocks = sampler.stop()
    return ms, reps, clocks


def _entry(name, config, work, unit_scale, unit, ms, ms_gather, peak, peak_note, sharding, launches):
    value = work / (ms * 1e-3) / unit_scale
    return {"kernel": name, "config": config, "value": value, "unit": unit, "ms": ms,
            "ms_with_output_gather": ms_gather, "frac_of_peak": value / peak if peak else None,
            "peak": peak, "peak_source": peak_note, "sharding": sharding, "launches_per_call": launches}


def gemm_bf16(dev, rank, world, peaks, m=8192, n=28672, k=8192):
    lo, hi = parallel.partition(n, world, rank, 256)
    g = torch.Generator(device=dev).manual_seed(2)
    a = (torch.randn(m, k, generator=g, device=dev) * 0.05).bfloat16()
    b = (torch.randn(k, hi - lo, generator=g, device=dev) * 0.05).bfloat16()
    so = parallel.ShardedOutput((m, n), 1, torch.bfloat16, dev, multiple=256)
    c = so.local
    ms = _time(lambda: ops.gemm(a, b, c), world)
    ms_g = _time(lambda: (ops.gemm(a, b, c), so.gather()), world, reps=3, warmup=2) if world > 1 else ms
    return _entry("gemm_pair_kernel", f"bf16 M{m} K{k} N{n}, B row-major [K,N]", 2.0 * m * n * k, 1e12, "TFLOP/s",
                  ms, ms_g, peaks["bf16_tflops"], peaks["note"], f"N columns / {world}", 1)


def gemm_fp8_plain(dev, rank, world, peaks, m=8192, n=28672, k=8192):
    """Un-scaled e4m3 GEMM (the FP8 operand form of ppl_gemm) at the C4 shape: what the FP8 tensor path of this
    library delivers without the per-128-K promotion; the block-scaled entry is read against it."""
    lo, hi = parallel.partition(n, world, rank, 256)
    g = torch.Generator(device=dev).manual_seed(2)
    a8 = torch.randn(m, k, generator=g, device=dev).to(torch.float8_e4m3fn)
    b8 = torch.randn(hi - lo, k, generator=g, device=dev).to(torch.float8_e4m3fn)
    so = parallel.ShardedOutput((m, n), 1, torch.bfloat16, dev, multiple=256)
    c = so.local
    ms = _time(lambda: ops.gemm(a8, b8, c, True), world)
    ms_g = _time(lambda: (ops.gemm(a8, b8, c, True), so.gather()), world, reps=3, warmup=2) if world > 1 else ms
    return _entry("gemm_pair_kernel (e4m3 operands)", f"e4m3 M{m} K{k} N{n}, B [N,K], no scales, bf16 out", 2.0 * m * n * k,
                  1e12, "TFLOP/s", ms, ms_g, 2 * peaks["bf16_tflops"], "2 x " + peaks["note"] + " (no FP8 peak was measured)",
                  f"N columns / {world}", 1)


def gemm_fp8(dev, rank, world, peaks, m=8192, n=28672, k=8192):
    lo, hi = parallel.partition(n, world, rank, 128)
    nl = hi - lo
    g = torch.Generator(device=dev).manual_seed(2)
    a8 = torch.randn(m, k, generator=g, device=dev).to(torch.float8_e4m3fn)
    b8 = torch.randn(nl, k, generator=g, device=dev).to(torch.float8_e4m3fn)
    sa = torch.rand(m, k // 128, generator=g, device=dev) * 1e-3 + 1e-4
    sb = torch.rand(-(-nl // 128), k // 128, generator=g, device=dev) * 1e-3 + 1e-4
    so = parallel.ShardedOutput((m, n), 1, torch.bfloat16, dev, multiple=128)
    c = so.local
    ms = _time(lambda: ops.gemm_fp8_blockscale(a8, b8, sa, sb, c), world)
    ms_g = _time(lambda: (ops.gemm_fp8_blockscale(a8, b8, sa, sb, c), so.gather()), world,
                 reps=3, warmup=2) if world > 1 else ms
    return _entry("gemm_fp8_blockscale_kernel", f"e4m3 M{m} K{k} N{n}, fp32 scales per 1x128 (A) and 128x128 (B)",
                  2.0 * m * n * k, 1e12, "TFLOP/s", ms, ms_g, 2 * peaks["bf16_tflops"],
                  "2 x " + peaks["note"] + " (no FP8 peak was measured)", f"N columns / {world}", 1)


def mlp_gate_up(dev, rank, world, peaks, m=8192, n=14336, k=4096):
    """Front half of the Llama-3-8B MLP: silu(x Wg^T) * (x Wu^T) in one kernel, against the two GEMMs plus the
    SwiGLU pass it replaces.  Sharded by output columns like the GEMM."""
    lo, hi = parallel.partition(n, world, rank, 128)
    nl = hi - lo
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(m, k, generator=g, device=dev).bfloat16()
    wg = (torch.randn(nl, k, generator=g, device=dev) * k ** -0.5).bfloat16()
    wu = (torch.randn(nl, k, generator=g, device=dev) * k ** -0.5).bfloat16()
    so = parallel.ShardedOutput((m, n), 1, torch.bfloat16, dev, multiple=128)
    out = so.local
    gate, up = torch.empty_like(out), torch.empty_like(out)
    ms = _time(lambda: ops.mlp_gate_up(x, wg, wu, out), world)

    def unfused():
        ops.gemm(x, wg, gate, True)
        ops.gemm(x, wu, up, True)
        ops.swiglu(gate, up, out)

    ms_u = _time(unfused, world)
    ms_g = _time(lambda: (ops.mlp_gate_up(x, wg, wu, out), so.gather()), world, reps=3, warmup=2) \
        if world > 1 else ms
    e = _entry("mlp_gate_up_tcgen05_kernel", f"bf16 M{m} K{k} N{n}: silu(x Wg^T) * (x Wu^T), weights [N,K]",
               4.0 * m * n * k, 1e12, "TFLOP/s", ms, ms_g, peaks["bf16_tflops"], peaks["note"], f"N columns / {world}", 1)
    e["ms_unfused_two_gemms_plus_swiglu"] = ms_u
    if world == 1:        # the whole MLP as the two-launch pipeline of ops.mlp (the down GEMM added): 6 M N K flop
        del gate, up
        wd = (torch.randn(k, n, generator=g, device=dev) * n ** -0.5).bfloat16()
        y = torch.empty(m, k, dtype=torch.bfloat16, device=dev)
        ms_full = _time(lambda: ops.mlp(x, wg, wu, wd, y, hidden=out), world)
        e["full_mlp"] = {"ms": ms_full, "value": 6.0 * m * n * k / (ms_full * 1e-3) / 1e12, "unit": "TFLOP/s",
                         "launches_per_call": 2}
    return e


def flash_attn(dev, rank, world, peaks, b=4, s=4096, h=32, d=128):
    lo, hi = parallel.partition(h, world, rank)
    hl = hi - lo
    g = torch.Generator(device=dev).manual_seed(4)
    q, k, v = (torch.randn(b, s, hl, d, generator=g, device=dev).bfloat16() for _ in range(3))
    so = parallel.ShardedOutput((b, s, h, d), 2, torch.bfloat16, dev)
    o = so.local
    ms = _time(lambda: ops.flash_attn_fwd(q, k, v, o, causal=True), world)
    ms_g = _time(lambda: (ops.flash_attn_fwd(q, k, v, o, causal=True), so.gather()), world,
                 reps=3, warmup=2) if world > 1 else ms
    return _entry("flash_attn_tcgen05_kernel", f"bf16 causal B{b} H{h} S{s} D{d} (bshd)", 4.0 * b * h * s * s * d * 0.5,
                  1e12, "TFLOP/s", ms, ms_g, peaks["bf16_tflops"], peaks["note"], f"heads / {world}", 1)


def mla_decode(dev, rank, world, peaks, batch=128, heads=128, d=576, dv=512, page=64, lo_len=1024, hi_len=8192):
    gc = torch.Generator(device="cpu").manual_seed(3)
    lens_all = torch.randint(lo_len, hi_len + 1, (batch,), generator=gc, dtype=torch.int32)
    mine = parallel.balance_by_length(lens_all.tolist(), world)[rank]
    lens = lens_all[mine].contiguous()
    nb = len(mine)
    pages_per = (lens + page - 1) // page
    total_pages = int(pages_per.sum()) + 8
    max_pages = -(-hi_len // page)
    perm = torch.randperm(total_pages, generator=gc).to(torch.int32)
    table = torch.zeros(nb, max_pages, dtype=torch.int32)
    cur = 0
    for i in range(nb):
        n = int(pages_per[i])
        table[i, :n] = perm[cur:cur + n]
        cur += n
    g = torch.Generator(device=dev).manual_seed(3)
    cache = torch.empty(total_pages, page, d, dtype=torch.float8_e4m3fn, device=dev)
    scale = torch.empty(total_pages, page, dtype=torch.float32, device=dev)
    for p0 in range(0, total_pages, 1024):
        p1 = min(total_pages, p0 + 1024)
        x = torch.randn(p1 - p0, page, d, generator=g, device=dev)
        sc = x.abs().amax(dim=-1, keepdim=True).clamp(min=1e-4) / 448.0
        cache[p0:p1] = (x / sc).to(torch.float8_e4m3fn)
        scale[p0:p1] = sc.squeeze(-1)
    q = torch.randn(nb, heads, d, generator=g, device=dev).bfloat16()
    lists = parallel.balance_by_length(lens_all.tolist(), world)
    so = parallel.ShardedOutput((batch, heads, dv), 0, torch.bfloat16, dev, index_lists=lists)
    out = so.local
    ordered = torch.empty(batch, heads, dv, dtype=torch.bfloat16, device=dev)
    table, lens_d = table.to(dev), lens.to(dev)
    fn = lambda: ops.mla_decode_paged(q, cache, scale, table, lens_d, out, softmax_scale=d ** -0.5)   # noqa: E731
    ms = _time(fn, world)
    ms_g = _time(lambda: (fn(), so.gather(), so.assemble(ordered)), world, reps=3, warmup=2) if world > 1 else ms
    tokens = int(lens_all.sum())
    flops = 2.0 * tokens * heads * (d + dv)
    nbytes = tokens * (d + 4) + batch * heads * (d + dv) * 2
    e = _entry("mla_decode_persistent_kernel", f"e4m3 paged cache, batch {batch}, {heads} heads, d {d}, dv {dv}, page {page}, "
               f"lengths U[{lo_len},{hi_len}] ({tokens} tokens)", nbytes, 1e9, "GB/s", ms, ms_g, peaks["hbm_gbs"],
               peaks["note"], f"sequences / {world} (balanced by length)", 3)     # prepare, decode, merge
    e["tflops"] = flops / (ms * 1e-3) / 1e12
    e["frac_of_bf16_tensor_peak"] = e["tflops"] / peaks["bf16_tflops"]
    return e


def mla_decode_bf16(dev, rank, world, peaks, batch=128, heads=128, d=576, dv=512, page=64, lo_len=1024, hi_len=8192):
    """The same decode with a bf16 latent cache (layout of examples/deepseek_mla/example_mla_decode_paged.py): the
    tcgen05 kernel for 16-bit caches, one CTA pair per sequence, no workspace."""
    gc = torch.Generator(device="cpu").manual_seed(3)
    lens_all = torch.randint(lo_len, hi_len + 1, (batch,), generator=gc, dtype=torch.int32)
    lists = parallel.balance_by_length(lens_all.tolist(), world)
    mine = lists[rank]
    lens = lens_all[mine].contiguous()
    nb = len(mine)
    pages_per = (lens + page - 1) // page
    total_pages = int(pages_per.sum()) + 8
    perm = torch.randperm(total_pages, generator=gc).to(torch.int32)
    table = torch.zeros(nb, -(-hi_len // page), dtype=torch.int32)
    cur = 0
    for i in range(nb):
        n = int(pages_per[i])
        table[i, :n] = perm[cur:cur + n]
        cur += n
    g = torch.Generator(device=dev).manual_seed(3)
    cache = torch.empty(total_pages, page, d, dtype=torch.bfloat16, device=dev)
    for p0 in range(0, total_pages, 1024):
        p1 = min(total_pages, p0 + 1024)
        cache[p0:p1] = torch.randn(p1 - p0, page, d, generator=g, device=dev).bfloat16()
    q = torch.randn(nb, heads, d, generator=g, device=dev).bfloat16()
    so = parallel.ShardedOutput((batch, heads, dv), 0, torch.bfloat16, dev, index_lists=lists)
    out = so.local
    ordered = torch.empty(batch, heads, dv, dtype=torch.bfloat16, device=dev)
    table, lens_d = table.to(dev), lens.to(dev)
    fn = lambda: ops.mla_decode_paged(q, cache, None, table, lens_d, out, softmax_scale=d ** -0.5)   # noqa: E731
    ms = _time(fn, world)
    ms_g = _time(lambda: (fn(), so.gather(), so.assemble(ordered)), world, reps=3, warmup=2) if world > 1 else ms
    tokens = int(lens_all.sum())
    flops = 2.0 * tokens * heads * (d + dv)
    nbytes = tokens * d * 2 + batch * heads * (d + dv) * 2
    e = _entry("mla_decode_f16_kernel", f"bf16 paged cache, batch {batch}, {heads} heads, d {d}, dv {dv}, page {page}, "
               f"lengths U[{lo_len},{hi_len}] ({tokens} tokens)", nbytes, 1e9, "GB/s", ms, ms_g, peaks["hbm_gbs"],
               peaks["note"], f"sequences / {world} (balanced by length)", 1)
    e["tflops"] = flops / (ms * 1e-3) / 1e12
    e["frac_of_bf16_tensor_peak"] = e["tflops"] / peaks["bf16_tflops"]
    return e


def small_ops(dev, rank, world, peaks, rows=8192, cols=4096):
    """The remaining tile-op programs (row reductions, sigmoid, elementwise add, gather, top-k) at sizes well
    above the L2, one entry each: algorithmic bytes / device time against the measured copy bandwidth."""
    g = torch.Generator(device=dev).manual_seed(6)
    out = []

    def add(name, config, nbytes, fn):
        ms = _time(fn, 1, reps=10)
        out.append(_entry(name, config, nbytes, 1e9, "GB/s", ms, ms, peaks["hbm_gbs"], peaks["note"], "none", 1))

    xb = torch.randn(4 * rows, cols, generator=g, device=dev).bfloat16()        # 268 MB at the default size: above the L2
    yb = torch.empty(4 * rows, 1, dtype=torch.bfloat16, device=dev)
    add("reduce_rows_kernel", f"row sum bf16 [{4 * rows}, {cols}]", xb.numel() * 2 + 4 * rows * 2, lambda: ops.reduce_rows(xb, yb, "sum"))
    del xb, yb
    xf = torch.randn(4 * rows, cols, generator=g, device=dev)
    yf = torch.empty(4 * rows, 1, device=dev)
    add("reduce_rows_kernel", f"row max fp32 [{4 * rows}, {cols}]", xf.numel() * 4 + 4 * rows * 4, lambda: ops.reduce_rows(xf, yf, "max"))
    zf = torch.empty_like(xf)
    add("unary_vec_kernel", f"sigmoid fp32 [{4 * rows}, {cols}]", xf.numel() * 8, lambda: ops.unary(xf, zf, "sigmoid"))
    wf = torch.randn(4 * rows, cols, generator=g, device=dev)
    add("binary_vec_kernel", f"add fp32 [{4 * rows}, {cols}]", xf.numel() * 12, lambda: ops.binary(xf, wf, zf, "add"))
    del wf
    idx = torch.randint(0, 4 * rows, (4 * rows,), generator=g, device=dev, dtype=torch.int32)
    add("gather_rows_kernel", f"gather {4 * rows} rows of {cols} fp32 from a [{4 * rows}, {cols}] table",
        2 * 4 * rows * cols * 4 + 4 * rows * 4, lambda: ops.gather_rows(xf, idx, zf))
    k = 8
    tv = torch.empty(4 * rows, k, device=dev)
    ti = torch.empty(4 * rows, k, dtype=torch.int32, device=dev)
    xt = xf.view(4 * rows * 4, cols // 4)             # 1024-wide rows: 8 cells per lane
    tv4 = torch.empty(xt.shape[0], k, device=dev)
    ti4 = torch.empty(xt.shape[0], k, dtype=torch.int32, device=dev)
    add("topk_cells_kernel", f"top-{k} of fp32 rows [{xt.shape[0]}, {xt.shape[1]}]", xt.numel() * 4 + xt.shape[0] * k * 8,
        lambda: ops.topk(xt, tv4, ti4, k))
    add("topk_cells_kernel", f"top-{k} of fp32 rows [{4 * rows}, {cols}]", xf.numel() * 4 + 4 * rows * k * 8,
        lambda: ops.topk(xf, tv, ti, k))
    k32 = 32
    tv32 = torch.empty(4 * rows, k32, device=dev)
    ti32 = torch.empty(4 * rows, k32, dtype=torch.int32, device=dev)
    add("topk_cells_kernel", f"top-{k32} of fp32 rows [{4 * rows}, {cols}]", xf.numel() * 4 + 4 * rows * k32 * 8,
        lambda: ops.topk(xf, tv32, ti32, k32))
    return out


def tile_program(dev, rank, world, peaks, rows=8192, cols=4096):
    """A row-local `ppl_*` program that no hand-written kernel matches, y = exp(x) * rsqrt(mean(x^2) + 1) + 0.5 on
    bf16 [rows, cols] in fp32 tiles (13 tile ops), run as ONE launch of the tile-program kernel; beside it the fused
    RMSNorm kernel on the same tensor (same bytes) and the op-by-op executor (one launch per tile op)."""
    import tilelang.language as T
    from tilelang.engine import fuser, interpreter
    bm = 32

    @T.prim_func
    def program(X: T.Tensor((rows, cols), "bfloat16"), Y: T.Tensor((rows, cols), "bfloat16")):
        with T.Kernel(rows // bm, is_cpu=True) as (bx,):
            x16 = T.alloc_shared((bm, cols), "bfloat16")
            x = T.alloc_shared((bm, cols), "float32")
            sq = T.alloc_shared((bm, cols), "float32")
            acc = T.alloc_shared((bm, 1), "float32")
            w0 = T.alloc_shared((bm, cols), "float32")
            coeff = T.alloc_shared((64, 32), "float32")
            table = T.alloc_shared((64, 192), "float32")
            T.ppl_copy(X[bx * bm, 0], x16)
            T.ppl_copy(x16, x)
            T.ppl_mul(sq, x, x)
            T.ppl_reduce_sum(sq, acc, dim=1)
            T.ppl_mul_C(acc, acc, T.float32(1.0 / cols))
            T.ppl_add_C(acc, acc, T.float32(1.0))
            T.ppl_rsqrt(acc, acc)
            T.ppl_exp2(x, w0, w0, coeff, table)
            T.ppl_mul(x, x, acc)
            T.ppl_add_C(x, x, T.float32(0.5))
            T.ppl_copy(x, x16)
            T.ppl_copy(x16, Y[bx * bm, 0])

    g = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(rows, cols, generator=g, device=dev).bfloat16()
    y = torch.empty_like(x)
    fused = fuser.build(program)
    ms = _time(lambda: fused(x, y), 1, reps=10)
    ms_norm = _time(lambda: ops.rmsnorm(x, y, None, 1e-6), 1, reps=10)
    by_op = interpreter.build(program)
    small = rows // bm <= 64
    ms_ops = _time(lambda: by_op(x, y), 1, reps=1, warmup=1) if small else None
    generated = bool(getattr(fused, "generated", False))
    e = _entry("tile_program (generated kernel)" if generated else "tile_vm_kernel",
               f"13-op row-local program on bf16 [{rows}, {cols}], {fused.instructions} instructions", 2.0 * x.numel() * 2,
               1e9, "GB/s", ms, ms, peaks["hbm_gbs"], peaks["note"], "none", 1)
    if generated:              # the interpreter kernel on the same instruction list
        e["ms_interpreter_kernel"] = _time(lambda: fused.interpreted(x, y), 1, reps=10)
    e["ms_fused_rmsnorm_same_tensor"] = ms_norm
    e["ratio_to_fused_rmsnorm"] = ms / ms_norm
    if ms_ops is not None:
        e["ms_op_by_op"] = ms_ops
    return e


def run_all(dev, rank, world, peaks):
    out = []
    plain_fp8 = None
    for fn in (gemm_bf16, gemm_fp8_plain, gemm_fp8, mlp_gate_up, flash_attn, mla_decode, mla_decode_bf16) + ((tile_program,) if world == 1 else ()):
        try:
            _last_call.clear()
            e = fn(dev, rank, world, peaks)
            if "fn" in _last_call:                 # the entry's first timed call is its compute-only call
                ms_s, reps, clocks = _sustained(_last_call["fn"], e["ms"], world, rank)
                e["timing"] = "value / ms: 5 launches after 3 warm-ups (burst)"
                e["sustained"] = {"ms": ms_s, "value": e["value"] * e["ms"] / ms_s, "launches": reps, "clocks": clocks}
            _last_call.clear()
            if fn is gemm_fp8_plain:
                plain_fp8 = e["value"]
            if fn is gemm_fp8 and plain_fp8:
                e["frac_of_plain_e4m3_gemm"] = e["value"] / plain_fp8
            if world > 1 and e.get("peak"):       # `value` is the whole job: compare with the peak of all GPUs
                e["peak"] *= world
                e["frac_of_peak"] = e["value"] / e["peak"]
                e["peak_source"] += f", x {world} GPUs"
                if "frac_of_bf16_tensor_peak" in e:
                    e["frac_of_bf16_tensor_peak"] /= world
            out.append(e)
        except Exception as exc:       # a failing extra must not lose the headline line
            out.append({"kernel": fn.__name__, "error": f"{type(exc).__name__}: {exc}"})
        torch.cuda.empty_cache()
        time.sleep(1.0)                # each entry is a burst figure: let the power limiter settle after the last one
    return out


SMALL = {      # reduced shapes for profiler captures: inputs above the 126 MB L2, a few hundred MB on the device
    "gemm_bf16": dict(m=4096, n=8192, k=4096),
    "gemm_fp8": dict(m=4096, n=8192, k=4096),
    "gemm_fp8_plain": dict(m=4096, n=8192, k=4096),
    "mlp_gate_up": dict(m=4096, n=4096, k=4096),
    "flash_attn": dict(b=2, s=4096, h=16, d=128),
    "mla_decode": dict(batch=32),
    "mla_decode_bf16": dict(batch=32),
    "small_ops": dict(rows=2048),
    "tile_program": dict(rows=2048),
}


def main(argv=None):
    """`python kernel_bench.py --kernel flash_attn [--small]` on one GPU."""
    import argparse
    import json
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True, choices=sorted(SMALL))
    ap.add_argument("--small", action="store_true", help="reduced shape (for profiler captures)")
    args = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "note": "of fallback"}
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        peaks = {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "note": "of measured"}
    fn = globals()[args.kernel]
    print(json.dumps(fn(dev, 0, 1, peaks, **(SMALL[args.kernel] if args.small else {}))))


if __name__ == "__main__":
    main()
