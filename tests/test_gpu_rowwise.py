"""Parity of the HBM-bound CUDA programs (through the C ABI) against the oracle."""
import pytest
import torch

import oracle.ops as O
from conftest import load_golden
from tilelang import ops, workloads

pytestmark = pytest.mark.gpu
BF, HF, F32 = torch.bfloat16, torch.float16, torch.float32
# tolerance for 16-bit outputs of fp32-internal programs (stated by the benchmark spec)
TOL16 = dict(atol=2e-2, rtol=2e-2)


def gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def max_rel(a, b):
    return ((a.double() - b.double()).abs() / b.double().abs().clamp_min(1e-30)).max().item()


# ------------------------------------------------------------------ RMSNorm
def test_rmsnorm_golden(cuda_device):
    g = load_golden("rmsnorm_bf16", dict(a=BF, ref=BF))
    x = g["a"].to(cuda_device)
    y = torch.zeros_like(x)
    assert ops.rmsnorm(x, y, eps=g["eps"]) == 0
    assert torch.allclose(y.cpu().float(), g["ref"].float(), **TOL16)
    # one-ulp agreement with the reference function on bf16 is expected almost everywhere
    assert (y.cpu().view(torch.int16).int() - g["ref"].view(torch.int16).int()).abs().max() <= 1


@pytest.mark.parametrize("dtype", [BF, HF, F32])
@pytest.mark.parametrize("rows,cols", [(128, 128), (3, 8), (33, 1000), (17, 4096), (5, 5000), (7, 16384),
                                       (4, 20000), (9, 4097), (1, 2)])
def test_rmsnorm_shapes(cuda_device, dtype, rows, cols):
    g = gen(rows * 131 + cols)
    x = torch.randn(rows, cols, generator=g).to(dtype)
    w = (1 + 0.02 * torch.randn(cols, generator=g)).to(dtype)
    for weight in (None, w):
        ref = O.rmsnorm(x, weight, eps=1e-6)
        y = torch.full_like(x, float("nan")).to(cuda_device)
        ops.rmsnorm(x.to(cuda_device), y, None if weight is None else weight.to(cuda_device), eps=1e-6)
        if dtype == F32:
            assert max_rel(y.cpu(), ref) < 1e-5
        else:
            assert torch.allclose(y.cpu().float(), ref.float(), **TOL16)


def test_rmsnorm_unaligned_base_pointer(cuda_device):
    x = torch.randn(6, 257, generator=gen(5)).to(BF)
    buf = torch.zeros(6 * 257 + 8, dtype=BF, device=cuda_device)
    xs = buf[1:1 + 6 * 257].view(6, 257)       # 2-byte offset: generic path
    xs.copy_(x)
    y = torch.zeros(6, 257, dtype=BF, device=cuda_device)
    ops.rmsnorm(xs, y, eps=1e-6)
    assert torch.allclose(y.cpu().float(), O.rmsnorm(x, eps=1e-6).float(), **TOL16)


def test_rmsnorm_empty(cuda_device):
    x = torch.empty(0, 64, dtype=BF, device=cuda_device)
    assert ops.rmsnorm(x, torch.empty_like(x)) == 0


def test_rmsnorm_llama_config(cuda_device):
    w = workloads.llama8b_memory_ops()
    x, wt = w["x"], w["weight"]
    y = torch.empty_like(x, device=cuda_device)
    ops.rmsnorm(x.to(cuda_device), y, wt.to(cuda_device), eps=w["eps"])
    ref = O.rmsnorm(x, wt, eps=w["eps"])
    assert torch.allclose(y.cpu().float(), ref.float(), **TOL16)
    # size-independent property: a normalised row scaled back by 1/weight has unit mean square
    ms = ((y.float() / wt.to(cuda_device).float()) ** 2).mean(dim=1)
    assert (ms - 1).abs().max().item() < 2e-2


# ------------------------------------------------------------------ RoPE
def test_rope_golden_bit_exact(cuda_device):
    g = load_golden("rope_bf16", dict(x=BF, cos=BF, sin=BF, ref=BF))
    out = torch.zeros_like(g["x"], device=cuda_device)
    ops.rope(g["x"].to(cuda_device), g["cos"].to(cuda_device), g["sin"].to(cuda_device), out)
    assert torch.equal(out.cpu().view(torch.int16), g["ref"].view(torch.int16))
    g = load_golden("rope_fp32")
    out = torch.zeros_like(g["x"], device=cuda_device)
    ops.rope(g["x"].to(cuda_device), g["cos"].to(cuda_device), g["sin"].to(cuda_device), out)
    # products and sum are separate roundings in the kernel as in the reference function
    assert torch.equal(out.cpu().view(torch.int32), g["ref"].view(torch.int32))


@pytest.mark.parametrize("dtype", [BF, HF, F32])
@pytest.mark.parametrize("tokens,heads,width", [(128, 1, 64), (5, 3, 128), (7, 2, 6), (64, 8, 128), (1, 1, 2)])
def test_rope_shapes(cuda_device, dtype, tokens, heads, width):
    g = gen(tokens * 7 + heads * 3 + width)
    x = torch.randn(tokens, heads, width, generator=g).to(dtype)
    cos, sin = workloads.rope_tables(tokens, width, 10000.0, dtype)
    ref = O.rope(x, cos, sin)
    out = torch.zeros_like(x, device=cuda_device)
    ops.rope(x.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device), out)
    # the kernel rounds where the reference's tile ops round: identical bits for every dtype
    assert torch.equal(out.cpu().view(torch.uint8), ref.view(torch.uint8))


def test_rope_llama_config(cuda_device):
    w = workloads.llama8b_memory_ops()
    cos, sin = w["cos"].to(cuda_device), w["sin"].to(cuda_device)
    for name in ("q", "k"):
        x = w[name]
        out = torch.empty_like(x, device=cuda_device)
        ops.rope(x.to(cuda_device), cos, sin, out)
        # oracle on a slice of tokens (full-size oracle is slow), plus a norm property on all
        sl = slice(4000, 4064)
        ref = O.rope(x[sl], w["cos"][sl], w["sin"][sl])
        assert torch.equal(out[sl].cpu().view(torch.int16), ref.view(torch.int16))
        # rotations preserve the norm of each pair up to bf16 rounding
        n_in = x.to(cuda_device).float().view(-1, 2).norm(dim=1)
        n_out = out.float().view(-1, 2).norm(dim=1)
        assert ((n_in - n_out).abs() <= 2e-2 * n_in + 2e-2).all()


# ------------------------------------------------------------------ SwiGLU
def test_swiglu_golden(cuda_device):
    g = load_golden("swiglu_bf16", dict(a=BF, b=BF, ref=BF))
    out = torch.zeros_like(g["a"], device=cuda_device)
    ops.swiglu(g["a"].to(cuda_device), g["b"].to(cuda_device), out)
    assert torch.allclose(out.cpu().float(), g["ref"].float(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", [BF, HF, F32])
@pytest.mark.parametrize("shape", [(64, 64), (1, 1), (3, 7), (1024, 1024), (129, 1031)])
def test_swiglu_shapes(cuda_device, dtype, shape):
    g = gen(shape[0] + shape[1])
    a = (torch.randn(*shape, generator=g) * 3).to(dtype)
    b = torch.randn(*shape, generator=g).to(dtype)
    ref = O.swiglu(a, b)
    out = torch.zeros_like(a, device=cuda_device)
    ops.swiglu(a.to(cuda_device), b.to(cuda_device), out)
    if dtype == F32:
        assert torch.allclose(out.cpu(), ref, atol=1e-6, rtol=1e-5)
    else:
        assert torch.allclose(out.cpu().float(), ref.float(), **TOL16)


def test_swiglu_llama_config(cuda_device):
    w = workloads.llama8b_memory_ops()
    out = torch.empty_like(w["gate"], device=cuda_device)
    ops.swiglu(w["gate"].to(cuda_device), w["up"].to(cuda_device), out)
    ref = O.swiglu(w["gate"], w["up"])
    assert torch.allclose(out.cpu().float(), ref.float(), **TOL16)


# ------------------------------------------------------------------ reductions and tile ops
def test_reduce_golden(cuda_device):
    g = load_golden("reduce_sum_fp16", dict(x=HF, ref=HF))
    y = torch.zeros(64, 1, dtype=HF, device=cuda_device)
    ops.reduce_rows(g["x"].to(cuda_device), y, "sum")
    assert torch.allclose(y.cpu().float(), g["ref"].float(), atol=1e-2, rtol=1e-2)
    g = load_golden("reduce_max_fp16", dict(x=HF, ref=HF))
    ops.reduce_rows(g["x"].to(cuda_device), y, "max")
    assert torch.equal(y.cpu().view(torch.int16), g["ref"].view(torch.int16))


@pytest.mark.parametrize("dtype", [BF, HF, F32])
@pytest.mark.parametrize("rows,cols", [(64, 64), (5, 1), (9, 33), (8192, 256), (3, 4096), (2, 100003), (11, 2050)])
def test_reduce_shapes(cuda_device, dtype, rows, cols):
    x = torch.randn(rows, cols, generator=gen(rows + cols)).to(dtype)
    y = torch.zeros(rows, 1, dtype=dtype, device=cuda_device)
    ops.reduce_rows(x.to(cuda_device), y, "max")
    assert torch.equal(y.cpu(), O.reduce_max(x))
    ops.reduce_rows(x.to(cuda_device), y, "sum")
    ref = x.double().sum(dim=1, keepdim=True)
    tol = 1e-4 * x.double().abs().sum(dim=1, keepdim=True) if dtype == F32 else \
        2e-2 * (1 + x.double().abs().sum(dim=1, keepdim=True).sqrt() + ref.abs())
    assert ((y.cpu().double() - ref).abs() <= tol).all()


@pytest.mark.parametrize("dtype", [torch.int32, torch.uint32, torch.int16])
@pytest.mark.parametrize("rows,cols", [(64, 64), (7, 1), (33, 1000), (3, 70001)])
def test_reduce_sum_integer_tiles_bit_exact(cuda_device, dtype, rows, cols):
    """ppl_reduce_sum on integer tiles (codegen_ppl.cc:1570-1592): exact, wrap-around included."""
    g = gen(rows * 3 + cols)
    if dtype == torch.int16:
        x = torch.randint(-2 ** 15, 2 ** 15, (rows, cols), generator=g, dtype=torch.int32).to(torch.int16)
    else:
        x = torch.randint(-2 ** 31, 2 ** 31 - 1, (rows, cols), generator=g, dtype=torch.int64).to(torch.int32)
        if dtype == torch.uint32:
            x = x.view(torch.uint32)
    y = torch.zeros(rows, 1, dtype=dtype, device=cuda_device)
    assert ops.reduce_rows(x.to(cuda_device), y, "sum") == 0
    ref = O.reduce_sum(x)
    bits = torch.int16 if dtype == torch.int16 else torch.int32
    assert torch.equal(y.cpu().view(bits), ref.view(bits))
    with pytest.raises(RuntimeError, match="sum only"):
        ops.reduce_rows(x.to(cuda_device), y, "max")


def test_sigmoid_golden_and_tile_ops(cuda_device):
    g = load_golden("sigmoid_fp32")
    y = torch.zeros_like(g["a"], device=cuda_device)
    ops.unary(g["a"].to(cuda_device), y, "sigmoid")
    assert max_rel(y.cpu(), g["ref"]) < 1e-5
    a = torch.randn(37, 53, generator=gen(1))
    b = torch.randn(37, 53, generator=gen(2)).abs() + 0.5
    col = torch.randn(37, 1, generator=gen(3)).abs() + 0.5
    ad, bd, cd = a.to(cuda_device), b.to(cuda_device), col.to(cuda_device)
    out = torch.zeros_like(ad)
    for name, fn in (("add", torch.add), ("sub", torch.sub), ("mul", torch.mul), ("div", torch.div)):
        ops.binary(ad, bd, out, name)
        assert max_rel(out.cpu(), fn(a, b)) < 1e-5
        ops.binary(ad, cd, out, name)
        assert max_rel(out.cpu(), fn(a, col)) < 1e-5
        ops.binary(ad, 1.5, out, name)
        assert max_rel(out.cpu(), fn(a, torch.tensor(1.5))) < 1e-5
    ops.unary(bd, out, "rsqrt")
    assert max_rel(out.cpu(), torch.rsqrt(b)) < 1e-5
    ops.unary(ad, out, "exp")
    assert max_rel(out.cpu(), torch.exp(a)) < 1e-5
    # copy with cast rounds to nearest even
    o16 = torch.zeros(37, 53, dtype=BF, device=cuda_device)
    ops.unary(ad, o16, "copy")
    assert torch.equal(o16.cpu(), a.to(BF))


def test_sigmoid_whole_range_vector_and_scalar_forms(cuda_device):
    """fp32 sigmoid at 1e-5 over the whole range where the result is a normal number, on the 16-byte vector form
    (size a multiple of 4) and on the scalar form (odd size, and a view that starts 4 bytes into an allocation)."""
    x = torch.cat([torch.linspace(-87.0, 88.0, 8191), torch.tensor([0.0, -0.0, 1e-30, -1e-30, 17.0])])
    ref = O.sigmoid(x)
    for n in (x.numel(), x.numel() - 3):
        y = torch.zeros(n, device=cuda_device)
        ops.unary(x[:n].to(cuda_device), y, "sigmoid")
        assert max_rel(y.cpu(), ref[:n]) < 1e-5
    base = torch.zeros(x.numel() + 1, device=cuda_device)
    base[1:] = x.to(cuda_device)
    y = torch.zeros(x.numel(), device=cuda_device)
    ops.unary(base[1:], y, "sigmoid")
    assert max_rel(y.cpu(), ref) < 1e-5


def test_bad_arguments_raise(cuda_device):
    x = torch.zeros(4, 4, dtype=BF, device=cuda_device)
    with pytest.raises(ValueError):
        ops.rmsnorm(x, torch.zeros(4, 5, dtype=BF, device=cuda_device))
    with pytest.raises(ValueError):
        ops.rmsnorm(torch.zeros(4, 4, dtype=BF), torch.zeros(4, 4, dtype=BF))   # CPU tensors
    with pytest.raises(ValueError):
        ops.swiglu(x, x.to(HF), x)
    with pytest.raises(ValueError):
        ops.rmsnorm(x.to(torch.float64), x.to(torch.float64))


def test_run_to_run_determinism(cuda_device):
    # same idea as the reference profiler's assert_consistent (tilelang/profiler/__init__.py:124-141)
    x = torch.randn(512, 4096, generator=gen(9)).to(BF).to(cuda_device)
    y0 = torch.empty_like(x)
    ops.rmsnorm(x, y0, eps=1e-6)
    for _ in range(3):
        y = torch.empty_like(x)
        ops.rmsnorm(x, y, eps=1e-6)
        assert torch.equal(y.view(torch.int16), y0.view(torch.int16))


# ------------------------------------------------------------------ window copy / fill / running max
@pytest.mark.parametrize("src_dt,dst_dt", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32),
                                           (torch.float16, torch.float16), (torch.float32, torch.float16),
                                           (torch.int32, torch.int32)])
def test_copy2d_windows_and_casts(cuda_device, src_dt, dst_dt):
    g = torch.Generator(device="cpu").manual_seed(21)
    big = (torch.randn(40, 72, generator=g) * 3).to(src_dt) if src_dt.is_floating_point else \
        torch.randint(-1000, 1000, (40, 72), generator=g, dtype=src_dt)
    src = big.to(cuda_device)
    dst = torch.zeros(64, 48, dtype=dst_dt, device=cuda_device)
    assert ops.copy2d(src[5:37, 8:40], dst[16:48, 3:35]) == 0           # window -> window
    ref = torch.zeros(64, 48, dtype=dst_dt)
    ref[16:48, 3:35] = big[5:37, 8:40].to(dst_dt)                        # round-to-nearest-even cast
    assert torch.equal(dst.cpu(), ref)
    assert ops.copy2d(src[:0, :48], dst[:0]) == 0                          # empty


def test_fill_window_and_running_max(cuda_device):
    t = torch.zeros(16, 32, dtype=torch.bfloat16, device=cuda_device)
    assert ops.fill(t[4:12, 8:24], 1.5) == 0
    ref = torch.zeros(16, 32, dtype=torch.bfloat16)
    ref[4:12, 8:24] = 1.5
    assert torch.equal(t.cpu(), ref)
    g = torch.Generator(device="cpu").manual_seed(22)
    a, b = torch.randn(8, 16, generator=g), torch.randn(8, 16, generator=g)
    out = torch.empty(8, 16, device=cuda_device)
    assert ops.binary(a.to(cuda_device), b.to(cuda_device), out, "max") == 0
    assert torch.equal(out.cpu(), torch.maximum(a, b))
    with pytest.raises(ValueError, match="contiguous rows"):
        ops.fill(t.t()[0:4, 0:4], 0.0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_swiglu_over_a_wide_gate_range(cuda_device, dtype):
    """The 16-bit path evaluates SiLU as 0.5 g (1 + tanh(g / 2)) with the hardware tanh (one XU operation):
    over gates in [-40, 40] the result stays 4x inside the stated 2e-2 tolerance; far-negative gates give 0."""
    g = torch.linspace(-40, 40, 1 << 18).to(dtype).view(512, 512)
    u = torch.ones_like(g)
    out = torch.empty_like(g).to(cuda_device)
    assert ops.swiglu(g.to(cuda_device), u.to(cuda_device), out) == 0
    ref = O.swiglu(g, u).float()
    assert torch.allclose(out.cpu().float(), ref, atol=5e-3, rtol=1e-2)
    assert (out.cpu().float()[g.float() < -17.5] == 0).all()


# ------------------------------------------------------------------ the generic void** entry point
def test_generic_entry_point_runs_programs(cuda_device):
    """`tl_b200_run(kernel_id, void** args, meta, stream)`: the pointer list in the shape of the reference's
    generated `tilelang_tpu_run(void** args)`, sizes in `meta`; same bits as the typed entry points."""
    from tilelang import _native as N
    g = gen(77)
    x = torch.randn(64, 512, generator=g).to(BF).to(cuda_device)
    w = (1 + 0.02 * torch.randn(512, generator=g)).to(BF).to(cuda_device)
    y_typed, y_run = torch.zeros_like(x), torch.zeros_like(x)
    assert ops.rmsnorm(x, y_typed, w, eps=1e-6) == 0
    stream = torch.cuda.current_stream().cuda_stream
    rc = N.run("rmsnorm", [x.data_ptr(), w.data_ptr(), y_run.data_ptr()], [64, 512, N.float_bits(1e-6), N.TL_BF16], stream)
    assert rc == 0 and torch.equal(y_typed.view(torch.int16), y_run.view(torch.int16))
    a = torch.randn(128, 64, generator=g).to(HF).to(cuda_device)
    b = torch.randn(64, 96, generator=g).to(HF).to(cuda_device)
    c_typed, c_run = (torch.zeros(128, 96, dtype=HF, device=cuda_device) for _ in range(2))
    assert ops.gemm(a, b, c_typed) == 0
    rc = N.run("gemm", [a.data_ptr(), b.data_ptr(), c_run.data_ptr()], [128, 96, 64, 0, N.TL_F16, N.TL_F16], stream)
    assert rc == 0 and torch.equal(c_typed.view(torch.int16), c_run.view(torch.int16))
    rc = N.run("swiglu", [0, 0, 0], [16, N.TL_BF16], stream)
    assert rc == -1 and "null" in N.last_error()


# ------------------------------------------------------------------ a bounded wait that runs out
def test_expired_bounded_wait_reaches_the_host_and_leaves_the_context_usable(cuda_device):
    """Every barrier wait of the tensor-core kernels is bounded; when one gives up the kernel raises its abort
    flag, returns and writes a host-visible status word.  The self-test kernel makes exactly that happen (one
    warp, a barrier nothing arrives at, a 2 ms budget - no copy or MMA in flight, nothing faults or hangs)."""
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert ops.selftest_bounded_wait(2000) == 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="TL_B200_EDEVICE"):
        ops.check_device_status()
    assert ops.device_status() == 0                              # reading clears it
    x = torch.randn(8, 64, generator=gen(3)).to(BF).to(cuda_device)
    y = torch.zeros_like(x)
    assert ops.rmsnorm(x, y, eps=1e-6) == 0                      # the context is still good
    torch.cuda.synchronize()
    assert torch.allclose(y.cpu().float(), O.rmsnorm(x.cpu(), eps=1e-6).float(), **TOL16)
    with pytest.raises(RuntimeError, match="budget"):
        ops.selftest_bounded_wait(10 ** 7)
