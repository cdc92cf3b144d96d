"""Operator-level entry points over the C ABI: CUDA tensors in, outputs written in place.

Each function corresponds to one reference program (the `tpu_demo` kernels built from
`T.ppl_*` intrinsics); the JIT front end binds matched programs to these.  Tensors must live on
the current CUDA device; torch is used only for device memory and the current stream.
"""
from __future__ import annotations

import torch

from . import _native as N

_DTYPES = {
    torch.float32: N.TL_F32,
    torch.float16: N.TL_F16,
    torch.bfloat16: N.TL_BF16,
    torch.int32: N.TL_I32,
    torch.uint32: N.TL_U32,
    torch.int16: N.TL_I16,
}
if hasattr(torch, "float8_e4m3fn"):
    _DTYPES[torch.float8_e4m3fn] = N.TL_E4M3

_initialised_devices: set[int] = set()


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise ValueError(f"dtype {dt} is not supported by the b200 kernel library") from None


def _prepare(*tensors: torch.Tensor) -> int:
    """Common argument checks; returns the raw handle of the current stream."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("b200 ops take CUDA tensors (there is no CPU path)")
        if not t.is_contiguous():
            raise ValueError("b200 ops take contiguous tensors")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"tensors on different devices: {dev} and {t.device}")
    index = dev.index if dev is not None and dev.index is not None else torch.cuda.current_device()
    if index != torch.cuda.current_device():
        raise ValueError(f"tensors are on cuda:{index} but the current device is "
                         f"cuda:{torch.cuda.current_device()}")
    if index not in _initialised_devices:
        N.check(N.load().tl_b200_init(index), "tl_b200_init")
        _initialised_devices.add(index)
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


generated_launches = 0          # launches of kernels generated for a program (engine/codegen.py), counted here


def launch_count() -> int:
    """Kernels this process has launched from the library and from generated programs."""
    return int(N.load().tl_b200_launch_count()) + generated_launches


def rmsnorm(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor | None = None, eps: float = 1e-12) -> int:
    """y = x * rsqrt(mean(x^2, -1) + eps) [* weight]; x, y are (rows, cols)."""
    if x.dim() != 2 or x.shape != y.shape or x.dtype != y.dtype:
        raise ValueError("rmsnorm: x and y must be 2-D with equal shape and dtype")
    if weight is not None and (weight.numel() != x.shape[1] or weight.dtype != x.dtype):
        raise ValueError("rmsnorm: weight must have cols elements of x's dtype")
    s = _prepare(x, y, weight)
    return N.check(N.load().tl_b200_rmsnorm(_ptr(x), _ptr(weight), _ptr(y), x.shape[0], x.shape[1],
                                           float(eps), dtype_code(x.dtype), s), "tl_b200_rmsnorm")


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, out: torch.Tensor) -> int:
    """Interleaved-pair rotation.  x/out: (..., W); cos/sin: (T, W) with x.numel()/W a multiple
    of T (each table row serves `rows/T` consecutive rows of x, e.g. the heads of a token)."""
    width = x.shape[-1]
    rows = x.numel() // max(width, 1)
    if out.shape != x.shape or out.dtype != x.dtype:
        raise ValueError("rope: out must match x")
    if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != width or cos.dtype != x.dtype \
            or sin.dtype != x.dtype:
        raise ValueError("rope: cos/sin must be (T, W) tables of x's dtype")
    t_rows = cos.shape[0]
    if t_rows == 0 or rows % t_rows != 0:
        raise ValueError(f"rope: {rows} rows cannot be served by a {t_rows}-row table")
    s = _prepare(x, cos, sin, out)
    return N.check(N.load().tl_b200_rope(_ptr(x), _ptr(cos), _ptr(sin), _ptr(out), rows, width,
                                        rows // t_rows, dtype_code(x.dtype), s), "tl_b200_rope")


def swiglu(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor) -> int:
    """out = up * silu(gate)."""
    if gate.shape != up.shape or gate.shape != out.shape or not (gate.dtype == up.dtype == out.dtype):
        raise ValueError("swiglu: gate, up and out must have equal shape and dtype")
    s = _prepare(gate, up, out)
    return N.check(N.load().tl_b200_swiglu(_ptr(gate), _ptr(up), _ptr(out), gate.numel(),
                                          dtype_code(gate.dtype), s), "tl_b200_swiglu")


def reduce_rows(x: torch.Tensor, y: torch.Tensor, op: str) -> int:
    """y[r, 0] = sum|max over x[r, :]."""
    if x.dim() != 2 or y.numel() != x.shape[0] or y.dtype != x.dtype:
        raise ValueError("reduce_rows: x must be (rows, cols) and y hold rows elements of x's dtype")
    code = {"sum": 0, "max": 1}[op]
    s = _prepare(x, y)
    return N.check(N.load().tl_b200_reduce_rows(_ptr(x), _ptr(y), x.shape[0], x.shape[1], code,
                                               dtype_code(x.dtype), s), "tl_b200_reduce_rows")


_UNARY = {"sigmoid": 0, "exp": 1, "rsqrt": 2, "copy": 3}
_BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "max": 4}


def unary(x: torch.Tensor, y: torch.Tensor, op: str) -> int:
    if x.numel() != y.numel():
        raise ValueError("unary: size mismatch")
    s = _prepare(x, y)
    return N.check(N.load().tl_b200_unary(_ptr(x), _ptr(y), x.numel(), _UNARY[op], dtype_code(x.dtype),
                                         dtype_code(y.dtype), s), "tl_b200_unary")


def binary(a: torch.Tensor, b, out: torch.Tensor, op: str) -> int:
    """out = a (op) b; b is a tensor shaped like a, a (rows, 1) column, a (1, cols) row, or a Python scalar."""
    if a.dim() != 2 or out.shape != a.shape or out.dtype != a.dtype:
        raise ValueError("binary: a and out must be 2-D with equal shape and dtype")
    rows, cols = a.shape
    scalar = 0.0
    if isinstance(b, torch.Tensor):
        if b.dtype != a.dtype:
            raise ValueError("binary: dtype mismatch")
        if b.shape == a.shape:
            mode = 0
        elif b.numel() == rows and (b.dim() < 2 or b.shape[-1] == 1 or cols == 1):
            mode = 1
        elif b.numel() == cols and b.dim() == 2 and b.shape[0] == 1:
            mode = 3
        else:
            raise ValueError("binary: b must match a, be a (rows, 1) column or a (1, cols) row")
        s = _prepare(a, b, out)
        bp = _ptr(b)
    else:
        mode, scalar, bp = 2, float(b), None
        s = _prepare(a, out)
    return N.check(N.load().tl_b200_binary(_ptr(a), bp, _ptr(out), rows, cols, _BINARY[op], mode, scalar,
                                          dtype_code(a.dtype), s), "tl_b200_binary")


def _window(t: torch.Tensor, what: str):
    """(rows, cols, row pitch in elements) of a 2-D window whose rows are contiguous."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise ValueError(f"{what}: expected a 2-D window with contiguous rows")
    return t.shape[0], t.shape[1], (t.stride(0) if t.shape[0] > 1 else max(t.shape[1], 1))


def _prepare_windows(*tensors: torch.Tensor) -> int:
    base = [t.view(-1) if t.is_contiguous() else t.as_strided((1,), (1,)) for t in tensors]
    return _prepare(*base)


def copy2d(src: torch.Tensor, dst: torch.Tensor) -> int:
    """dst[r, c] = cast(src[r, c]) between two 2-D windows (views with contiguous rows) of equal shape."""
    if src.shape != dst.shape:
        raise ValueError("copy2d: shapes differ")
    rows, cols, sld = _window(src, "copy2d")
    _, _, dld = _window(dst, "copy2d")
    s = _prepare_windows(src, dst)
    return N.check(N.load().tl_b200_copy2d(_ptr(src), _ptr(dst), rows, cols, sld, dld, dtype_code(src.dtype),
                                          dtype_code(dst.dtype), s), "tl_b200_copy2d")


def fill(dst: torch.Tensor, value: float) -> int:
    """dst[:, :] = value for a 2-D window with contiguous rows."""
    rows, cols, ld = _window(dst, "fill")
    s = _prepare_windows(dst)
    return N.check(N.load().tl_b200_fill(_ptr(dst), rows, cols, ld, float(value), dtype_code(dst.dtype), s), "tl_b200_fill")


def rope_add(out: torch.Tensor, even1: torch.Tensor, even2: torch.Tensor, odd1: torch.Tensor, odd2: torch.Tensor) -> int:
    """out[:, 2i] = even1[:, 2i] + even2[:, 2i+1]; out[:, 2i+1] = odd1[:, 2i+1] + odd2[:, 2i] on 2-D tiles."""
    ts = (out, even1, even2, odd1, odd2)
    if out.dim() != 2 or any(t.shape != out.shape or t.dtype != out.dtype for t in ts):
        raise ValueError("rope_add: five 2-D tiles of one shape and dtype")
    s = _prepare(*ts)
    return N.check(N.load().tl_b200_rope_add(_ptr(out), _ptr(even1), _ptr(even2), _ptr(odd1), _ptr(odd2), out.shape[0],
                                            out.shape[1], dtype_code(out.dtype), s), "tl_b200_rope_add")


def gather_rows(param: torch.Tensor, index: torch.Tensor, out: torch.Tensor) -> int:
    """out[i, :] = param[index[i], :]; index holds uint32 (or non-negative int32) row ids."""
    if param.dim() != 2 or out.dim() != 2 or out.shape[1] != param.shape[1] or out.dtype != param.dtype:
        raise ValueError("gather_rows: param (R, H) and out (n, H) must share H and dtype")
    if index.dtype not in (torch.uint32, torch.int32) or index.numel() != out.shape[0]:
        raise ValueError("gather_rows: index must hold out.shape[0] uint32/int32 entries")
    s = _prepare(param, index, out)
    row_bytes = param.shape[1] * param.element_size()
    return N.check(N.load().tl_b200_gather_rows(_ptr(param), _ptr(index), _ptr(out), out.shape[0], row_bytes,
                                               param.shape[0], s), "tl_b200_gather_rows")


def topk(src: torch.Tensor, out_vals: torch.Tensor, out_idx: torch.Tensor, k: int, descending: bool = True) -> int:
    """Sorted top-k of each row of src ((length,) or (rows, length)); the first k entries of each
    row of out_vals / out_idx (int32) are written."""
    if src.dim() not in (1, 2):
        raise ValueError("topk: src must be 1-D or 2-D")
    rows = 1 if src.dim() == 1 else src.shape[0]
    length = src.shape[-1]
    if src.dtype not in (torch.float32, torch.int32, torch.uint32):
        raise ValueError("topk: src must be float32, int32 or uint32")
    if out_vals.dtype != src.dtype or out_idx.dtype != torch.int32:
        raise ValueError("topk: out_vals must have src's dtype and out_idx must be int32")
    out_stride = out_vals.shape[-1]
    if out_idx.shape[-1] != out_stride or out_vals.numel() != rows * out_stride \
            or out_idx.numel() != rows * out_stride:
        raise ValueError("topk: out_vals / out_idx must be (rows, stride) with equal stride")
    s = _prepare(src, out_vals, out_idx)
    return N.check(N.load().tl_b200_topk(_ptr(src), _ptr(out_vals), _ptr(out_idx), rows, length, int(k),
                                        1 if descending else 0, out_stride, dtype_code(src.dtype), s),
                   "tl_b200_topk")


def device_status() -> int:
    """Status word left by a kernel that gave up a bounded wait (0 = none); clears it."""
    return int(N.load().tl_b200_device_status())


def check_device_status() -> None:
    """Raise if a kernel gave up a bounded wait since the last check (status TL_B200_EDEVICE); call after the
    stream has been synchronised.  The adapter of the reference raises on a non-zero native status in the same
    way (cython_wrapper.pyx:160-163)."""
    code = device_status()
    if code:
        raise RuntimeError(f"device status {code} (TL_B200_EDEVICE): {N.last_error()}")


def selftest_bounded_wait(budget_us: int = 1000) -> int:
    """Launch the one-warp kernel whose bounded wait is made to run out (nothing arrives at its barrier)."""
    index = torch.cuda.current_device()
    if index not in _initialised_devices:
        N.check(N.load().tl_b200_init(index), "tl_b200_init")
        _initialised_devices.add(index)
    return N.check(N.load().tl_b200_selftest_bounded_wait(int(budget_us), torch.cuda.current_stream().cuda_stream),
                   "tl_b200_selftest_bounded_wait")


def gemm(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, transpose_b: bool = False, tile_n: int | None = None) -> int:
    """c = a @ b (b is (K, N)) or a @ b.T (b is (N, K), transpose_b=True); fp32 accumulation.
    fp16 / bf16 / fp32 operands, or e4m3 (the plain, un-scaled FP8 form of ppl_gemm)."""
    if a.dim() != 2 or b.dim() != 2 or c.dim() != 2:
        raise ValueError("gemm: a, b, c must be 2-D")
    m, k = a.shape
    n, kb = (b.shape[0], b.shape[1]) if transpose_b else (b.shape[1], b.shape[0])
    if kb != k:
        raise ValueError("gemm K shape check failed")          # message of ppl_gemm's assert
    if tuple(c.shape) != (m, n):
        raise ValueError(f"gemm: c must be ({m}, {n})")
    f8 = getattr(torch, "float8_e4m3fn", None)
    if a.dtype != b.dtype:
        raise ValueError("gemm: a and b must share a dtype")
    if a.dtype == f8:
        if c.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise ValueError("gemm: e4m3 operands take a float32, bfloat16 or float16 output")
    elif c.dtype not in (a.dtype, torch.float32):
        raise ValueError("gemm: a and b must share a dtype; c has that dtype or float32")
    if a.dtype not in (torch.float16, torch.bfloat16, torch.float32, f8):
        raise ValueError(f"gemm: unsupported dtype {a.dtype}")
    s = _prepare(a, b, c)
    if tile_n is None:                      # a choice the tuner stored for this shape, else the library's own rule
        from .cache import tile_choice
        tuned = tile_choice("gemm", m=m, n=n, k=k, dtype=str(a.dtype), transpose_b=bool(transpose_b))
        tile_n = int(tuned["tile_n"]) if tuned else 0
    return N.check(N.load().tl_b200_gemm_tiled(_ptr(a), _ptr(b), _ptr(c), m, n, k, 1 if transpose_b else 0,
                                              dtype_code(a.dtype), dtype_code(c.dtype), int(tile_n), s), "tl_b200_gemm")


def mlp_gate_up(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, out: torch.Tensor) -> int:
    """out = silu(x @ w_gate.T) * (x @ w_up.T): x (M, K), w_gate and w_up (N, K), out (M, N), one dtype.
    Both products are rounded to that dtype before the fp32 SiLU-product, as the MLP program does."""
    if x.dim() != 2 or w_gate.dim() != 2 or tuple(w_up.shape) != tuple(w_gate.shape):
        raise ValueError("mlp_gate_up: x (M, K), w_gate and w_up (N, K)")
    m, k = x.shape
    n = w_gate.shape[0]
    if w_gate.shape[1] != k:
        raise ValueError("gemm K shape check failed")          # message of ppl_gemm's assert
    if tuple(out.shape) != (m, n):
        raise ValueError(f"mlp_gate_up: out must be ({m}, {n})")
    if not (x.dtype == w_gate.dtype == w_up.dtype == out.dtype):
        raise ValueError("mlp_gate_up: all tensors must share a dtype")
    if x.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError(f"mlp_gate_up: unsupported dtype {x.dtype}")
    s = _prepare(x, w_gate, w_up, out)
    return N.check(N.load().tl_b200_mlp_gate_up(_ptr(x), _ptr(w_gate), _ptr(w_up), _ptr(out), m, n, k,
                                               dtype_code(x.dtype), s), "tl_b200_mlp_gate_up")


_MASK_MODES = {False: 0, None: 0, "none": 0, True: 1, "causal": 1, "block": 2}


_mlp_hidden: dict = {}


def mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, out: torch.Tensor,
        hidden: torch.Tensor | None = None) -> int:
    """The gated MLP as one pipeline of two launches: hidden = silu(x Wg^T) * (x Wu^T) (SiLU-product in the epilogue of
    the gate and up GEMMs), out = hidden Wd^T.  x (M, K); w_gate, w_up (N, K); w_down (K_out, N); out (M, K_out).
    The only intermediate is `hidden` (M, N): the caller's buffer, or one kept per (device, stream, shape, dtype).
    Roundings are where the reference program has them (tpu_demo/ppl/mlp/mlp_bf16.py:100-131)."""
    if x.dim() != 2 or w_gate.dim() != 2 or w_down.dim() != 2:
        raise ValueError("mlp: x (M, K), w_gate and w_up (N, K), w_down (K_out, N)")
    m, n = x.shape[0], w_gate.shape[0]
    if w_down.shape[1] != n:
        raise ValueError("gemm K shape check failed")          # message of ppl_gemm's assert
    if tuple(out.shape) != (m, w_down.shape[0]):
        raise ValueError(f"mlp: out must be ({m}, {w_down.shape[0]})")
    if hidden is None:
        key = (x.device, torch.cuda.current_stream(x.device).cuda_stream, m, n, x.dtype)
        hidden = _mlp_hidden.get(key)
        if hidden is None:
            _mlp_hidden.clear()                               # one shape at a time: no growth without bound
            hidden = _mlp_hidden[key] = torch.empty(m, n, dtype=x.dtype, device=x.device)
    elif tuple(hidden.shape) != (m, n) or hidden.dtype != x.dtype:
        raise ValueError(f"mlp: hidden must be ({m}, {n}) of x's dtype")
    rc = mlp_gate_up(x, w_gate, w_up, hidden)
    return rc or gemm(hidden, w_down, out, transpose_b=True)


def flash_attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, scale: float | None = None,
                   causal=False, block_m: int = 0, block_n: int = 0) -> int:
    """Attention forward on bshd tensors.  causal: False / True (key <= query) / "block" (the
    reference program's shortened KV loop without a mask inside the last tile; needs block sizes)."""
    if q.dim() != 4 or k.dim() != 4 or k.shape != v.shape or o.shape != q.shape:
        raise ValueError("flash_attn_fwd: q, o are (B, Sq, H, D); k, v are (B, Skv, H, D)")
    b, sq, h, d = q.shape
    if k.shape[0] != b or k.shape[2] != h or k.shape[3] != d:
        raise ValueError("flash_attn_fwd: q and k/v disagree on batch, heads or head dim")
    if not (q.dtype == k.dtype == v.dtype == o.dtype):
        raise ValueError("flash_attn_fwd: one dtype for q, k, v, o")
    try:
        mode = _MASK_MODES[causal]
    except (KeyError, TypeError):
        raise ValueError(f"flash_attn_fwd: unknown mask {causal!r}") from None
    if scale is None:
        scale = d ** -0.5
    s = _prepare(q, k, v, o)
    return N.check(N.load().tl_b200_flash_attn_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(o), b, sq, k.shape[1], h, d,
                                                  float(scale), mode, int(block_m), int(block_n),
                                                  dtype_code(q.dtype), s), "tl_b200_flash_attn_fwd")


def mla_decode_dense(q: torch.Tensor, q_pe: torch.Tensor, kv: torch.Tensor, k_pe: torch.Tensor, out: torch.Tensor,
                     scale: float | None = None) -> int:
    """Dense-cache MLA decode: q (B,H,1,D), q_pe (B,H,1,P), kv (B,S,1,D), k_pe (B,S,1,P), out (B,H,1,D)."""
    if q.dim() != 4 or q.shape[2] != 1 or kv.dim() != 4 or kv.shape[2] != 1 or out.shape != q.shape:
        raise ValueError("mla_decode_dense: expected q (B,H,1,D), kv (B,S,1,D), out like q")
    b, h, _, d = q.shape
    pe = q_pe.shape[-1]
    if q_pe.shape != (b, h, 1, pe) or k_pe.shape != (b, kv.shape[1], 1, pe) or kv.shape[0] != b or kv.shape[3] != d:
        raise ValueError("mla_decode_dense: inconsistent shapes")
    if not (q.dtype == q_pe.dtype == kv.dtype == k_pe.dtype == out.dtype):
        raise ValueError("mla_decode_dense: one dtype for all tensors")
    if scale is None:
        scale = (d + pe) ** -0.5
    s = _prepare(q, q_pe, kv, k_pe, out)
    return N.check(N.load().tl_b200_mla_decode_dense(_ptr(q), _ptr(q_pe), _ptr(kv), _ptr(k_pe), _ptr(out), b, h,
                                                    kv.shape[1], d, pe, float(scale), dtype_code(q.dtype), s),
                   "tl_b200_mla_decode_dense")


def gemm_fp8_blockscale(a8: torch.Tensor, b8: torch.Tensor, scales_a: torch.Tensor, scales_b: torch.Tensor,
                        c: torch.Tensor) -> int:
    """c = (a8 * scales_a) @ (b8 * scales_b)^T with 128-granular fp32 scales: a8 (M,K) e4m3 with
    scales_a (M, K/128); b8 (N,K) e4m3 with scales_b (ceil(N/128), K/128); c (M,N) bf16 or fp32."""
    f8 = torch.float8_e4m3fn
    if a8.dtype != f8 or b8.dtype != f8 or a8.dim() != 2 or b8.dim() != 2 or a8.shape[1] != b8.shape[1]:
        raise ValueError("gemm_fp8_blockscale: a8 (M,K) and b8 (N,K) must be e4m3 with equal K")
    m, k = a8.shape
    n = b8.shape[0]
    if k % 128 != 0:
        raise ValueError("gemm_fp8_blockscale: K must be a multiple of 128")
    if tuple(scales_a.shape) != (m, k // 128) or tuple(scales_b.shape) != (-(-n // 128), k // 128) \
            or scales_a.dtype != torch.float32 or scales_b.dtype != torch.float32:
        raise ValueError("gemm_fp8_blockscale: scales_a must be (M, K/128) and scales_b (ceil(N/128), K/128), fp32")
    if tuple(c.shape) != (m, n) or c.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("gemm_fp8_blockscale: c must be (M, N) bfloat16 or float32")
    s = _prepare(a8, b8, scales_a, scales_b, c)
    return N.check(N.load().tl_b200_gemm_fp8_blockscale(_ptr(a8), _ptr(b8), _ptr(scales_a), _ptr(scales_b), _ptr(c),
                                                       m, n, k, dtype_code(c.dtype), s),
                   "tl_b200_gemm_fp8_blockscale")


def mla_decode_paged_gqa(q: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor, cache_seqlens: torch.Tensor,
                         out: torch.Tensor, softmax_scale: float | None = None) -> int:
    """Paged decode with s_q query tokens per sequence and h_kv kv heads: q (B, s_q, h_q, D), kv_cache
    (num_pages, page, h_kv, D) of q's 16-bit dtype, out (B, s_q, h_q, DV); query token i sees keys up to len - s_q + i."""
    if q.dim() != 4 or kv_cache.dim() != 4 or out.dim() != 4 or kv_cache.shape[-1] != q.shape[-1]:
        raise ValueError("mla_decode_paged_gqa: q (B, s_q, h_q, D), kv_cache (pages, page, h_kv, D), out (B, s_q, h_q, DV)")
    b, s_q, h_q, d = q.shape
    num_pages, page, h_kv, _ = kv_cache.shape
    dv = out.shape[-1]
    if tuple(out.shape[:3]) != (b, s_q, h_q) or out.dtype != q.dtype or kv_cache.dtype != q.dtype:
        raise ValueError("mla_decode_paged_gqa: out must be (B, s_q, h_q, DV); q, cache and out share a 16-bit dtype")
    if block_table.dtype != torch.int32 or cache_seqlens.dtype != torch.int32 or block_table.shape[0] != b or cache_seqlens.numel() != b:
        raise ValueError("mla_decode_paged_gqa: block_table (B, max_pages) and cache_seqlens (B,) must be int32")
    if softmax_scale is None:
        softmax_scale = d ** -0.5
    s = _prepare(q, kv_cache, block_table, cache_seqlens, out)
    return N.check(N.load().tl_b200_mla_decode_paged_gqa(_ptr(q), _ptr(kv_cache), _ptr(block_table), _ptr(cache_seqlens), _ptr(out),
                                                        b, s_q, h_q, h_kv, d, dv, page, block_table.shape[1], num_pages,
                                                        float(softmax_scale), dtype_code(q.dtype), s),
                   "tl_b200_mla_decode_paged_gqa")


_workspaces: dict = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch owned by this module (the library never allocates): one growing buffer per
    (device, stream).  Calls on different streams may overlap on the GPU and must not share the
    partial results kept there; on one stream they are ordered, and a buffer that is replaced by a
    larger one goes back to torch's allocator, which reuses it only in stream order."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 4096), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def mla_decode_paged(q: torch.Tensor, kv_cache: torch.Tensor, kv_scale: torch.Tensor | None, block_table: torch.Tensor,
                     cache_seqlens: torch.Tensor, out: torch.Tensor, dv: int | None = None,
                     softmax_scale: float | None = None, balanced: bool = True) -> int:
    """Paged MLA decode.  q (B, H, D) or (B, 1, H, D); kv_cache (num_pages, page, D) or
    (num_pages, page, 1, D) in e4m3 / fp16 / bf16; kv_scale (num_pages, page) fp32 for e4m3;
    block_table (B, max_pages) int32; cache_seqlens (B,) int32; out (B, H, DV) or (B, 1, H, DV).
    `balanced` hands the library the large workspace of its persistent, work-balanced kernel;
    False passes only the small one (one CTA pair per sequence)."""
    b, h, d = q.shape[0], q.shape[-2], q.shape[-1]
    if q.numel() != b * h * d or kv_cache.shape[-1] != d:
        raise ValueError("mla_decode_paged: q must hold one token per sequence and share D with the cache")
    num_pages, page = kv_cache.shape[0], kv_cache.shape[1]
    if kv_cache.numel() != num_pages * page * d:
        raise ValueError("mla_decode_paged: the cache must have a single kv head")
    dv = int(dv if dv is not None else out.shape[-1])
    if out.numel() != b * h * dv or out.dtype != q.dtype:
        raise ValueError("mla_decode_paged: out must be (B, H, DV) of q's dtype")
    if block_table.dtype != torch.int32 or cache_seqlens.dtype != torch.int32 or block_table.shape[0] != b \
            or cache_seqlens.numel() != b:
        raise ValueError("mla_decode_paged: block_table (B, max_pages) and cache_seqlens (B,) must be int32")
    if kv_scale is not None and (kv_scale.dtype != torch.float32 or kv_scale.numel() != num_pages * page):
        raise ValueError("mla_decode_paged: kv_scale must be (num_pages, page) float32")
    if kv_cache.dtype == torch.float8_e4m3fn and kv_scale is None:
        raise ValueError("mla_decode_paged: an e4m3 cache needs kv_scale")
    if softmax_scale is None:
        softmax_scale = d ** -0.5
    s = _prepare(q, kv_cache, kv_scale, block_table, cache_seqlens, out)
    lib = N.load()
    if balanced:
        ws_bytes = int(lib.tl_b200_mla_decode_paged_split_workspace_bytes(b, block_table.shape[1], page))
    else:
        ws_bytes = int(lib.tl_b200_mla_decode_paged_workspace_bytes(b))
    ws = _workspace(q.device, ws_bytes)
    return N.check(lib.tl_b200_mla_decode_paged(_ptr(q), _ptr(kv_cache), _ptr(kv_scale), _ptr(block_table),
                                               _ptr(cache_seqlens), _ptr(out), b, h, d, dv, page,
                                               block_table.shape[1], num_pages, float(softmax_scale),
                                               dtype_code(q.dtype), dtype_code(kv_cache.dtype), _ptr(ws), ws_bytes, s),
                   "tl_b200_mla_decode_paged")
