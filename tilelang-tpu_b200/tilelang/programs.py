"""Programs of the benchmark configurations, written against the tile DSL.

The reference's demo programs (tpu_demo/rms_norm/rms_norm_bf16.py:9-35, tpu_demo/tpu_test_rope_bf16.py:5-51,
tpu_demo/tpu_test_swiglu_bf16.py:5-54) run small shapes; the builders here are the same tile programs at
the Llama-3-8B shapes, with the two things the benchmark adds: a per-column weight for RMSNorm
(`ppl_mul` by a (1, N) row) and cos/sin tables held per token and shared by the heads of a token.
`tilelang.compile(program, out_idx=-1, target="b200")` binds each of them to its fused kernel.

Two benchmark operators have no `ppl_*` form in the reference at all (its FP8 block-scaled GEMM and its
paged MLA decode are written in the upstream GPU dialect, examples/deepseek_deepgemm/
example_deepgemm_fp8_2xAcc.py and examples/deepseek_mla/example_mla_decode_paged.py).  They are offered
as *library programs*: a parameter list plus the name of the kernel that implements it, so that they go
through the same `tilelang.compile` / JITKernel / adapter call convention as everything else.
"""

from . import language as T
from .language.ir import Buffer, PrimFunc, Tracer


def rmsnorm(M: int, N: int, blk_m: int = 32, dtype: str = "bfloat16", eps: float = 1e-6, weight: bool = True) -> PrimFunc:
    """B = A * rsqrt(mean(A^2, -1) + eps) [* W]; A, B are (M, N), W is (1, N); fp32 inside."""
    def body(A, W, B, bx):
        inv_n = T.float32(1.0 / N)
        a16 = T.alloc_shared((blk_m, N), dtype)
        a32 = T.alloc_shared((blk_m, N), "float32")
        sq = T.alloc_shared((blk_m, N), "float32")
        acc = T.alloc_shared((blk_m, 1), "float32")
        T.ppl_copy(A[bx * blk_m, 0], a16)
        T.ppl_copy(a16, a32)
        T.ppl_mul(sq, a32, a32)
        T.ppl_reduce_sum(sq, acc, dim=1)
        T.ppl_mul_C(acc, acc, inv_n)
        T.ppl_add_C(acc, acc, T.float32(eps))
        T.ppl_rsqrt(acc, acc)
        T.ppl_mul(a32, a32, acc)
        if W is not None:
            w16 = T.alloc_shared((1, N), dtype)
            w32 = T.alloc_shared((1, N), "float32")
            T.ppl_copy(W[0, 0], w16)
            T.ppl_copy(w16, w32)
            T.ppl_mul(a32, a32, w32)          # (1, N) row, broadcast down the rows of the tile
        T.ppl_copy(a32, a16)
        T.ppl_copy(a16, B[bx * blk_m, 0])

    if weight:
        @T.prim_func
        def rmsnorm_kernel(A: T.Tensor((M, N), dtype), W: T.Tensor((1, N), dtype), B: T.Tensor((M, N), dtype)):
            with T.Kernel(T.ceildiv(M, blk_m), is_cpu=True) as (bx,):
                body(A, W, B, bx)
        return rmsnorm_kernel

    @T.prim_func
    def rmsnorm_kernel(A: T.Tensor((M, N), dtype), B: T.Tensor((M, N), dtype)):     # noqa: F811
        with T.Kernel(T.ceildiv(M, blk_m), is_cpu=True) as (bx,):
            body(A, None, B, bx)
    return rmsnorm_kernel


def rope(tokens: int, heads: int, width: int, blk_t: int = 64, dtype: str = "bfloat16") -> PrimFunc:
    """Interleaved-pair rotation of X (tokens, heads, width) by per-token tables Cos, Sin (tokens, width)
    in the pair-duplicated layout of make_rope_cos_sin (tpu_demo/tpu_test_rope_bf16.py:53-74)."""
    @T.prim_func
    def rope_kernel(X: T.Tensor((tokens, heads, width), dtype), Cos: T.Tensor((tokens, width), dtype),
                    Sin: T.Tensor((tokens, width), dtype), Out: T.Tensor((tokens, heads, width), dtype)):
        with T.Kernel(T.ceildiv(tokens, blk_t), heads, is_cpu=True) as (bx, by):
            x = T.alloc_shared((blk_t, width), dtype)
            c = T.alloc_shared((blk_t, width), dtype)
            s = T.alloc_shared((blk_t, width), dtype)
            xc = T.alloc_shared((blk_t, width), dtype)
            xs = T.alloc_shared((blk_t, width), dtype)
            nx = T.alloc_shared((blk_t, width), dtype)
            nxs = T.alloc_shared((blk_t, width), dtype)
            o = T.alloc_shared((blk_t, width), dtype)
            T.ppl_copy(X[bx * blk_t:(bx + 1) * blk_t, by, 0:width], x)
            T.ppl_copy(Cos[bx * blk_t, 0], c)
            T.ppl_copy(Sin[bx * blk_t, 0], s)
            T.ppl_mul(xc, x, c)
            T.ppl_mul(xs, x, s)
            T.ppl_mul_C(nx, x, -1.0)
            T.ppl_mul(nxs, nx, s)
            T.ppl_rope_add(o, xc, nxs, xc, xs)
            T.ppl_copy(o, Out[bx * blk_t:(bx + 1) * blk_t, by, 0:width])
    return rope_kernel


def swiglu(C: int, W: int, blk_c: int = 32, blk_w: int = 1024, dtype: str = "bfloat16") -> PrimFunc:
    """Out = Up * Gate / (1 + exp(-Gate)) in fp32, rounded once (tpu_demo/tpu_test_swiglu_bf16.py:5-54)."""
    @T.prim_func
    def swiglu_kernel(Gate: T.Tensor((C, W), dtype), Up: T.Tensor((C, W), dtype), Out: T.Tensor((C, W), dtype)):
        with T.Kernel(T.ceildiv(C, blk_c), T.ceildiv(W, blk_w), is_cpu=True) as (bx, by):
            one = T.alloc_shared((blk_c, blk_w), "float32")
            g16 = T.alloc_shared((blk_c, blk_w), dtype)
            u16 = T.alloc_shared((blk_c, blk_w), dtype)
            g = T.alloc_shared((blk_c, blk_w), "float32")
            u = T.alloc_shared((blk_c, blk_w), "float32")
            e = T.alloc_shared((blk_c, blk_w), "float32")
            o16 = T.alloc_shared((blk_c, blk_w), dtype)
            work0 = T.alloc_shared((blk_c, blk_w), "float32")
            work1 = T.alloc_shared((blk_c, blk_w), "float32")
            coeff = T.alloc_shared((64, 32), "float32")
            table = T.alloc_shared((64, 192), "float32")
            T.ppl_fill(one, T.float32(1.0))
            T.ppl_copy(Gate[bx * blk_c, by * blk_w], g16)
            T.ppl_copy(Up[bx * blk_c, by * blk_w], u16)
            T.ppl_copy(g16, g)
            T.ppl_copy(u16, u)
            T.ppl_mul_C(e, g, -1.0)
            T.ppl_exp2(e, work0, work1, coeff, table)
            T.ppl_add(e, e, one)
            T.ppl_div(g, g, e)
            T.ppl_mul(u, u, g)
            T.ppl_copy(u, o16)
            T.ppl_copy(o16, Out[bx * blk_c, by * blk_w])
    return swiglu_kernel


# ------------------------------------------------------------------------------- library programs
def _library_program(name: str, params, kernel: str, **facts) -> PrimFunc:
    """A program that is a parameter list plus the library kernel implementing it (no tile ops)."""
    bufs = [Buffer(pname, tuple(int(d) for d in shape), dtype, "global", param_index=i)
            for i, (pname, shape, dtype) in enumerate(params)]
    func = PrimFunc(name, bufs, Tracer())
    func.attrs["library_kernel"] = kernel
    func.attrs["facts"] = dict(facts)
    return func


def gemm_fp8_blockscale(M: int, N: int, K: int, out_dtype: str = "bfloat16") -> PrimFunc:
    """C = (A8 * SA) (B8 * SB)^T, DeepGEMM-style: e4m3 operands, fp32 scales per 1x128 block of A and per
    128x128 block of B, promotion of every 128-wide K block in fp32
    (examples/deepseek_deepgemm/example_deepgemm_fp8_2xAcc.py:17-90 of the reference)."""
    assert K % 128 == 0, "gemm K shape check failed"
    return _library_program(
        "gemm_fp8_blockscale",
        [("A8", (M, K), "float8_e4m3"), ("B8", (N, K), "float8_e4m3"), ("SA", (M, K // 128), "float32"),
         ("SB", (-(-N // 128), K // 128), "float32"), ("C", (M, N), out_dtype)],
        "gemm_fp8_blockscale", M=M, N=N, K=K)


def mlp(M: int, hidden_size: int, intermediate_size: int, dtype: str = "bfloat16") -> PrimFunc:
    """The gated MLP at full size: Out = (silu(X Wg^T) * (X Wu^T)) Wd^T with the roundings of the reference's per-tile
    program (tpu_demo/ppl/mlp/mlp_bf16.py:57-136; same parameter order: output first)."""
    return _library_program(
        "mlp",
        [("Out", (M, hidden_size), dtype), ("X", (M, hidden_size), dtype), ("Wg", (intermediate_size, hidden_size), dtype),
         ("Wu", (intermediate_size, hidden_size), dtype), ("Wd", (hidden_size, intermediate_size), dtype)],
        "mlp", M=M, hidden_size=hidden_size, intermediate_size=intermediate_size)


def mla_decode_paged(batch: int, heads: int, d: int, dv: int, num_pages: int, page_size: int, max_pages: int,
                     dtype: str = "bfloat16", cache_dtype: str = "float8_e4m3", softmax_scale: float | None = None) -> PrimFunc:
    """Paged MLA decode, one query token per sequence (tensor layout of
    examples/deepseek_mla/example_mla_decode_paged.py:20-97,259-308): Q (batch, 1, heads, d), the latent
    cache (num_pages, page_size, 1, d) whose first dv columns are V, an int32 block table
    (batch, max_pages), int32 lengths (batch,), Out (batch, 1, heads, dv).  An e4m3 cache comes with one
    fp32 scale per token, (num_pages, page_size); 16-bit caches take no scale parameter."""
    params = [("Q", (batch, 1, heads, d), dtype), ("KV", (num_pages, page_size, 1, d), cache_dtype)]
    fp8 = cache_dtype in ("float8_e4m3", "e4m3_float8")
    if fp8:
        params.append(("KVScale", (num_pages, page_size), "float32"))
    params += [("BlockTable", (batch, max_pages), "int32"), ("CacheSeqlens", (batch,), "int32"),
               ("Out", (batch, 1, heads, dv), dtype)]
    return _library_program("mla_decode_paged", params, "mla_decode_paged", batch=batch, heads=heads, d=d, dv=dv,
                            page_size=page_size, scaled=fp8,
                            softmax_scale=float(softmax_scale if softmax_scale is not None else d ** -0.5))
