/*
 * tl_b200.h — C ABI of libtl_b200.so, the sm_100a kernel library behind the
 * `T.ppl_*` operator path.
 *
 * The reference binds ONE generated symbol per compiled program,
 *     extern "C" int tilelang_tpu_run(void** args)
 * (src/tl_templates/tpu/main_template.cpp:39, bound with ctypes in
 * tilelang/jit/adapter/cython/adapter.py:213-216), with all sizes baked in at
 * code-generation time.  This library is pre-built instead, so every entry
 * point takes the sizes explicitly.  Conventions shared by all entry points:
 *
 *   - every pointer is a DEVICE pointer on the current CUDA device; the library
 *     never allocates, frees or copies user tensors and never synchronises;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - the return value is 0 on success or a negative TL_B200_E* code; the
 *     message for the calling thread is available from tl_b200_last_error()
 *     (same shape as the `init()/call()/get_last_error()` convention of the
 *     reference's CUDA host wrappers, tilelang/jit/adapter/wrapper.py:22-42);
 *   - all tensors are dense row-major unless a stride argument says otherwise.
 */
#ifndef TL_B200_H_
#define TL_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TL_B200_VERSION 100

/* error codes */
#define TL_B200_OK 0
#define TL_B200_EINVAL (-1)   /* bad argument (null pointer, size, alignment, dtype) */
#define TL_B200_ECUDA (-2)    /* a CUDA runtime/driver call failed */
#define TL_B200_EUNSUP (-3)   /* valid request this build has no kernel for */
#define TL_B200_EDEVICE (-4)  /* a kernel reported an error through its status word */

/* element types (values are part of the ABI) */
#define TL_F32 0
#define TL_F16 1
#define TL_BF16 2
#define TL_E4M3 3
#define TL_I32 4
#define TL_U32 5
#define TL_I16 6   /* integer row sums only */

/* ---- library management ---------------------------------------------------
 * Replaces init()/post() of the generated host (main_template.cpp:14-37).    */
int tl_b200_init(int device);
int tl_b200_version(void);
const char* tl_b200_last_error(void);
/* Number of kernels this library has launched in the calling process. */
int64_t tl_b200_launch_count(void);
/* Kernels that wait on barriers bound every wait; one that gives up writes a non-zero code to
 * a host-visible status word and exits cleanly.  Returns that code (0 = none) and clears it.
 * Meaningful after the stream has been synchronised.  (The generated TPU host reports launch
 * failures through its return value, main_template.cpp:64-67.)                               */
int tl_b200_device_status(void);
/* Self-test of that path: launches one warp that waits, with the library's bounded wait and a budget
 * of budget_us microseconds (1 .. 100000), on a barrier nothing arrives at.  The wait expires, the
 * kernel writes the status word and returns; after a stream synchronise tl_b200_device_status()
 * reports it and the context stays usable.  (No counterpart in the reference, whose launches block
 * inside the vendor runtime.)                                                                    */
int tl_b200_selftest_bounded_wait(int64_t budget_us, void* stream);

/* ---- RMSNorm program ------------------------------------------------------
 * y[r,:] = x[r,:] * rsqrt(mean(x[r,:]^2) + eps) (* weight[:] if weight != NULL),
 * fp32 arithmetic, one rounding to `dtype` at the end.
 * Replaces the program tpu_demo/rms_norm/rms_norm_bf16.py:9-35 (ppl_copy, ppl_mul,
 * ppl_reduce_sum, ppl_mul_C, ppl_add_C, ppl_rsqrt chain; eps 1e-12, no weight).  */
int tl_b200_rmsnorm(const void* x, const void* weight, void* y, int64_t rows, int64_t cols,
                    float eps, int dtype, void* stream);

/* ---- RoPE program (interleaved pairs) --------------------------------------
 * out[r,2i]   = x[r,2i]*cos[t,2i]   + (-x[r,2i+1])*sin[t,2i]
 * out[r,2i+1] = x[r,2i+1]*cos[t,2i+1] + x[r,2i]*sin[t,2i+1],   t = r / rows_per_table_row,
 * every product and the sum rounded to `dtype` as the reference's tile ops do.
 * Replaces tpu_demo/tpu_test_rope_bf16.py:5-51 (ppl_mul, ppl_mul_C, ppl_rope_add,
 * src/target/codegen_ppl.cc:1809-1848).  rows_per_table_row = 1 is the reference's
 * full-size-table form; = heads broadcasts one table row over the heads of a token. */
int tl_b200_rope(const void* x, const void* cos_tab, const void* sin_tab, void* out, int64_t rows,
                 int64_t width, int64_t rows_per_table_row, int dtype, void* stream);

/* ---- SwiGLU program --------------------------------------------------------
 * out = up * gate / (1 + exp(-gate)), fp32 arithmetic, one rounding at the end.
 * Replaces tpu_demo/tpu_test_swiglu_bf16.py:5-54.                                 */
int tl_b200_swiglu(const void* gate, const void* up, void* out, int64_t n_elems, int dtype,
                   void* stream);

/* ---- row reductions --------------------------------------------------------
 * y[r] = sum or max over x[r, 0:cols];  op 0 = sum (ppl_reduce_sum,
 * codegen_ppl.cc:1554-1792), op 1 = max (ppl_reduce_max, :1352-1553).
 * Accumulation in fp32; output in `dtype`.  Programs: tpu_demo/tpu_test_reduce_sum.py,
 * tpu_demo/tpu_test_reduce_max.py.  The sum also takes TL_I32 / TL_U32 / TL_I16 tiles
 * (codegen_ppl.cc:1570-1592): exact sums modulo 2^32, TL_I16 cut to 16 bits.         */
int tl_b200_reduce_rows(const void* x, void* y, int64_t rows, int64_t cols, int op, int dtype,
                        void* stream);

/* ---- elementwise tile ops --------------------------------------------------
 * Unary: op 0 = sigmoid (ppl_sigmoid, codegen_ppl.cc:1321-1351), 1 = exp (ppl_exp2,
 * natural exponential, :1294-1320), 2 = rsqrt (ppl_rsqrt, :1793-1807), 3 = copy/cast
 * (ppl_copy with differing dtypes, round-to-nearest-even, :1138-1151).              */
int tl_b200_unary(const void* x, void* y, int64_t n_elems, int op, int in_dtype, int out_dtype,
                  void* stream);
/* The tile op ppl_rope_add on contiguous rows x cols tiles (cols even):
 * out[:, 2i] = even1[:, 2i] + even2[:, 2i+1], out[:, 2i+1] = odd1[:, 2i+1] + odd2[:, 2i], one
 * rounding to `dtype` (customize.py:563-603, codegen_ppl.cc:1809-1848).  The fused RoPE program is
 * tl_b200_rope; this entry serves programs that assemble the rotation from their own terms.      */
int tl_b200_rope_add(void* out, const void* even1, const void* even2, const void* odd1, const void* odd2,
                     int64_t rows, int64_t cols, int dtype, void* stream);
/* Strided 2-D copy with a cast: dst[r, c] = cast(src[r, c]) for a rows x cols window; src_ld and
 * dst_ld are the row pitches in elements.  What ppl_copy does between a window of a global tensor
 * and a tile, or between two tiles of different dtypes (customize.py:136-207,
 * codegen_ppl.cc:958-1243; round-to-nearest-even on narrowing).  Float dtypes convert freely;
 * TL_I32 / TL_U32 copy bits.                                                              */
int tl_b200_copy2d(const void* src, void* dst, int64_t rows, int64_t cols, int64_t src_ld, int64_t dst_ld,
                   int src_dtype, int dst_dtype, void* stream);
/* dst[r, c] = value over a rows x cols window with row pitch ld (ppl_fill, customize.py:210-231). */
int tl_b200_fill(void* dst, int64_t rows, int64_t cols, int64_t ld, float value, int dtype, void* stream);
/* Binary: out = a (op) b with op 0 add, 1 sub, 2 mul, 3 div (ppl_add/subtract/mul/div,
 * codegen_ppl.cc:891-913,1280-1287), 4 max (the running maximum that ppl_reduce_max keeps with
 * clear=False, customize.py:519-560).  b_mode 0: b has the shape of a; 1: b is (rows,1)
 * and broadcasts across columns (:868-889); 2: b is ignored and `scalar` is used
 * (ppl_mul_C / ppl_add_C, :917-957); 3: b is (1,cols) and broadcasts down the rows (no reference
 * form: the per-column weight of the Llama RMSNorm).  fp32 arithmetic, rounded to `dtype`.     */
int tl_b200_binary(const void* a, const void* b, void* out, int64_t rows, int64_t cols, int op,
                   int b_mode, float scalar, int dtype, void* stream);

/* ---- gather ----------------------------------------------------------------
 * out[i,:] = param[index[i],:] for i < n_index; index is uint32; rows whose index is
 * >= param_rows are written as zeros (never read out of bounds).  row_bytes is the
 * byte length of one row.  Replaces ppl_gather (customize.py:352-356,
 * codegen_ppl.cc:1849-1877); program tpu_demo/tpu_test_gather_fp32.py.             */
int tl_b200_gather_rows(const void* param, const uint32_t* index, void* out, int64_t n_index,
                        int64_t row_bytes, int64_t param_rows, void* stream);

/* ---- top-k -----------------------------------------------------------------
 * For each of `rows` independent arrays of `length` elements (row stride = length):
 * the k largest (descending != 0) or smallest values, sorted, with their int32 source
 * positions; ties are ordered by lower index first.  Results go to the first k entries
 * of each row of out_vals / out_idx, whose row stride is out_stride elements (the
 * reference passes length-sized output buffers, tpu_demo/tpu_test_topk_fp32.py:11-13).
 * dtype: TL_F32, TL_I32 or TL_U32 (codegen_ppl.cc:1898-1903).  Replaces ppl_topk
 * (customize.py:358-362, codegen_ppl.cc:1878-1907).                                */
int tl_b200_topk(const void* src, void* out_vals, int32_t* out_idx, int64_t rows, int64_t length,
                 int k, int descending, int64_t out_stride, int dtype, void* stream);

/* ---- dense GEMM -------------------------------------------------------------
 * C[m,n] = A[m,k] * B with fp32 accumulation, rounded once to out_dtype.  A is row-major
 * [m,k].  trans_b == 0: B is row-major [k,n] (the matmul program,
 * tpu_demo/matmul/tpu_test_matmul_fp16.py:9-30); trans_b != 0: B is row-major [n,k]
 * (`transpose_B=True` of ppl_gemm, customize.py:101-133, codegen_ppl.cc:1244-1279).
 * in_dtype TL_F16 / TL_BF16 run on tcgen05 tensor cores when A, B are 16-byte aligned,
 * k % 8 == 0 and (trans_b or n % 8 == 0); other shapes and TL_F32 use an FMA kernel.
 * out_dtype is in_dtype or TL_F32.  in_dtype TL_E4M3 is the plain (un-scaled) FP8 operand form
 * of ppl_gemm (codegen_ppl.cc:775-790): tensor cores only (16-byte aligned tensors, k % 16 == 0,
 * trans_b or n % 16 == 0), out_dtype TL_F32, TL_BF16 or TL_F16.                        */
int tl_b200_gemm(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int trans_b,
                 int in_dtype, int out_dtype, void* stream);
/* The same with the width of the C tile chosen by the caller: tile_n 64, 128 or 256 columns (0 = the
 * library's own rule, the widest tile that still gives every SM one), or 512 = tiles of 256 x 256 computed
 * by pairs of CTAs on neighbouring SMs (each loads half of the tile's B).  For a shape -> tile table kept by
 * the host (role of the reference's tuner, tilelang/autotuner/__init__.py:90-345).  Results do not depend
 * on the choice.                                                                                        */
int tl_b200_gemm_tiled(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int trans_b,
                       int in_dtype, int out_dtype, int tile_n, void* stream);

/* ---- gated MLP, front half -----------------------------------------------------
 * out[m,n] = silu(x Wg^T) * (x Wu^T) with x [m,k] and w_gate, w_up [n,k] row-major, all of
 * `dtype`.  The arithmetic of the reference's MLP program up to its down projection
 * (tpu_demo/ppl/mlp/mlp_bf16.py:103-125, mlp_fp32.py): both GEMMs accumulate in fp32 and
 * deliver tiles of `dtype`, SiLU (g / (1 + exp(-g))) and the product run in fp32, and the
 * result is rounded once more.  The two GEMMs share the x tiles and the SiLU-product is their
 * epilogue, so neither intermediate is written to memory.  The down projection is
 * tl_b200_gemm(out, w_down [hidden, n], y, m, hidden, n, trans_b = 1, ...).
 * TL_F16 / TL_BF16 run on tcgen05 tensor cores when x, w_gate, w_up are 16-byte aligned and
 * k % 8 == 0; other shapes and TL_F32 use an FMA kernel.                                  */
int tl_b200_mlp_gate_up(const void* x, const void* w_gate, const void* w_up, void* out, int64_t m,
                        int64_t n, int64_t k, int dtype, void* stream);

/* ---- FP8 GEMM with 128-granular scales --------------------------------------------
 * c[m,n] = sum_kb scales_a[m,kb] * scales_b[n/128,kb] * (a[m, kb*128:(kb+1)*128] . b[n, same]),
 * a [m,k] and b [n,k] row-major e4m3, scales_a [m, k/128] and scales_b [ceil(n/128), k/128]
 * fp32, every 128-wide partial product accumulated in fp32; c is TL_BF16 or TL_F32.
 * Follows the block-scaled program examples/deepseek_deepgemm/example_deepgemm_fp8_2xAcc.py:14-83
 * (quantisers :93-112).  k must be a multiple of 128.                                        */
int tl_b200_gemm_fp8_blockscale(const void* a, const void* b, const float* scales_a,
                                const float* scales_b, void* c, int64_t m, int64_t n, int64_t k,
                                int out_dtype, void* stream);

/* ---- FlashAttention forward -----------------------------------------------------
 * o = softmax(scale * q k^T + mask) v on bshd tensors: q, o [batch, seq_q, heads, dim];
 * k, v [batch, seq_kv, heads, dim]; fp32 softmax statistics; P is rounded to `dtype` before the
 * second product, as the program does.  Replaces the program
 * tpu_demo/flashattn/tpu_test_flashattn_bf16.py:14-135 (ppl_gemm / ppl_reduce_max / ppl_exp2 /
 * ppl_reduce_sum chain).  mask_mode 0: none; 1: causal (key <= query), the mask of the
 * reference's check function (:171-182); 2: the reference program's own causal form, a KV loop
 * shortened to ceil((bx+1)*block_m/block_n) tiles with no mask inside the last tile (:116-118).
 * TL_BF16 / TL_F16 with dim 64 or 128 run on tcgen05; other cases use an FMA kernel.          */
int tl_b200_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, int64_t batch,
                           int64_t seq_q, int64_t seq_kv, int64_t heads, int64_t dim, float scale,
                           int mask_mode, int block_m, int block_n, int dtype, void* stream);

/* ---- MLA decode, dense cache ----------------------------------------------------
 * out[b,h,0,:] = softmax(scale * (q.kv^T + q_pe.k_pe^T)) kv with q [batch,heads,1,dim],
 * q_pe [batch,heads,1,pe_dim], kv [batch,seq_kv,1,dim], k_pe [batch,seq_kv,1,pe_dim],
 * out [batch,heads,1,dim]; V is the latent kv itself.  Replaces the program
 * tpu_demo/ppl/deepseek_mla/mla_decode.py:9-121.                                             */
int tl_b200_mla_decode_dense(const void* q, const void* q_pe, const void* kv, const void* k_pe,
                             void* out, int64_t batch, int64_t heads, int64_t seq_kv, int64_t dim,
                             int64_t pe_dim, float scale, int dtype, void* stream);

/* ---- MLA decode, paged cache ------------------------------------------------------
 * One query token per sequence: out[b,h,:] = softmax(softmax_scale * q[b,h,:] . K_b^T) K_b[:, :dv]
 * where K_b gathers the first cache_seqlens[b] tokens of sequence b through its page list
 * block_table[b, 0:ceil(len/page_size)] from kv_cache [num_pages, page_size, d]; with an e4m3
 * cache every token is multiplied by kv_scale[page, slot] (fp32).  q [batch, heads, d] and out
 * [batch, heads, dv] are TL_BF16 or TL_F16; cache_dtype TL_E4M3 (kv_scale required), TL_F16 or
 * TL_BF16 (kv_scale may be NULL).  Paging follows the reference's
 * examples/deepseek_mla/example_mla_decode_paged.py:20-97 (block table, cache_seqlens, masked tail)
 * with h_kv = 1; the FP8 cache with per-token scales is the benchmark's extension of it.
 * The tensor-core path (e4m3, d 576, dv 512, heads <= 128, page_size % 64 == 0) needs a scratch
 * buffer, 16-byte aligned, that it may overwrite; other cases ignore it.  Two sizes are accepted:
 * tl_b200_mla_decode_paged_workspace_bytes(batch), the minimum (one int32 per sequence), runs one
 * CTA pair per sequence, longest first;                                                        */
int64_t tl_b200_mla_decode_paged_workspace_bytes(int64_t batch);
/* ... and this larger size (about 145 KB per sequence plus 39 MB) selects the persistent kernel:
 * the query is cut into its two e4m3 terms once per call, the (sequence, 64-token tile) pairs are
 * dealt out in equal contiguous ranges to one CTA pair per two SMs whatever the batch size, and
 * sequences cut by a range boundary are merged from fp32 partials by their log-sum-exp (split-KV
 * as in examples/deepseek_mla/example_mla_decode_paged.py:99-221).  With a 16-bit cache the same scratch
 * lets every sequence be cut into up to 8 shares of its key tiles, merged the same way.  Equals the minimum when the
 * persistent kernel cannot be used (batch above 4096).  max_pages_per_seq and page_size are
 * accepted for symmetry with the call and do not change the size.                              */
int64_t tl_b200_mla_decode_paged_split_workspace_bytes(int64_t batch, int64_t max_pages_per_seq,
                                                       int64_t page_size);
int tl_b200_mla_decode_paged(const void* q, const void* kv_cache, const float* kv_scale,
                             const int32_t* block_table, const int32_t* cache_seqlens, void* out,
                             int64_t batch, int64_t heads, int64_t d, int64_t dv, int64_t page_size,
                             int64_t max_pages_per_seq, int64_t num_pages, float softmax_scale,
                             int q_dtype, int cache_dtype, void* workspace, int64_t workspace_bytes,
                             void* stream);

/* The paged form with several query tokens per sequence and several kv heads
 * (examples/deepseek_mla/example_mla_decode_paged.py:99-256): q [batch, s_q, h_q, d], kv_cache
 * [num_pages, page_size, h_kv, d] of the same 16-bit type, out [batch, s_q, h_q, dv]; head h reads kv head
 * h / (h_q / h_kv); query token i of a sequence sees its keys up to len - s_q + i (the example's causal rule,
 * :266-274).  d 576, dv 512, s_q * (h_q / h_kv) <= 128 (and h_q / h_kv a multiple of 8 when s_q > 1),
 * page_size % 64 == 0 run on tcgen05 tensor cores (also what tl_b200_mla_decode_paged and
 * tl_b200_mla_decode_dense use for 16-bit caches at that shape); other shapes use the FMA kernel.       */
int tl_b200_mla_decode_paged_gqa(const void* q, const void* kv_cache, const int32_t* block_table,
                                 const int32_t* cache_seqlens, void* out, int64_t batch, int64_t s_q, int64_t h_q,
                                 int64_t h_kv, int64_t d, int64_t dv, int64_t page_size, int64_t max_pages_per_seq,
                                 int64_t num_pages, float softmax_scale, int dtype, void* stream);

/* Same computation as tl_b200_mla_decode_paged on its tensor-core configuration (e4m3 cache with
 * per-token scales, d 576, dv 512, heads <= 128, page_size % 64 == 0), for callers that must not
 * allocate device memory when they decode (a pool already handed out to the KV cache, code that
 * runs under another component's allocator lock, hosts that forbid cudaMalloc after warm-up).
 * This entry point has no counterpart in the reference.  It takes no workspace: the sequence
 * ordering scratch is a fixed 16 KB array inside the library image, held by every GPU that
 * loads the library until the process exits, which limits batch to 4096 sequences (larger
 * batches are rejected with TL_B200_EINVAL).  It calls no allocating routine.  The first call on
 * a device looks up the array's device address; make that call before any stream capture.  All
 * calls on a device share the array, so calls that may overlap on the GPU (different streams)
 * race on it; within one stream they are ordered.  A bounded wait that gives up is reported
 * through tl_b200_device_status() only if tl_b200_init() (which creates the host-mapped status
 * word) ran in this process before; this entry point never creates it.                        */
int tl_b200_mla_decode_paged_noalloc(const void* q, const void* kv_cache, const float* kv_scale,
                                     const int32_t* block_table, const int32_t* cache_seqlens,
                                     void* out, int64_t batch, int64_t heads, int64_t page_size,
                                     int64_t max_pages_per_seq, int64_t num_pages, float softmax_scale,
                                     int q_dtype, void* stream);

/* ---- fused row-local tile programs ------------------------------------------------
 * Runs a whole `ppl_*` program whose ops all work row by row - ppl_copy (load, store, cast), ppl_fill,
 * ppl_add / subtract / mul / div with a full, (M,1) or (1,N) second operand, ppl_mul_C / add_C, ppl_exp2,
 * ppl_sigmoid, ppl_rsqrt, ppl_reduce_sum / max, ppl_rope_add (customize.py:136-603) - in ONE launch: a row of
 * every tile lives in registers, every global element is read once and written once.  The reference executes
 * such a program as one runtime call per tile op (codegen_ppl.cc:879-1906).  The host lowers the program to
 * instructions of a small accumulator machine: A is the accumulator row, T[0..n) are tile registers
 * (n = tl_b200_tile_program_registers(max_width)), S[0..8) are per-row scalars ((M,1) tiles).  Results are
 * rounded to `dtype` where an instruction names one (a tile's element type), as the reference's tile ops do.
 *   LD_A / ST_A   A <-> param[base + coef . block + row * row_stride + col], col < width, cast from/to dtype
 *                 (vec != 0 promises 16-byte alignment of every chunk of 8 elements)
 *   LD_S / ST_S   S[r0] <-> param[base + coef . block + row * row_stride]
 *   MOV_A_T  A = T[r0]           MOV_T_A  T[r0] = round(A)        BIN_A_T  A = A (sub) T[r0]
 *   BIN_A_S  A = A (sub) S[r0]   BIN_A_I  A = A (sub) imm         UN_A     A = f_sub(A)
 *   FILL_A   A = imm             ROUND_A  A = round(A)            BCAST_A_S A = S[r0]
 *   RED_S    S[r0] = round(sum (sub 0) or max (sub 1) of A[col < width])
 *   MOV_S_I  S[r0] = imm         MOV_S_S  S[r0] = round(S[r1])    BIN_S_S  S[r0] = round(S[r1] (sub) S[r2])
 *   BIN_S_I  S[r0] = round(S[r1] (sub) imm)                       UN_S     S[r0] = round(f_sub(S[r1]))
 *   ROPE_A   A[2i] = T[r0][2i] + T[r1][2i+1];  A[2i+1] = T[r2][2i+1] + T[r3][2i]
 * binary sub: 0 add, 1 sub, 2 mul, 3 div, 4 max; unary sub: 0 sigmoid, 1 exp, 2 rsqrt.
 * `instrs` and `params` are HOST arrays (params holds device pointers); blocks are numbered x fastest.      */
#define TL_B200_VM_MAX_INSTR 96
#define TL_B200_VM_MAX_PARAMS 16
enum {
  TL_VM_LD_A = 0, TL_VM_ST_A, TL_VM_LD_S, TL_VM_ST_S, TL_VM_MOV_A_T, TL_VM_MOV_T_A, TL_VM_BIN_A_T, TL_VM_BIN_A_S,
  TL_VM_BIN_A_I, TL_VM_UN_A, TL_VM_FILL_A, TL_VM_ROUND_A, TL_VM_BCAST_A_S, TL_VM_RED_S, TL_VM_MOV_S_I, TL_VM_MOV_S_S,
  TL_VM_BIN_S_S, TL_VM_BIN_S_I, TL_VM_UN_S, TL_VM_ROPE_A, TL_VM_OPCODES
};
typedef struct {
  int32_t op, sub;
  int32_t r0, r1, r2, r3;
  int32_t dtype, width;
  int32_t param, row_stride;
  int32_t vec;
  float imm;
  int64_t base;
  int64_t coef[3];
} tl_b200_vm_instr;
int tl_b200_tile_program_registers(int64_t max_width);
int tl_b200_tile_program(const tl_b200_vm_instr* instrs, int n_instr, const void* const* params, int n_params,
                         int grid_x, int grid_y, int grid_z, int rows_per_block, int64_t max_width, void* stream);

/* ---- generic entry point ---------------------------------------------------------
 * One symbol with the shape of the reference's generated
 *     extern "C" int tilelang_tpu_run(void** args)
 * (src/tl_templates/tpu/main_template.cpp:39; ctypes prototype argtypes=[POINTER(c_void_p)],
 * restype=c_int at tilelang/jit/adapter/cython/adapter.py:215-216), for bindings that want to keep
 * a single prototype.  `args` holds the POINTER arguments of the typed entry point `kernel_id`
 * names, in declaration order (a workspace pointer, where there is one, comes last); `meta` holds
 * its non-pointer arguments in declaration order (the workspace size, where there is one, comes
 * last), integers as they are and every float as its IEEE-754 bit pattern in the low 32 bits.
 * The generated symbol has its program's sizes baked in; a pre-built library cannot, hence `meta`. */
#define TL_B200_K_RMSNORM 1
#define TL_B200_K_ROPE 2
#define TL_B200_K_SWIGLU 3
#define TL_B200_K_REDUCE_ROWS 4
#define TL_B200_K_UNARY 5
#define TL_B200_K_BINARY 6
#define TL_B200_K_ROPE_ADD 7
#define TL_B200_K_COPY2D 8
#define TL_B200_K_FILL 9
#define TL_B200_K_GATHER_ROWS 10
#define TL_B200_K_TOPK 11
#define TL_B200_K_GEMM 12
#define TL_B200_K_MLP_GATE_UP 13
#define TL_B200_K_GEMM_FP8_BLOCKSCALE 14
#define TL_B200_K_FLASH_ATTN_FWD 15
#define TL_B200_K_MLA_DECODE_DENSE 16
#define TL_B200_K_MLA_DECODE_PAGED 17
int tl_b200_run(int kernel_id, void** args, const int64_t* meta, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TL_B200_H_ */
