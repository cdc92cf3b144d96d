// Constants and small device helpers shared by the two tensor-core MLA decode kernels.
#pragma once
#include "sm100.cuh"

namespace tl {
using namespace sm100;

constexpr int kMlaD = 576, kMlaDV = 512, kMlaHeads = 128, kMlaBN = 64;
constexpr int kMlaSlabs = 5;                     // 128-byte column slabs per token row (last one half used)
constexpr int kMlaStages = 3;
constexpr int kMlaTile = kMlaSlabs * kMlaBN * 128;          // 40 KB of cache bytes per stage
constexpr int kMlaStageBytes = kMlaTile + kMlaBN * 4;       // + 64 token scales
constexpr int kMlaQBytes = kMlaSlabs * kMlaHeads * 128;     // 80 KB: e4m3 Q (value term; slab 4 also holds
                                                            // the residual term of columns 512..575)
constexpr int kMlaOffKV = kMlaQBytes;
constexpr int kMlaOffBar = kMlaOffKV + kMlaStages * (kMlaTile + 1024);   // scale area padded to 1 KB
constexpr int kMlaSmem = kMlaOffBar + 6144 + 1024;
constexpr int kMlaThreads = 384;                 // warp 0 TMA, warp 1 MMA, warp 2 TMEM alloc, warps 4-11 softmax
constexpr int kMlaSoftmaxThreads = 256;          // two warpgroups: tokens 0-31 and 32-63 of every tile
constexpr int kMlaSoftmaxWarps = kMlaSoftmaxThreads / 32;   // barriers count one arrival per warp
constexpr int kMlaTmemCols = 512;
// tensor memory: S buffers [0,64) and [64,128) (P overwrites the first 32 columns of its S buffer),
// residual term of Q for columns 0..511 in [128,256), O in [256,512)
constexpr int kMlaColS = 0, kMlaColQlo = 128, kMlaColO = 256;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}
__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t v) {
  __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v & 0xffffu), __NV_E4M3);
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}

// Sequence lengths and page ids live in device memory, so the host cannot validate them.  A length is
// clamped to what the block-table row and the cache can hold; a page id outside the cache marks its tile
// as masked (the loads are redirected to row 0 of the cache and the scores of the tile become -inf).
__device__ __forceinline__ int mla_len(const int* __restrict__ seqlens, int b, int cap) {
  return min(max(__ldg(seqlens + b), 0), cap);
}
__device__ __forceinline__ bool mla_page_ok(int page, int num_pages) { return (unsigned)page < (unsigned)num_pages; }
inline int mla_len_cap(int64_t max_pages_per_seq, int64_t num_pages, int64_t page_size) {
  const int64_t cap = (max_pages_per_seq < num_pages ? max_pages_per_seq : num_pages) * page_size;
  return (int)(cap < 0x7fffffc0ll ? cap : 0x7fffffc0ll);
}

// Launches the persistent, work-balanced decode (mla_persistent.cu).  `workspace` must hold
// mla_persistent_workspace_bytes(batch) bytes.  Returns 0 or a TL_B200_E code.
int64_t mla_persistent_workspace_bytes(int64_t batch);
bool mla_persistent_supported(int64_t batch);
int mla_persistent_launch(const void* q, const void* kv_cache, const float* kv_scale, const int32_t* block_table,
                          const int32_t* cache_seqlens, void* out, int64_t batch, int64_t heads, int64_t page_size,
                          int64_t max_pages_per_seq, int64_t num_pages, float softmax_scale, int q_dtype,
                          void* workspace, cudaStream_t stream);

// 16-bit caches on tcgen05 (mla_f16.cu): q [batch, s_q, h_q, 576] or split (q 512 + q_pe 64 columns); cache
// [tokens, h_kv, 576] or split; paged (block_table, seqlens) or dense (both nullptr, dense_len tokens each).
int64_t mla_f16_workspace_bytes(int64_t units);
bool mla_f16_shape_ok(int64_t s_q, int64_t h_q, int64_t h_kv, int64_t d, int64_t dv);
int mla_order_launch(const int* seqlens, int* order, int batch, cudaStream_t s);
int mla_f16_launch(const void* q, const void* q_pe, const void* kv, const void* k_pe, const int32_t* block_table,
                   const int32_t* seqlens, void* out, int64_t batch, int64_t s_q, int64_t h_q, int64_t h_kv,
                   int64_t total_tokens, int64_t page_size, int64_t max_pages, int64_t num_pages, int64_t dense_len,
                   float softmax_scale, int dtype, cudaStream_t stream, void* workspace = nullptr,
                   int64_t workspace_bytes = 0);

}  // namespace tl
