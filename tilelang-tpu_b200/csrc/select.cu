// Index-producing / index-consuming programs: row gather and top-k.  Integer results are
// deterministic and bit-exact by construction (no atomics, no data-dependent ordering).
#include "common.cuh"

namespace tl {

constexpr int kThreads = 256;

// =================================================================================
// gather: out[i,:] = param[index[i],:]
// =================================================================================
template <int UNROLL>
__global__ void __launch_bounds__(kThreads)
gather_vec_kernel(const uint4* __restrict__ param, const uint32_t* __restrict__ index, uint4* __restrict__ out,
                  int64_t total_vec, int vec_per_row, uint32_t param_rows) {
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t base = (int64_t)blockIdx.x * kThreads + threadIdx.x; base < total_vec;
       base += stride * UNROLL) {
    uint4 v[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      int64_t i = base + u * stride;
      v[u] = make_uint4(0, 0, 0, 0);
      if (i < total_vec) {
        int64_t r = i / vec_per_row;
        int c = (int)(i - r * vec_per_row);
        uint32_t src = __ldg(index + r);
        if (src < param_rows) v[u] = ld_stream16(param + (int64_t)src * vec_per_row + c);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      int64_t i = base + u * stride;
      if (i < total_vec) st_stream16(out + i, v[u]);
    }
  }
}

__global__ void __launch_bounds__(kThreads)
gather_byte_kernel(const uint8_t* __restrict__ param, const uint32_t* __restrict__ index,
                   uint8_t* __restrict__ out, int64_t total, int64_t row_bytes, uint32_t param_rows) {
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride) {
    int64_t r = i / row_bytes;
    int64_t c = i - r * row_bytes;
    uint32_t src = __ldg(index + r);
    out[i] = src < param_rows ? param[(int64_t)src * row_bytes + c] : (uint8_t)0;
  }
}

// =================================================================================
// top-k.  Every element gets a unique 64-bit key (order-preserving image of the value in the
// high word, inverted position in the low word), so "the next winner" is simply the largest
// key strictly below the previous winner's: k rounds of a max-reduction, no marking, no
// scratch memory, and ties resolve to the lower index.
// =================================================================================
template <int DTYPE> __device__ __forceinline__ uint32_t order_bits(uint32_t b) {
  if constexpr (DTYPE == TL_F32) return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  else if constexpr (DTYPE == TL_I32) return b ^ 0x80000000u;
  else return b;
}

__device__ __forceinline__ uint64_t make_key(uint32_t ord, uint32_t pos) {
  return ((uint64_t)ord << 32) | (uint64_t)(0xffffffffu - pos);
}

__device__ __forceinline__ uint64_t warp_max_u64(uint64_t v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    uint64_t other = __shfl_xor_sync(0xffffffffu, v, o);
    v = other > v ? other : v;
  }
  return v;
}

// One warp per row, the row's keys in registers (length <= 32 * ITEMS).
template <int DTYPE, int ITEMS>
__global__ void __launch_bounds__(kThreads)
topk_warp_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ out_vals, int32_t* __restrict__ out_idx,
                 int64_t rows, int length, int k, bool descending, int64_t out_stride) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + threadIdx.x / 32;
  if (row >= rows) return;
  const uint32_t* in = src + row * length;
  uint32_t ord[ITEMS];
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    int pos = lane + 32 * j;
    uint32_t o = 0;
    if (pos < length) {
      o = order_bits<DTYPE>(in[pos]);
      if (!descending) o = ~o;
    }
    ord[j] = o;
  }
  uint64_t prev = ~0ull;
  for (int r = 0; r < k; ++r) {
    uint64_t best = 0;
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
      int pos = lane + 32 * j;
      uint64_t key = make_key(ord[j], (uint32_t)pos);
      if (pos < length && key < prev && key > best) best = key;
    }
    best = warp_max_u64(best);
    prev = best;
    if (lane == 0) {
      uint32_t pos = 0xffffffffu - (uint32_t)(best & 0xffffffffu);
      out_idx[row * out_stride + r] = (int32_t)pos;
      out_vals[row * out_stride + r] = in[pos];
    }
  }
}

// One CTA per row; keys are rebuilt from the row on every round (the row stays in L1/L2).
template <int DTYPE>
__global__ void __launch_bounds__(kThreads)
topk_cta_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ out_vals, int32_t* __restrict__ out_idx,
                int64_t length, int k, bool descending, int64_t out_stride) {
  __shared__ uint64_t warp_best[kThreads / 32];
  __shared__ uint64_t round_best;
  const int64_t row = blockIdx.x;
  const uint32_t* in = src + row * length;
  uint64_t prev = ~0ull;
  for (int r = 0; r < k; ++r) {
    uint64_t best = 0;
    for (int64_t pos = threadIdx.x; pos < length; pos += kThreads) {
      uint32_t o = order_bits<DTYPE>(__ldg(in + pos));
      if (!descending) o = ~o;
      uint64_t key = make_key(o, (uint32_t)pos);
      if (key < prev && key > best) best = key;
    }
    best = warp_max_u64(best);
    if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x / 32] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
      uint64_t b = 0;
#pragma unroll
      for (int w = 0; w < kThreads / 32; ++w) b = warp_best[w] > b ? warp_best[w] : b;
      round_best = b;
      uint32_t pos = 0xffffffffu - (uint32_t)(b & 0xffffffffu);
      out_idx[row * out_stride + r] = (int32_t)pos;
      out_vals[row * out_stride + r] = in[pos];
    }
    __syncthreads();
    prev = round_best;
  }
}

template <int DTYPE>
static int topk_dispatch(const void* src, void* vals, int32_t* idx, int64_t rows, int64_t length, int k,
                         bool desc, int64_t out_stride, cudaStream_t s) {
  const uint32_t* in = (const uint32_t*)src;
  uint32_t* ov = (uint32_t*)vals;
  if (length <= 1024) {
    int64_t grid = (rows + kThreads / 32 - 1) / (kThreads / 32);
    TL_REQUIRE(grid < (1ll << 31), "topk: too many rows");
    if (length <= 256)
      topk_warp_kernel<DTYPE, 8><<<(unsigned)grid, kThreads, 0, s>>>(in, ov, idx, rows, (int)length, k, desc,
                                                                   out_stride);
    else
      topk_warp_kernel<DTYPE, 32><<<(unsigned)grid, kThreads, 0, s>>>(in, ov, idx, rows, (int)length, k, desc,
                                                                    out_stride);
    TL_LAUNCH_CHECK("topk_warp_kernel");
  } else {
    TL_REQUIRE(rows < (1ll << 31), "topk: too many rows");
    topk_cta_kernel<DTYPE><<<(unsigned)rows, kThreads, 0, s>>>(in, ov, idx, length, k, desc, out_stride);
    TL_LAUNCH_CHECK("topk_cta_kernel");
  }
  return TL_B200_OK;
}

}  // namespace tl

using namespace tl;

extern "C" {

int tl_b200_gather_rows(const void* param, const uint32_t* index, void* out, int64_t n_index, int64_t row_bytes,
                        int64_t param_rows, void* stream) {
  TL_REQUIRE(n_index >= 0 && row_bytes >= 0 && param_rows >= 0, "gather_rows: negative size");
  TL_REQUIRE(param_rows <= 0xffffffffll, "gather_rows: param_rows exceeds the uint32 index range");
  if (n_index == 0 || row_bytes == 0) return TL_B200_OK;
  TL_REQUIRE(param && index && out, "gather_rows: null tensor pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (row_bytes % 16 == 0 && aligned16(param) && aligned16(out) && row_bytes / 16 < (1ll << 31)) {
    constexpr int UNROLL = 4;
    int64_t total = n_index * (row_bytes / 16);
    int64_t need = (total + kThreads * UNROLL - 1) / (kThreads * UNROLL);
    unsigned grid = (unsigned)(need < cap ? need : cap);
    gather_vec_kernel<UNROLL><<<grid, kThreads, 0, s>>>((const uint4*)param, index, (uint4*)out, total,
                                                       (int)(row_bytes / 16), (uint32_t)param_rows);
    TL_LAUNCH_CHECK("gather_vec_kernel");
  } else {
    int64_t total = n_index * row_bytes;
    int64_t need = (total + kThreads - 1) / kThreads;
    unsigned grid = (unsigned)(need < cap ? need : cap);
    gather_byte_kernel<<<grid, kThreads, 0, s>>>((const uint8_t*)param, index, (uint8_t*)out, total, row_bytes,
                                                 (uint32_t)param_rows);
    TL_LAUNCH_CHECK("gather_byte_kernel");
  }
  return TL_B200_OK;
}

int tl_b200_topk(const void* src, void* out_vals, int32_t* out_idx, int64_t rows, int64_t length, int k,
                 int descending, int64_t out_stride, int dtype, void* stream) {
  TL_REQUIRE(rows >= 0 && length >= 0 && k >= 0, "topk: negative size");
  TL_REQUIRE(k <= length, "topk: k (%d) exceeds length (%lld)", k, (long long)length);
  TL_REQUIRE(out_stride >= k, "topk: out_stride (%lld) smaller than k (%d)", (long long)out_stride, k);
  TL_REQUIRE(length < 0xffffffffll, "topk: length exceeds the 32-bit position range");
  if (rows == 0 || k == 0) return TL_B200_OK;
  TL_REQUIRE(src && out_vals && out_idx, "topk: null tensor pointer");
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case TL_F32: return topk_dispatch<TL_F32>(src, out_vals, out_idx, rows, length, k, descending != 0, out_stride, s);
    case TL_I32: return topk_dispatch<TL_I32>(src, out_vals, out_idx, rows, length, k, descending != 0, out_stride, s);
    case TL_U32: return topk_dispatch<TL_U32>(src, out_vals, out_idx, rows, length, k, descending != 0, out_stride, s);
    default: return fail(TL_B200_EINVAL, "topk: dtype %d not supported (float32, int32, uint32 only)", dtype);
  }
}

}  // extern "C"
