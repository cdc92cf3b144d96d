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
// top-k.  Values are mapped to an order-preserving unsigned image (inverted for an ascending
// search); candidates compare by (image, position): larger image first, lower position on ties.
// k rounds of an arg-max reduction; a taken element is masked out in its owner's registers, the
// winners are recovered from their images (no second read of the row) and stay in registers - result
// r in lane r % 32 - until they are written out, 32 at a time.
// =================================================================================
template <int DTYPE> __device__ __forceinline__ uint32_t order_bits(uint32_t b) {
  if constexpr (DTYPE == TL_F32) return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  else if constexpr (DTYPE == TL_I32) return b ^ 0x80000000u;
  else return b;
}
template <int DTYPE> __device__ __forceinline__ uint32_t value_bits(uint32_t o) {      // inverse of order_bits
  if constexpr (DTYPE == TL_F32) return (o & 0x80000000u) ? (o ^ 0x80000000u) : ~o;
  else if constexpr (DTYPE == TL_I32) return o ^ 0x80000000u;
  else return o;
}

constexpr uint32_t kNoPos = 0xffffffffu;       // "no candidate": loses every comparison

// (o, p) <- the better of (o, p) and (o2, p2)
__device__ __forceinline__ void take_better(uint32_t& o, uint32_t& p, uint32_t o2, uint32_t p2) {
  const bool other = (p2 != kNoPos) && (p == kNoPos || o2 > o || (o2 == o && p2 < p));
  o = other ? o2 : o;
  p = other ? p2 : p;
}
__device__ __forceinline__ void warp_argmax(uint32_t& o, uint32_t& p) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const uint32_t o2 = __shfl_xor_sync(0xffffffffu, o, d), p2 = __shfl_xor_sync(0xffffffffu, p, d);
    take_better(o, p, o2, p2);
  }
}

// One warp per row, the row's images in registers (length <= 32 * ITEMS); element j of a lane sits at
// position lane + 32 j, so a lane's candidates are scanned in increasing position.
template <int DTYPE, int ITEMS>
__global__ void __launch_bounds__(kThreads)
topk_warp_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ out_vals, int32_t* __restrict__ out_idx,
                 int64_t rows, int length, int k, bool descending, int64_t out_stride) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + threadIdx.x / 32;
  if (row >= rows) return;
  const uint32_t* in = src + row * length;
  uint32_t ord[ITEMS];
  uint32_t live = 0;                            // bit j: element j exists and has not been taken
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    const int pos = lane + 32 * j;
    uint32_t o = 0;
    if (pos < length) {
      o = order_bits<DTYPE>(__ldg(in + pos));
      if (!descending) o = ~o;
      live |= 1u << j;
    }
    ord[j] = o;
  }
  uint32_t res_o = 0, res_p = 0;
  for (int r = 0; r < k; ++r) {
    uint32_t bo = 0, bj = ITEMS;
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {           // first of the equal images wins: lowest position of the lane
      const bool better = ((live >> j) & 1u) && (bj == ITEMS || ord[j] > bo);
      bo = better ? ord[j] : bo;
      bj = better ? j : bj;
    }
    uint32_t wo = bo, wp = bj == ITEMS ? kNoPos : (uint32_t)(lane + 32 * bj);
    warp_argmax(wo, wp);
    if ((wp & 31u) == (uint32_t)lane) live &= ~(1u << (wp >> 5));       // k <= length: a winner always exists
    if ((r & 31) == lane) { res_o = wo; res_p = wp; }
    if ((r & 31) == 31 || r == k - 1) {         // write the last (up to) 32 winners, one per lane
      const int first = r & ~31;
      if (first + lane <= r) {
        out_idx[row * out_stride + first + lane] = (int32_t)res_p;
        out_vals[row * out_stride + first + lane] = value_bits<DTYPE>(descending ? res_o : ~res_o);
      }
    }
  }
}

// One CTA per row of up to 256 * ITEMS elements, images in registers (element j of a thread sits at
// position thread + 256 j); longer rows are re-read from L1/L2 on every round (ITEMS == 0).
template <int DTYPE, int ITEMS>
__global__ void __launch_bounds__(kThreads)
topk_cta_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ out_vals, int32_t* __restrict__ out_idx,
                int64_t length, int k, bool descending, int64_t out_stride) {
  __shared__ uint32_t warp_o[2][kThreads / 32], warp_p[2][kThreads / 32];
  const int64_t row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x / 32;
  const uint32_t* in = src + row * length;
  constexpr int NREG = ITEMS > 0 ? ITEMS : 1;
  uint32_t ord[NREG];
  uint32_t live = 0;
  if constexpr (ITEMS > 0) {
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
      const int64_t pos = threadIdx.x + (int64_t)kThreads * j;
      uint32_t o = 0;
      if (pos < length) {
        o = order_bits<DTYPE>(__ldg(in + pos));
        if (!descending) o = ~o;
        live |= 1u << j;
      }
      ord[j] = o;
    }
  }
  uint32_t prev_o = 0, prev_p = kNoPos;          // generic path: the last winner; everything at or above it is gone
  uint32_t res_o = 0, res_p = 0;
  for (int r = 0; r < k; ++r) {
    uint32_t bo = 0, bp = kNoPos;
    if constexpr (ITEMS > 0) {
      uint32_t bj = ITEMS;
#pragma unroll
      for (int j = 0; j < ITEMS; ++j) {
        const bool better = ((live >> j) & 1u) && (bj == ITEMS || ord[j] > bo);
        bo = better ? ord[j] : bo;
        bj = better ? j : bj;
      }
      bp = bj == ITEMS ? kNoPos : (uint32_t)(threadIdx.x + kThreads * bj);
    } else {
      for (int64_t pos = threadIdx.x; pos < length; pos += kThreads) {
        uint32_t o = order_bits<DTYPE>(__ldg(in + pos));
        if (!descending) o = ~o;
        // still available: strictly after the previous winner in (image desc, position asc) order
        const bool avail = prev_p == kNoPos || o < prev_o || (o == prev_o && (uint32_t)pos > prev_p);
        if (avail) take_better(bo, bp, o, (uint32_t)pos);
      }
    }
    warp_argmax(bo, bp);
    const int buf = r & 1;                      // two exchange buffers: one barrier per round is enough
    if (lane == 0) { warp_o[buf][warp] = bo; warp_p[buf][warp] = bp; }
    __syncthreads();
    uint32_t wo = warp_o[buf][0], wp = warp_p[buf][0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) take_better(wo, wp, warp_o[buf][w], warp_p[buf][w]);
    if constexpr (ITEMS > 0) {
      if ((wp % kThreads) == threadIdx.x) live &= ~(1u << (wp / kThreads));
    } else {
      prev_o = wo; prev_p = wp;
    }
    if (warp == 0) {
      if ((r & 31) == lane) { res_o = wo; res_p = wp; }
      if ((r & 31) == 31 || r == k - 1) {
        const int first = r & ~31;
        if (first + lane <= r) {
          out_idx[row * out_stride + first + lane] = (int32_t)res_p;
          out_vals[row * out_stride + first + lane] = value_bits<DTYPE>(descending ? res_o : ~res_o);
        }
      }
    }
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
    if (length <= 16 * kThreads)
      topk_cta_kernel<DTYPE, 16><<<(unsigned)rows, kThreads, 0, s>>>(in, ov, idx, length, k, desc, out_stride);
    else
      topk_cta_kernel<DTYPE, 0><<<(unsigned)rows, kThreads, 0, s>>>(in, ov, idx, length, k, desc, out_stride);
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
