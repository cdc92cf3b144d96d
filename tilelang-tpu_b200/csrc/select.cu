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

// Rows of at least 32 vectors: one warp per output row (the source row is looked up once and no index arithmetic is
// done per vector: a 64-bit division per 16 bytes made the kernel above issue-bound), UNROLL loads in flight per lane.
template <int UNROLL>
__global__ void __launch_bounds__(kThreads)
gather_rows_kernel(const uint4* __restrict__ param, const uint32_t* __restrict__ index, uint4* __restrict__ out,
                   int64_t n_index, int vec_per_row, uint32_t param_rows) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (kThreads / 32);
  for (int64_t r = (int64_t)blockIdx.x * (kThreads / 32) + threadIdx.x / 32; r < n_index; r += warps) {
    const uint32_t src = __ldg(index + r);
    const bool ok = src < param_rows;                       // an index outside the table gives a row of zeros
    const uint4* from = param + (int64_t)(ok ? src : 0) * vec_per_row;
    uint4* to = out + r * vec_per_row;
    for (int c = lane; c < vec_per_row; c += 32 * UNROLL) {
      uint4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        v[u] = make_uint4(0, 0, 0, 0);
        if (ok && c + 32 * u < vec_per_row) v[u] = ld_stream16(from + c + 32 * u);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (c + 32 * u < vec_per_row) st_stream16(to + c + 32 * u, v[u]);
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


// ---- threshold selection (k <= 32, one warp per row) -------------------------------------------------------------
// The k-th largest of the 32 lane maxima, T, is a lower bound of the k-th largest element (k lanes hold an element
// >= T), so only elements >= T can be winners: about k of them for small k, about 120 for k = 32 on random data.  They
// are appended to the warp's 256 slots of shared memory and sorted there (one rank count or one bitonic network over
// the lanes), instead of k rounds of arg-max over the whole row.  Rows with more than 256 candidates (many equal
// values) fall back to k rounds over the row.  Candidates compare by (image, position): larger image first, lower
// position on ties, as everywhere in this file.
constexpr int kSlots = 256;

__device__ __forceinline__ bool pair_before(uint32_t o, uint32_t p, uint32_t o2, uint32_t p2) {     // (o, p) sorts before (o2, p2)
  return o > o2 || (o == o2 && p < p2);
}

// Bitonic sort of E (image, position) pairs per lane, element lane * E + e of the sequence in o[e]; best pair first.
template <int E>
__device__ __forceinline__ void warp_sort_pairs(uint32_t (&o)[E], uint32_t (&p)[E], int lane) {
#pragma unroll
  for (int size = 2; size <= 32 * E; size <<= 1) {
#pragma unroll
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (stride >= E) {                                   // partner in another lane
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const uint32_t o2 = __shfl_xor_sync(0xffffffffu, o[e], stride / E);
          const uint32_t p2 = __shfl_xor_sync(0xffffffffu, p[e], stride / E);
          const int at = lane * E + e;
          const bool lower = (at & stride) == 0;           // this side keeps the pair that sorts first ...
          const bool forward = (at & size) == 0;           // ... when its block sorts forward
          const bool mine_first = pair_before(o[e], p[e], o2, p2);
          const bool keep = (lower == forward) ? mine_first : !mine_first;
          o[e] = keep ? o[e] : o2;
          p[e] = keep ? p[e] : p2;
        }
      } else {                                             // partner in this lane
#pragma unroll
        for (int e = 0; e < E; ++e) {
          if ((e & stride) == 0) {
            const int f = e | stride;
            const bool forward = ((lane * E + e) & size) == 0;
            const bool in_order = pair_before(o[e], p[e], o[f], p[f]);
            const bool swap = forward ? !in_order : in_order;
            const uint32_t oe = o[e], pe = p[e];
            o[e] = swap ? o[f] : oe;  p[e] = swap ? p[f] : pe;
            o[f] = swap ? oe : o[f];  p[f] = swap ? pe : p[f];
          }
        }
      }
    }
  }
}

// The k-th largest (with multiplicity) of one value per lane.  Small k: rounds of a warp-wide maximum that retire
// every lane holding it; larger k: one sort.  Lanes without elements pass 0 and can only lower the result, which
// keeps it a valid threshold.
__device__ __forceinline__ uint32_t kth_largest_of_lanes(uint32_t v, int k, int lane) {
  if (k <= 10) {
    bool alive = true;
    int seen = 0;
    uint32_t m = 0;
    for (int r = 0; r < k; ++r) {
      m = __reduce_max_sync(0xffffffffu, alive ? v : 0u);
      const uint32_t hit = __ballot_sync(0xffffffffu, alive && v == m);
      seen += __popc(hit);
      if (seen >= k || hit == 0u) break;
      alive = alive && v != m;
    }
    return m;
  }
  uint32_t so[1] = {v}, sp[1] = {(uint32_t)lane};
  warp_sort_pairs<1>(so, sp, lane);
  return __shfl_sync(0xffffffffu, so[0], k - 1);
}

template <int DTYPE, int E>
__device__ __noinline__ void sort_slots_and_write(const uint32_t* slot_o, const uint32_t* slot_p, int total, int k, int lane,
                                                     bool descending, uint32_t* out_vals, int32_t* out_idx) {
  // an empty slot (image 0, position kNoPos) sorts after every real element: kNoPos is above every real position
  uint32_t o[E], p[E];
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const int at = lane * E + e;
    o[e] = at < total ? slot_o[at] : 0u;
    p[e] = at < total ? slot_p[at] : kNoPos;
  }
  warp_sort_pairs<E>(o, p, lane);
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const int at = lane * E + e;
    if (at < k) {
      out_idx[at] = (int32_t)p[e];
      out_vals[at] = value_bits<DTYPE>(descending ? o[e] : ~o[e]);
    }
  }
}

// The image of the k-th best of a warp's kSlots full slots: at least k elements of the row reach it, so it is a
// valid (and higher) threshold when the first one let too many candidates through.
__device__ __noinline__ uint32_t kth_image_of_full_slots(const uint32_t* slot_o, const uint32_t* slot_p, int k, int lane) {
  constexpr int E = kSlots / 32;
  uint32_t o[E], p[E];
#pragma unroll
  for (int e = 0; e < E; ++e) { o[e] = slot_o[lane * E + e]; p[e] = slot_p[lane * E + e]; }
  warp_sort_pairs<E>(o, p, lane);
  uint32_t v = 0;
#pragma unroll
  for (int e = 0; e < E; ++e) v = ((k - 1) % E == e) ? o[e] : v;
  return __shfl_sync(0xffffffffu, v, (k - 1) / E);
}

// The best k of `total` <= kSlots candidates in a warp's slots, written in order.  Few candidates: every lane ranks
// its own candidate against all of them (positions are distinct, so ranks are); more: one sort.
template <int DTYPE>
__device__ __forceinline__ void write_best_of_slots(const uint32_t* slot_o, const uint32_t* slot_p, int total, int k, int lane,
                                                    bool descending, uint32_t* out_vals, int32_t* out_idx) {
  if (total <= 16) {
    const uint32_t o = lane < total ? slot_o[lane] : 0u, p = lane < total ? slot_p[lane] : kNoPos;
    int rank = 0;
#pragma unroll 4
    for (int i = 0; i < total; ++i) rank += pair_before(slot_o[i], slot_p[i], o, p) ? 1 : 0;
    if (lane < total && rank < k) {
      out_idx[rank] = (int32_t)p;
      out_vals[rank] = value_bits<DTYPE>(descending ? o : ~o);
    }
  } else if (total <= 32) {
    sort_slots_and_write<DTYPE, 1>(slot_o, slot_p, total, k, lane, descending, out_vals, out_idx);
  } else if (total <= 128) {
    sort_slots_and_write<DTYPE, 4>(slot_o, slot_p, total, k, lane, descending, out_vals, out_idx);
  } else {
    sort_slots_and_write<DTYPE, 8>(slot_o, slot_p, total, k, lane, descending, out_vals, out_idx);
  }
}

// A warp's view of one row: lane L reads cells of 4 consecutive elements, cell c at position (c * 32 + L) * 4, as one
// 16-byte load when the row allows it.
template <int DTYPE, bool VEC>
struct RowCells {
  const uint32_t* in;
  int length, lane;
  uint32_t flip;                                           // ascending order: complemented images
  __device__ __forceinline__ int pos0(int cell) const { return (cell * 32 + lane) * 4; }
  __device__ __forceinline__ void load(int cell, uint32_t (&raw)[4]) const {
    const int at = pos0(cell);
    if constexpr (VEC) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (at < length) v = __ldg(reinterpret_cast<const uint4*>(in + at));
      raw[0] = v.x; raw[1] = v.y; raw[2] = v.z; raw[3] = v.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) raw[e] = at + e < length ? __ldg(in + at + e) : 0u;
    }
  }
  __device__ __forceinline__ uint32_t image(uint32_t raw) const { return order_bits<DTYPE>(raw) ^ flip; }
  // visit(cell, images[4]) for every cell of the row, 8 cells per lane in flight; elements past the end of the row have
  // image 0 and must be told apart by position (`exists`)
  __device__ __forceinline__ bool exists(int cell, int e) const { return pos0(cell) + e < length; }
  template <class F>
  __device__ __forceinline__ void for_each_cell(F&& visit) const {
    for (int base = 0; base * 128 < length; base += 8) {
      uint32_t raw[8][4];
#pragma unroll
      for (int u = 0; u < 8; ++u) load(base + u, raw[u]);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
#pragma unroll
        for (int e = 0; e < 4; ++e) raw[u][e] = exists(base + u, e) ? image(raw[u][e]) : 0u;
        visit(base + u, raw[u]);
      }
    }
  }
};

// More than kSlots candidates: k rounds, each one pass over the row that picks the best element strictly after the
// previous winner in the (image, position) order, so no "taken" state is kept.
template <int DTYPE, bool VEC>
__device__ __noinline__ void topk_by_rounds(const RowCells<DTYPE, VEC>& row, int k, bool descending, uint32_t* out_vals,
                                            int32_t* out_idx) {
  uint32_t prev_o = 0, prev_p = 0, res_o = 0, res_p = kNoPos;
  for (int r = 0; r < k; ++r) {
    uint32_t bo = 0, bp = kNoPos;
    row.for_each_cell([&](int cell, const uint32_t (&o)[4]) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t pos = (uint32_t)(row.pos0(cell) + e);
        const bool after = r == 0 || pair_before(prev_o, prev_p, o[e], pos);
        const bool better = row.exists(cell, e) && after && (bp == kNoPos || pair_before(o[e], pos, bo, bp));
        bo = better ? o[e] : bo;
        bp = better ? pos : bp;
      }
    });
    warp_argmax(bo, bp);
    prev_o = bo; prev_p = bp;
    if (row.lane == (r & 31)) { res_o = bo; res_p = bp; }
  }
  if (row.lane < k) {
    out_idx[row.lane] = (int32_t)res_p;
    out_vals[row.lane] = value_bits<DTYPE>(descending ? res_o : ~res_o);
  }
}

struct WarpSlots {
  uint32_t o[kThreads / 32][kSlots], p[kThreads / 32][kSlots];
};
// Every lane of the warp calls this together; lanes with `hit` append (o, pos) behind the `count` pairs already there.
// The count is the same in every lane, so no shared counter and no atomics are needed.
__device__ __forceinline__ void append_slots(WarpSlots& sl, int warp, int lane, int& count, bool hit, uint32_t o, uint32_t pos) {
  const uint32_t m = __ballot_sync(0xffffffffu, hit);
  if (m == 0u) return;
  const int slot = count + __popc(m & ((1u << lane) - 1u));
  if (hit && slot < kSlots) { sl.o[warp][slot] = o; sl.p[warp][slot] = pos; }
  count += __popc(m);
}

// Rows of up to 128 * CELLS elements, read from memory ONCE: a lane keeps the maximum of each of its cells, and after T
// is known reads again (from L1 / L2) only the cells whose maximum reaches T.  Above 32 cells only the upper 16 bits
// of a maximum are kept, two per register: comparing them with T's upper bits selects a superset of the cells.
template <int DTYPE, int CELLS, bool VEC>
__global__ void __launch_bounds__(kThreads, CELLS > 32 ? 2 : CELLS == 32 ? 3 : 4)
topk_cells_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ out_vals, int32_t* __restrict__ out_idx,
                  int64_t rows, int length, int k, bool descending, int64_t out_stride) {
  __shared__ WarpSlots sl;
  const int lane = threadIdx.x & 31, warp = threadIdx.x / 32;
  const int64_t r = (int64_t)blockIdx.x * (kThreads / 32) + warp;
  if (r >= rows) return;
  const RowCells<DTYPE, VEC> row{src + r * length, length, lane, descending ? 0u : ~0u};
  constexpr bool kPacked = CELLS > 32;
  static_assert(CELLS <= 64 && (CELLS % 2 == 0), "one 64-bit mask of cells per lane");
  uint32_t cell_max[kPacked ? CELLS / 2 : CELLS], lm = 0;
  constexpr int kBatch = CELLS < 8 ? CELLS : 8;
#pragma unroll
  for (int c0 = 0; c0 < CELLS; c0 += kBatch) {
    uint32_t raw[kBatch][4];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) row.load(c0 + u, raw[u]);
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      uint32_t m = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (row.pos0(c0 + u) + e < length) m = max(m, row.image(raw[u][e]));
      if constexpr (!kPacked) cell_max[c0 + u] = m;
      else if ((c0 + u) % 2 == 0) cell_max[(c0 + u) / 2] = m >> 16;
      else cell_max[(c0 + u) / 2] |= m & 0xffff0000u;
      lm = max(lm, m);
    }
  }
  // candidates >= T into the slots; every lane walks its own list of cells that reach T, all lanes in step: one load
  // latency per step, not per cell
  auto collect = [&](uint32_t T) {
    unsigned long long need = 0;
#pragma unroll
    for (int c = 0; c < CELLS; ++c) {
      bool reaches;
      if constexpr (!kPacked) reaches = cell_max[c] >= T;
      else reaches = (c % 2 == 0 ? cell_max[c / 2] & 0xffffu : cell_max[c / 2] >> 16) >= (T >> 16);
      need |= (unsigned long long)(reaches ? 1u : 0u) << c;
    }
    int total = 0;
    while (__any_sync(0xffffffffu, need != 0ull)) {
      const bool active = need != 0ull;
      const int c = active ? __ffsll((long long)need) - 1 : 0;
      need &= need - 1ull;
      uint32_t raw[4] = {0u, 0u, 0u, 0u};
      if (active) row.load(c, raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t o = row.image(raw[e]);
        append_slots(sl, warp, lane, total, active && row.exists(c, e) && o >= T, o, (uint32_t)(row.pos0(c) + e));
      }
    }
    __syncwarp();
    return total;
  };
  int total = collect(kth_largest_of_lanes(lm, k, lane));
  if (total > kSlots) {                                    // a loose threshold (one lane with a low maximum): tighten it once
    const uint32_t T2 = kth_image_of_full_slots(sl.o[warp], sl.p[warp], k, lane);
    __syncwarp();
    total = collect(T2);
  }
  if (total <= kSlots)
    write_best_of_slots<DTYPE>(sl.o[warp], sl.p[warp], total, k, lane, descending, out_vals + r * out_stride, out_idx + r * out_stride);
  else
    topk_by_rounds<DTYPE, VEC>(row, k, descending, out_vals + r * out_stride, out_idx + r * out_stride);
}

// Longer rows: the row is streamed twice (the second pass from L2), with nothing kept per cell.
template <int DTYPE, bool VEC>
__global__ void __launch_bounds__(kThreads, 4)
topk_stream_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ out_vals, int32_t* __restrict__ out_idx,
                   int64_t rows, int length, int k, bool descending, int64_t out_stride) {
  __shared__ WarpSlots sl;
  const int lane = threadIdx.x & 31, warp = threadIdx.x / 32;
  const int64_t r = (int64_t)blockIdx.x * (kThreads / 32) + warp;
  if (r >= rows) return;
  const RowCells<DTYPE, VEC> row{src + r * length, length, lane, descending ? 0u : ~0u};
  uint32_t lm = 0;
  row.for_each_cell([&](int, const uint32_t (&o)[4]) { lm = max(max(lm, max(o[0], o[1])), max(o[2], o[3])); });
  auto collect = [&](uint32_t T) {
    int total = 0;
    row.for_each_cell([&](int cell, const uint32_t (&o)[4]) {
      const uint32_t top = max(max(o[0], o[1]), max(o[2], o[3]));
      if (__any_sync(0xffffffffu, top >= T)) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          append_slots(sl, warp, lane, total, row.exists(cell, e) && o[e] >= T, o[e], (uint32_t)(row.pos0(cell) + e));
      }
    });
    __syncwarp();
    return total;
  };
  int total = collect(kth_largest_of_lanes(lm, k, lane));
  if (total > kSlots) {                                    // a loose threshold: tighten it once
    const uint32_t T2 = kth_image_of_full_slots(sl.o[warp], sl.p[warp], k, lane);
    __syncwarp();
    total = collect(T2);
  }
  if (total <= kSlots)
    write_best_of_slots<DTYPE>(sl.o[warp], sl.p[warp], total, k, lane, descending, out_vals + r * out_stride, out_idx + r * out_stride);
  else
    topk_by_rounds<DTYPE, VEC>(row, k, descending, out_vals + r * out_stride, out_idx + r * out_stride);
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
  const int64_t warp_grid = (rows + kThreads / 32 - 1) / (kThreads / 32);
  const bool vec = aligned16(src) && length % 4 == 0;
  // one warp per row: rows short enough for it to be the better split, or enough rows to fill the machine
  if (k <= 32 && (length <= 1024 || (length <= 16384 && rows >= 4 * sm_count()))) {
    TL_REQUIRE(warp_grid < (1ll << 31), "topk: too many rows");
#define TL_TOPK_CELLS(CELLS)                                                                                                  \
    if (vec) topk_cells_kernel<DTYPE, CELLS, true><<<(unsigned)warp_grid, kThreads, 0, s>>>(in, ov, idx, rows, (int)length, k, desc, out_stride); \
    else topk_cells_kernel<DTYPE, CELLS, false><<<(unsigned)warp_grid, kThreads, 0, s>>>(in, ov, idx, rows, (int)length, k, desc, out_stride)
    if (length <= 256) { TL_TOPK_CELLS(2); }
    else if (length <= 512) { TL_TOPK_CELLS(4); }
    else if (length <= 1024) { TL_TOPK_CELLS(8); }
    else if (length <= 2048) { TL_TOPK_CELLS(16); }
    else if (length <= 4096) { TL_TOPK_CELLS(32); }
    else if (length <= 8192) { TL_TOPK_CELLS(64); }
    else if (vec) topk_stream_kernel<DTYPE, true><<<(unsigned)warp_grid, kThreads, 0, s>>>(in, ov, idx, rows, (int)length, k, desc, out_stride);
    else topk_stream_kernel<DTYPE, false><<<(unsigned)warp_grid, kThreads, 0, s>>>(in, ov, idx, rows, (int)length, k, desc, out_stride);
#undef TL_TOPK_CELLS
    TL_LAUNCH_CHECK("topk_cells_kernel");
  } else if (length <= 1024) {
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
    if (row_bytes / 16 >= 32) {
      int64_t need = (n_index + kThreads / 32 - 1) / (kThreads / 32);
      unsigned grid = (unsigned)(need < cap ? need : cap);
      gather_rows_kernel<UNROLL><<<grid, kThreads, 0, s>>>((const uint4*)param, index, (uint4*)out, n_index,
                                                          (int)(row_bytes / 16), (uint32_t)param_rows);
      TL_LAUNCH_CHECK("gather_rows_kernel");
      return TL_B200_OK;
    }
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
