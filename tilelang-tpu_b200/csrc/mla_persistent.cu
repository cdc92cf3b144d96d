// Persistent, work-balanced FP8 paged MLA decode for sm_100a.
//
// Same arithmetic as the per-sequence kernel of mla_decode.cu (two e4m3 terms for Q and P, raw cache
// bytes as both MMA operands), but the work is laid out differently:
//
//   * a preparation kernel cuts every query row into its two e4m3 terms ONCE per call (instead of
//     once per CTA), stores them in the layouts the decode kernel consumes (value term: rows of
//     128-byte slabs for TMA; residual term: 16-byte units interleaved over the 128 rows so that a
//     warp's loads are contiguous), takes the largest token scale of each sequence, and builds a
//     schedule: the flattened list of (sequence, 64-token tile) pairs is cut into one contiguous
//     range per CTA pair, each range costing the same number of tiles plus a fixed charge per
//     sequence touched;
//   * the decode kernel launches one CTA per SM (a pair shares a range, each CTA owning 256 output
//     columns) and walks its range.  A sequence that lies wholly inside a range is written to the
//     output directly; a sequence cut by a range boundary leaves normalised fp32 partials and their
//     log2-sum-exp, and a combine kernel merges them.  The TMA pipeline, the S-two-tiles-ahead MMA
//     order and the tensor-memory buffers keep running across sequence boundaries.
//
// Paged semantics: examples/deepseek_mla/example_mla_decode_paged.py:20-97,259-308 of the reference.
#include "mla_common.cuh"

namespace tl {

constexpr int kMlaSegOverhead = 5;        // fixed charge per (range, sequence) piece, in key tiles
constexpr int kMlaSchedMaxBatch = 4096;   // the schedule is built from a shared-memory copy of the lengths
constexpr int kMlaQvBytes = kMlaQBytes;                   // per sequence: 5 slabs x 128 rows x 128 bytes
constexpr int kMlaQloBytes = 32 * kMlaHeads * 16;         // per sequence: 32 units x 128 rows x 16 bytes
constexpr int kMlaSmemP = kMlaOffBar + 1024 + 6144 + 16 * 1024 + 1024;   // barriers, exchange, epilogue staging, alignment

struct MlaPrepParams {
  const void* q;               // [batch, heads, 576]
  const float* kv_scale;
  const int* block_table;
  const int* seqlens;
  uint8_t* qv;                 // [batch][5][128][128]
  uint8_t* qlo;                // [batch][32][128][16]
  float* q_scale;              // [batch][128]
  float* seq_max_ts;           // [batch]
  int4* sched;                 // [workers] begin sequence, begin tile, end sequence, end tile (exclusive)
  int2* seq_info;              // [batch] partial slot of the first piece, number of pieces
  int batch, heads, page_size, max_pages, workers;
  int len_cap, num_pages;      // bounds for the lengths and page ids read on the device
};

// Block 0: the schedule (one thread walks the sequences, so it starts first).  Blocks [1, batch]:
// largest token scale of a sequence.  The other 4 * batch blocks: 32 query rows each.
template <typename TQ>
__global__ void __launch_bounds__(256, 2)
mla_prepare_kernel(const MlaPrepParams p) {
  __shared__ __align__(16) uint8_t stage[32 * 528];       // residual units of 32 rows, pitch 33 units
  __shared__ float red[8];
  dependency_release();                          // the decode kernel may set up its barriers and tensor memory meanwhile
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  if (blockIdx.x == 0) {
    // ---------------------------------------------------------------- schedule
    // Cost line: sequence b occupies [C[b], C[b+1]) with C[b+1] - C[b] = overhead + tiles; the first
    // `overhead` units stand for its fixed charge, the rest for its key tiles.  Range w begins at the
    // (sequence, tile) under cost w * P, P = ceil(total / ranges), and ends where range w + 1 begins.
    int* C = reinterpret_cast<int*>(stage);                // [batch + 1] exclusive prefix sums
    __shared__ int warp_tot[8];
    const int per = (p.batch + 255) / 256;                 // consecutive sequences per thread (<= 16)
    const int b0 = threadIdx.x * per;
    int local = 0;
    for (int i = 0; i < per; ++i)
      if (b0 + i < p.batch) local += (mla_len(p.seqlens, b0 + i, p.len_cap) + kMlaBN - 1) / kMlaBN + kMlaSegOverhead;
    int incl = local;                                      // inclusive scan over the block
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = incl - local;
    for (int i = 0; i < warp; ++i) before += warp_tot[i];
    for (int i = 0; i < per; ++i)
      if (b0 + i < p.batch) {
        C[b0 + i] = before;
        before += (mla_len(p.seqlens, b0 + i, p.len_cap) + kMlaBN - 1) / kMlaBN + kMlaSegOverhead;
      }
    if (threadIdx.x == 255) C[p.batch] = before;           // the last thread's running sum is the total
    __syncthreads();
    const int total = C[p.batch];
    const int P = max((total + p.workers - 1) / p.workers, 1);
    auto position = [&](int x) {                           // (sequence, tile) under cost x
      if (x >= total) return make_int2(p.batch, 0);
      int lo = 0, hi = p.batch;                            // largest b with C[b] <= x
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (C[mid] <= x) lo = mid; else hi = mid;
      }
      return make_int2(lo, max(0, x - C[lo] - kMlaSegOverhead));
    };
    for (int w = threadIdx.x; w < p.workers; w += 256) {
      const int2 bg = position(w * P);
      const int2 en = (w + 1 == p.workers) ? make_int2(p.batch, 0) : position((w + 1) * P);
      p.sched[w] = make_int4(bg.x, bg.y, en.x, en.y);
    }
    for (int b = threadIdx.x; b < p.batch; b += 256) {
      const int tiles = C[b + 1] - C[b] - kMlaSegOverhead;
      const int w0 = min((C[b] + kMlaSegOverhead) / P, p.workers - 1);
      const int w1 = tiles > 0 ? min((C[b] + kMlaSegOverhead + tiles - 1) / P, p.workers - 1) : w0;
      // the first piece is its range's first piece exactly when the range begins inside this sequence
      p.seq_info[b] = make_int2(2 * w0 + (w0 * P >= C[b] ? 0 : 1), w1 - w0 + 1);
    }
    return;
  }
  if (blockIdx.x <= p.batch) {
    // ---------------------------------------------------------------- largest token scale of a sequence
    // (P is multiplied by 32 * scale[t] / this before it is cut to e4m3)
    const int b = blockIdx.x - 1;
    const int seqlen = mla_len(p.seqlens, b, p.len_cap);
    const int* table = p.block_table + (int64_t)b * p.max_pages;
    float m = 0.f;
    for (int t0 = 0; t0 < seqlen; t0 += 4 * 1024) {
      float4 v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {                     // all loads of the pass in flight; a page holds a multiple of 64 tokens
        const int t = t0 + i * 1024 + threadIdx.x * 4;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < seqlen) {
          const int page = __ldg(table + t / p.page_size);
          if (mla_page_ok(page, p.num_pages))       // the tokens of a page id outside the cache are masked
            v[i] = __ldg(reinterpret_cast<const float4*>(p.kv_scale + (int64_t)page * p.page_size + t % p.page_size));
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = t0 + i * 1024 + threadIdx.x * 4;
        if (t < seqlen) m = fmaxf(m, v[i].x);           // slots past the end hold arbitrary bytes
        if (t + 1 < seqlen) m = fmaxf(m, v[i].y);
        if (t + 2 < seqlen) m = fmaxf(m, v[i].z);
        if (t + 3 < seqlen) m = fmaxf(m, v[i].w);
      }
    }
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
      p.seq_max_ts[b] = m;
    }
    return;
  }
  // ------------------------------------------------------------------ query rows
  const int qb = blockIdx.x - p.batch - 1;
  const int b = qb / 4, r0 = (qb % 4) * 32;
  // Four rows per warp, every load in flight together.  A row is 36 units of 16 columns: lane l takes
  // unit l of each of the four rows, and the 4 x 4 units left over (32..35) go to lanes 0..15, lane l
  // taking unit 32 + l % 4 of row l / 4.
  const int rw = r0 + warp * 4;                                    // first row of this warp
  const TQ* qbase = reinterpret_cast<const TQ*>(p.q) + (int64_t)b * p.heads * kMlaD;
  Vec16<TQ> mainv[4][2], tailv[2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    mainv[i][0].raw = mainv[i][1].raw = make_uint4(0, 0, 0, 0);
    if (rw + i < p.heads) {
      const uint4* qrow = reinterpret_cast<const uint4*>(qbase + (int64_t)(rw + i) * kMlaD);
      mainv[i][0].raw = __ldg(qrow + 2 * lane);
      mainv[i][1].raw = __ldg(qrow + 2 * lane + 1);
    }
  }
  const int ti = (lane >> 2) & 3, tc = lane & 3;                   // tail: row within the warp, unit - 32
  tailv[0].raw = tailv[1].raw = make_uint4(0, 0, 0, 0);
  if (lane < 16 && rw + ti < p.heads) {
    const uint4* qrow = reinterpret_cast<const uint4*>(qbase + (int64_t)(rw + ti) * kMlaD);
    tailv[0].raw = __ldg(qrow + 64 + 2 * tc);
    tailv[1].raw = __ldg(qrow + 65 + 2 * tc);
  }
  float tail_max = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) tail_max = fmaxf(tail_max, fmaxf(fabsf(to_f32(tailv[0].e[e])), fabsf(to_f32(tailv[1].e[e]))));
  float inv[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float amax = (lane < 16 && ti == i) ? tail_max : 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fmaxf(fabsf(to_f32(mainv[i][0].e[e])), fabsf(to_f32(mainv[i][1].e[e]))));
    amax = fmaxf(warp_max(amax), 1e-10f);
    inv[i] = 448.0f / amax;
    if (lane == 0) p.q_scale[(int64_t)b * kMlaHeads + rw + i] = amax / 448.0f;
  }
  // 16 columns -> 16 bytes of the value term and 16 bytes of the residual term
  auto cut16 = [](const Vec16<TQ>& lo8, const Vec16<TQ>& hi8, float scale, uint4& val, uint4& res) {
    uint32_t v[4], r[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      float f[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) f[e] = to_f32(w < 2 ? lo8.e[(w % 2) * 4 + e] : hi8.e[(w % 2) * 4 + e]) * scale;
      v[w] = pack_e4m3x4(f[0], f[1], f[2], f[3]);
      const float2 a = e4m3x2_to_float2(v[w]), c = e4m3x2_to_float2(v[w] >> 16);
      r[w] = pack_e4m3x4(f[0] - a.x, f[1] - a.y, f[2] - c.x, f[3] - c.y);
    }
    val = make_uint4(v[0], v[1], v[2], v[3]);
    res = make_uint4(r[0], r[1], r[2], r[3]);
  };
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 val, res;
    cut16(mainv[i][0], mainv[i][1], inv[i], val, res);
    const int slab = lane / 8, c = lane % 8;                        // unit = lane
    *reinterpret_cast<uint4*>(p.qv + (((int64_t)b * kMlaSlabs + slab) * kMlaHeads + rw + i) * 128 + c * 16) = val;
    *reinterpret_cast<uint4*>(stage + (warp * 4 + i) * 528 + lane * 16) = res;
  }
  if (lane < 16) {
    const float scale = ti == 0 ? inv[0] : ti == 1 ? inv[1] : ti == 2 ? inv[2] : inv[3];
    uint4 val, res;
    cut16(tailv[0], tailv[1], scale, val, res);
    uint8_t* vrow = p.qv + (((int64_t)b * kMlaSlabs + 4) * kMlaHeads + rw + ti) * 128;
    *reinterpret_cast<uint4*>(vrow + tc * 16) = val;                // columns 512..575: value | residual in one row
    *reinterpret_cast<uint4*>(vrow + 64 + tc * 16) = res;
  }
  __syncthreads();
  // residual units, interleaved over the rows: [unit][row][16 bytes]
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int unit = pass * 8 + warp;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + lane * 528 + unit * 16);
    *reinterpret_cast<uint4*>(p.qlo + (((int64_t)b * 32 + unit) * kMlaHeads + r0 + lane) * 16) = v;
  }
}

struct MlaSchedParams {
  const uint8_t* qlo;          // [batch][32][128][16]
  const float* q_scale;        // [batch][128]
  const float* seq_max_ts;     // [batch]
  const float* kv_scale;       // [num_pages * page_size]
  const int* block_table;      // [batch, max_pages]
  const int* seqlens;          // [batch]
  const int4* sched;           // [workers]
  void* out;                   // [batch, heads, 512]
  float* part_o;               // [2 * workers][128][512] normalised partial outputs
  float* part_lse;             // [2 * workers][128] their log2-sum-exp
  int batch, heads, page_size, max_pages;
  int len_cap, num_pages;
  float scale_log2;
  int* status;
};

// One piece of a CTA pair's range: tiles [t0, t0 + n) of sequence `seq`.
struct MlaPiece {
  int seq, t0, n;
  bool whole;                  // the piece is the entire sequence: write the output directly
  bool valid;
};

// The pieces of a range are its sequences in order; the first starts at the range's begin tile, the
// last (if the end tile is not zero) stops at the end tile.  An empty sequence is a piece of zero tiles.
__device__ __forceinline__ MlaPiece mla_piece(const int4 sc, int seq, const int* __restrict__ seqlens, int batch, int len_cap) {
  MlaPiece pc{seq, 0, 0, false, false};
  if (seq >= batch || seq > sc.z || (seq == sc.z && sc.w == 0)) return pc;
  const int n_seq = (mla_len(seqlens, seq, len_cap) + kMlaBN - 1) / kMlaBN;
  pc.t0 = (seq == sc.x) ? sc.y : 0;
  const int t1 = (seq == sc.z) ? sc.w : n_seq;
  pc.n = max(t1 - pc.t0, 0);
  pc.whole = (pc.t0 == 0 && t1 == n_seq);
  pc.valid = true;
  return pc;
}

template <typename TQ>
__global__ void __launch_bounds__(kMlaThreads, 1)
mla_decode_persistent_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_q,
                             const MlaSchedParams p) {
  constexpr int kWG = kMlaSoftmaxWarps / 4;                   // softmax warpgroups
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t sm_q = base;
  const uint32_t sm_kv = base + kMlaOffKV;                   // stage s at s * (tile + 1 KB)
  const uint32_t bar0 = base + kMlaOffBar;
  const uint32_t bar_kvfull = bar0;                          // [stages]
  const uint32_t bar_kvempty = bar0 + 8 * kMlaStages;
  const uint32_t bar_sfull = bar_kvempty + 8 * kMlaStages;   // [2 S buffers]
  const uint32_t bar_pfull = bar_sfull + 16;                 // [2]
  const uint32_t bar_pvdone = bar_pfull + 16;                // [2]
  const uint32_t bar_xch = bar_pvdone + 16;                  // [2] row maxima of the two softmax warpgroups
  // once per piece (phase = piece count & 1)
  const uint32_t bar_qfull = bar_xch + 16;                   // value term of Q has landed in shared memory
  const uint32_t bar_qfree = bar_qfull + 8;                  // every S MMA of the piece has completed
  const uint32_t bar_qlo = bar_qfree + 8;                    // residual term of Q is in tensor memory
  const uint32_t bar_ofree = bar_qlo + 8;                    // O has been read out of tensor memory
  const uint32_t bar_post = bar_ofree + 8;                   // row sums exchanged
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + kMlaOffBar + 8 * (2 * kMlaStages + 13));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // exchange area of the softmax warpgroups: row maxima [2 tile parities][kWG][128], then row sums [kWG][128]
  float* exch = reinterpret_cast<float*>(base_ptr + kMlaOffBar + 1024);
  const uint32_t sm_stage = base + kMlaOffBar + 1024 + 6144;  // 1 KB per softmax warp for the epilogue

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int worker = blockIdx.x >> 1, half = blockIdx.x & 1;
  dependency_release();                          // lets the merge kernel's blocks take their places early

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kMlaStages; ++s) {
      mbar_init(bar_kvfull + 8 * s, 1);
      mbar_init(bar_kvempty + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_sfull + 8 * i, 1);
      mbar_init(bar_pfull + 8 * i, 4 * kWG);
      mbar_init(bar_pvdone + 8 * i, 1);
      mbar_init(bar_xch + 8 * i, 4 * kWG);
    }
    mbar_init(bar_qfull, 1);
    mbar_init(bar_qfree, 1);
    mbar_init(bar_qlo, 4 * kWG);
    mbar_init(bar_ofree, 4 * kWG);
    mbar_init(bar_post, 4 * kWG);
    mbar_fence_init();
    prefetch_tensormap(&tm_kv);
    prefetch_tensormap(&tm_q);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_slot), kMlaTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  auto stage_addr = [&](int s) { return sm_kv + s * (kMlaTile + 1024); };
  dependency_wait();                             // everything below reads what the preparation kernel wrote
  const int4 sc = p.sched[worker];

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      bool ok = true;
      int g = 0, a = 0;                            // tiles and non-empty pieces so far
      MlaPiece nxt = mla_piece(sc, sc.x, p.seqlens, p.batch, p.len_cap);
      while (nxt.valid && ok) {
        const MlaPiece pc = nxt;
        const int seq = pc.seq;
        nxt = mla_piece(sc, seq + 1, p.seqlens, p.batch, p.len_cap);        // its length is on the way while this piece runs
        if (pc.n == 0) continue;
        if (a > 0 && !(ok = mbar_wait(bar_qfree, (a - 1) & 1, abort_flag))) break;
        mbar_expect_tx(bar_qfull, kMlaQBytes);
#pragma unroll
        for (int s = 0; s < kMlaSlabs; ++s)
          tma_load_2d(sm_q + s * (kMlaHeads * 128), &tm_q, bar_qfull, 0, (seq * kMlaSlabs + s) * kMlaHeads);
        const int* table = p.block_table + (int64_t)seq * p.max_pages;
        for (int j = 0; j < pc.n; ++j, ++g) {
          const int st = g % kMlaStages;
          if (!(ok = mbar_wait(bar_kvempty + 8 * st, ((g / kMlaStages) & 1) ^ 1, abort_flag))) break;
          const int tok = (pc.t0 + j) * kMlaBN;
          const int page = __ldg(table + tok / p.page_size);
          // row of the flattened cache; a page id outside the cache reads row 0 and the softmax masks the tile
          const int row = mla_page_ok(page, p.num_pages) ? page * p.page_size + tok % p.page_size : 0;
          const uint32_t full = bar_kvfull + 8 * st;
          mbar_expect_tx(full, kMlaStageBytes);
#pragma unroll
          for (int s = 0; s < kMlaSlabs; ++s)         // columns 576..639 of the last slab are out of range: zero fill
            tma_load_2d(stage_addr(st) + s * (kMlaBN * 128), &tm_kv, full, s * 128, row);
          bulk_load(stage_addr(st) + kMlaTile, p.kv_scale + row, kMlaBN * 4, full);
        }
        ++a;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // Inside a piece S runs two tiles ahead of P V:  S(0) S(1) | PV(0) S(2) | PV(1) S(3) | ...
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc(kFmtE4M3, kFmtE4M3, false, false, kMlaHeads, kMlaBN);
      const uint32_t idesc_o = make_idesc(kFmtE4M3, kFmtE4M3, false, true, kMlaHeads, 256);
      // descriptors are built once; every MMA's operands are a constant byte offset further on
      const uint64_t q_desc = smem_desc_sw128(sm_q, 16, 1024), k_desc = smem_desc_sw128(sm_kv, 16, 1024);
      const uint64_t v_desc = smem_desc_sw128(sm_kv, kMlaBN * 128, 1024);
      bool ok = true;
      int g0 = 0, a = 0;                           // first tile counter of the piece, non-empty pieces so far
      MlaPiece nxt = mla_piece(sc, sc.x, p.seqlens, p.batch, p.len_cap);
      while (nxt.valid && ok) {
        const MlaPiece pc = nxt;
        nxt = mla_piece(sc, pc.seq + 1, p.seqlens, p.batch, p.len_cap);
        if (pc.n == 0) continue;
        auto issue_s = [&](int j) {
          const int g = g0 + j, st = g % kMlaStages;
          if (!(ok = mbar_wait(bar_kvfull + 8 * st, (g / kMlaStages) & 1, abort_flag))) return;
          tc_fence_after_sync();
          const uint64_t kd = desc_at(k_desc, st * (kMlaTile + 1024));      // this stage, K-major view
          const uint32_t d = tmem_base + kMlaColS + (g & 1) * kMlaBN;
          // value term of Q (shared memory) x K, all 576 columns
#pragma unroll
          for (int kk = 0; kk < kMlaD / 32; ++kk) {
            mma_f8_ss(d, desc_at(q_desc, (kk / 4) * (kMlaHeads * 128) + (kk % 4) * 32),
                      desc_at(kd, (kk / 4) * (kMlaBN * 128) + (kk % 4) * 32), idesc_s, kk ? 1u : 0u);
          }
          // residual term of Q x K: columns 0..511 from tensor memory (8 columns per 32-byte step) ...
#pragma unroll
          for (int kk = 0; kk < 16; ++kk) {
            mma_f8_ts(d, tmem_base + kMlaColQlo + kk * 8, desc_at(kd, (kk / 4) * (kMlaBN * 128) + (kk % 4) * 32), idesc_s, 1u);
          }
          // ... columns 512..575 from the upper half of Q slab 4
#pragma unroll
          for (int kk = 0; kk < 2; ++kk) {
            mma_f8_ss(d, desc_at(q_desc, 4 * (kMlaHeads * 128) + 64 + kk * 32), desc_at(kd, 4 * (kMlaBN * 128) + kk * 32),
                      idesc_s, 1u);
          }
          mma_commit(bar_sfull + 8 * (g & 1));
          if (j == pc.n - 1) mma_commit(bar_qfree);          // Q may be replaced by the next piece's
        };
        if (!(ok = mbar_wait(bar_qfull, a & 1, abort_flag))) break;
        if (!(ok = mbar_wait(bar_qlo, a & 1, abort_flag))) break;
        issue_s(0);
        if (ok && pc.n > 1) issue_s(1);
        for (int j = 0; j < pc.n && ok; ++j) {
          const int g = g0 + j;
          if (!(ok = mbar_wait(bar_pfull + 8 * (g & 1), (g >> 1) & 1, abort_flag))) break;
          // the first P V of a piece overwrites O: the previous piece's epilogue must have read it
          if (j == 0 && a > 0 && !(ok = mbar_wait(bar_ofree, (a - 1) & 1, abort_flag))) break;
          tc_fence_after_sync();
          const uint64_t vd = desc_at(v_desc, (g % kMlaStages) * (kMlaTile + 1024) + (2 * half) * (kMlaBN * 128));
          const uint32_t pa = tmem_base + kMlaColS + (g & 1) * kMlaBN;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            // A: P row = [value(64 tokens) | residual(64 tokens)] in 32 columns, 8 columns per step.
            // B: this half's 256 V columns = two 128-column slabs (8 KB apart), 32 tokens = 4 KB per
            // step; the residual steps reuse the same tokens.
            mma_f8_ts(tmem_base + kMlaColO, pa + kk * 8, desc_at(vd, (kk & 1) * 4096), idesc_o, (j | kk) ? 1u : 0u);
          }
          mma_commit(bar_pvdone + 8 * (g & 1));
          mma_commit(bar_kvempty + 8 * (g % kMlaStages));
          if (j + 2 < pc.n) issue_s(j + 2);
        }
        g0 += pc.n;
        ++a;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax, epilogue
    // kWG warpgroups share every tile: warpgroup wg owns TOK = 64 / kWG of its tokens (columns of
    // S) and OC = 256 / kWG of the output columns; thread (wg, h) works on row h.
    constexpr int TOK = kMlaBN / kWG, NV = TOK / 4, OC = 256 / kWG;
    const int wg = (warp - 4) / 4;
    const int quarter = warp % 4;
    const int h = quarter * 32 + lane;            // head = TMEM lane
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t t_o = tmem_base + kMlaColO + wg * OC + lane_off;
    constexpr float kPScale = 32.0f;
    bool ok = true;
    // The residual term of Q (columns 0..511 of row h) of the first non-empty piece at or after `pc`
    // goes to tensor memory: each warpgroup moves its share of the columns, 16-byte loads that are
    // contiguous across a warp, all in flight together, then stores of 32 words.
    auto stage_qlo = [&](MlaPiece pc) {
      while (pc.valid && pc.n == 0) pc = mla_piece(sc, pc.seq + 1, p.seqlens, p.batch, p.len_cap);
      if (!pc.valid) return;
      constexpr int UN = 32 / kWG;                // 16-byte units per thread
      const uint4* src = reinterpret_cast<const uint4*>(p.qlo) + ((int64_t)pc.seq * 32 + wg * UN) * kMlaHeads + h;
      uint4 v[UN];
#pragma unroll
      for (int i = 0; i < UN; ++i) v[i] = __ldg(src + i * kMlaHeads);
#pragma unroll
      for (int c = 0; c < UN / 8; ++c) {
        uint32_t words[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          words[4 * i] = v[8 * c + i].x; words[4 * i + 1] = v[8 * c + i].y;
          words[4 * i + 2] = v[8 * c + i].z; words[4 * i + 3] = v[8 * c + i].w;
        }
        tmem_st_32x32(tmem_base + kMlaColQlo + (wg * (UN / 8) + c) * 32 + lane_off, words);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_qlo);
    };
    MlaPiece nxt = mla_piece(sc, sc.x, p.seqlens, p.batch, p.len_cap);
    stage_qlo(nxt);
    int g0 = 0, a = 0;
    while (nxt.valid && ok) {
      const MlaPiece pc = nxt;
      const int seq = pc.seq;
      nxt = mla_piece(sc, seq + 1, p.seqlens, p.batch, p.len_cap);          // its length is on the way while this piece runs
      if (pc.n == 0) {
        TQ* out = reinterpret_cast<TQ*>(p.out) + ((int64_t)seq * p.heads + h) * kMlaDV + half * 256 + wg * OC;
        if (pc.whole && h < p.heads)              // an empty sequence: zeros
          for (int c = 0; c < OC / 8; ++c) reinterpret_cast<uint4*>(out)[c] = make_uint4(0, 0, 0, 0);
        continue;
      }
      const float q_scale = __ldg(p.q_scale + (int64_t)seq * kMlaHeads + h);
      const float max_ts = __ldg(p.seq_max_ts + seq);
      const float ts_norm = max_ts > 0.f ? kPScale / max_ts : kPScale;
      const float s_scale = q_scale * p.scale_log2;
      const int seqlen = mla_len(p.seqlens, seq, p.len_cap);
      const int* table = p.block_table + (int64_t)seq * p.max_pages;
      // online softmax: a row is shared by one thread of each warpgroup
      float m_used = -INFINITY, row_sum = 0.f;
      for (int j = 0; j < pc.n && ok; ++j) {
        const int g = g0 + j;
        const uint32_t t_s = tmem_base + kMlaColS + (g & 1) * kMlaBN + lane_off;
        const int tile_page = __ldg(table + (pc.t0 + j) * kMlaBN / p.page_size);     // on its way during the wait
        ok = mbar_wait(bar_sfull + 8 * (g & 1), (g >> 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t sv[TOK];
        static_assert(TOK == 32, "two softmax warpgroups");
        tmem_ld_32x32(t_s + wg * TOK, sv);
        tmem_ld_wait();
        const float4* ts4 = reinterpret_cast<const float4*>(base_ptr + (stage_addr(g % kMlaStages) - base) + kMlaTile) + wg * NV;
        // tokens of this share that exist; none if the tile's page id is outside the cache
        const int valid = mla_page_ok(tile_page, p.num_pages) ? seqlen - (pc.t0 + j) * kMlaBN - wg * TOK : 0;
        // sp = acc * token_scale (packed pairs); the per-head factor s_scale > 0 is applied inside the
        // exponent, so the row maximum can be taken on sp
        float2 sp[TOK / 2];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const float4 t = ts4[i];
          sp[2 * i] = mul2(make_float2(__uint_as_float(sv[4 * i]), __uint_as_float(sv[4 * i + 1])), make_float2(t.x, t.y));
          sp[2 * i + 1] = mul2(make_float2(__uint_as_float(sv[4 * i + 2]), __uint_as_float(sv[4 * i + 3])), make_float2(t.z, t.w));
        }
        if (valid < TOK) {                                     // last tile of the sequence only
#pragma unroll
          for (int c = 0; c < TOK; ++c)
            if (c >= valid) reinterpret_cast<float*>(sp)[c] = -INFINITY;
        }
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < TOK / 2; i += 2) {
          m4[0] = fmaxf(m4[0], sp[i].x); m4[1] = fmaxf(m4[1], sp[i].y);
          m4[2] = fmaxf(m4[2], sp[i + 1].x); m4[3] = fmaxf(m4[3], sp[i + 1].y);
        }
        float* ex = exch + (g & 1) * (kWG * 128);
        ex[wg * 128 + h] = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_xch + 8 * (g & 1));
        ok = mbar_wait(bar_xch + 8 * (g & 1), (g >> 1) & 1, abort_flag);   // also: all of S is in registers now
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        float m_tile = ex[h];
#pragma unroll
        for (int i = 1; i < kWG; ++i) m_tile = fmaxf(m_tile, ex[i * 128 + h]);
        m_tile *= s_scale;
        const float m_new = fmaxf(m_used, m_tile);
        // e4m3 has little dynamic range (largest 448, smallest normal 2^-6), so P is kept in (0, 8] -
        // the running maximum may lag by at most three binades - and scaled by kPScale = 32 before it
        // is cut to its two e4m3 terms
        const bool grow = (j == 0) || (m_new - m_used > 3.0f);
        if (j > 0 && __any_sync(0xffffffffu, grow && m_used != -INFINITY)) {
          ok = mbar_wait(bar_pvdone + 8 * ((g - 1) & 1), ((g - 1) >> 1) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          const float alpha = (grow && m_used != -INFINITY) ? ex2_approx(m_used - m_new) : 1.0f;
          row_sum *= alpha;
#pragma unroll 1
          for (int c = 0; c < OC / 32; ++c) {
            uint32_t ov[32];
            tmem_ld_32x32(t_o + c * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
            tmem_st_32x32(t_o + c * 32, ov);
          }
          tmem_st_wait();
        }
        if (grow) m_used = m_new;
        const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
        const float2 k2 = make_float2(s_scale, s_scale), nm2 = make_float2(-m_safe, -m_safe);
        const float2 n2 = make_float2(ts_norm, ts_norm);
        float2 sum2a = make_float2(0.f, 0.f), sum2b = make_float2(0.f, 0.f);
        uint32_t hi[NV], lo[NV];
        // value + residual e4m3 terms of a pair.  Float conversions share the slow XU pipe with
        // ex2, so only the two float->e4m3 cuts use it; the value term is decoded back with integer
        // and FMA-pipe work: (byte << 20) as a float is the e4m3 value times 2^-120, exactly.
        auto split = [](float2 w, uint32_t& v8, uint32_t& r8) {
          v8 = __nv_cvt_float2_to_fp8x2(w, __NV_SATFINITE, __NV_E4M3);
          const float2 dec = mul2(make_float2(__uint_as_float((v8 & 0xffu) << 20), __uint_as_float((v8 & 0xff00u) << 12)),
                                  make_float2(0x1p120f, 0x1p120f));
          r8 = __nv_cvt_float2_to_fp8x2(make_float2(w.x - dec.x, w.y - dec.y), __NV_SATFINITE, __NV_E4M3);
        };
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const float4 t = ts4[i];
          const float2 a0 = fma2(sp[2 * i], k2, nm2), a1 = fma2(sp[2 * i + 1], k2, nm2);
          const float2 p0 = make_float2(ex2_approx(a0.x), ex2_approx(a0.y));
          const float2 p1 = make_float2(ex2_approx(a1.x), ex2_approx(a1.y));
          sum2a = add2(sum2a, p0);
          sum2b = add2(sum2b, p1);
          float2 w0 = mul2(p0, mul2(make_float2(t.x, t.y), n2));
          float2 w1 = mul2(p1, mul2(make_float2(t.z, t.w), n2));
          if (valid < TOK) {       // token scales of slots past the end are arbitrary bytes
            if (4 * i >= valid) w0.x = 0.f;
            if (4 * i + 1 >= valid) w0.y = 0.f;
            if (4 * i + 2 >= valid) w1.x = 0.f;
            if (4 * i + 3 >= valid) w1.y = 0.f;
          }
          uint32_t v0, r0, v1, r1;
          split(w0, v0, r0);
          split(w1, v1, r1);
          hi[i] = v0 | (v1 << 16);
          lo[i] = r0 | (r1 << 16);
        }
        row_sum += (sum2a.x + sum2a.y) + (sum2b.x + sum2b.y);
        // P row: value term of the 64 tokens in columns 0..15, residual term in columns 16..31
        tmem_st_32x8(t_s + wg * NV, hi);
        tmem_st_32x8(t_s + 16 + wg * NV, lo);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_pfull + 8 * (g & 1));
      }
      if (!ok) break;
      // every S MMA of this piece has completed: the next piece's residual term may replace this one's
      stage_qlo(nxt);
      // epilogue: each warpgroup writes OC of this CTA's 256 output columns
      const int gl = g0 + pc.n - 1;
      ok = mbar_wait(bar_pvdone + 8 * (gl & 1), (gl >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      float* ex = exch + 2 * kWG * 128;           // read by everyone before the next piece's first exchange
      ex[wg * 128 + h] = row_sum;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_post);
      ok = mbar_wait(bar_post, a & 1, abort_flag) && ok;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      float total = ex[h];
#pragma unroll
      for (int i = 1; i < kWG; ++i) total += ex[i * 128 + h];
      tc_fence_after_sync();
      const float inv = total > 0.f ? max_ts / (kPScale * total) : 0.f;     // undo the P normalisation
      const int slot = 2 * worker + (seq == sc.x ? 0 : 1);
      if (!pc.whole && half == 0 && wg == 0)
        p.part_lse[(int64_t)slot * kMlaHeads + h] = total > 0.f ? m_used + log2f(total) : -INFINITY;
      // A lane owns a row, so storing straight from registers would touch 32 different 128-byte lines
      // per instruction.  Each warp turns 16-row x 64-byte blocks around in shared memory instead
      // (16-byte units, XOR-swizzled by the row) and stores 8 rows x 64 contiguous bytes at a time.
      const uint32_t stg = sm_stage + (warp - 4) * 1024;
      const int sr = lane >> 2, sk = lane & 3;                      // read side: row within a group of 8, unit
      auto turn_and_store = [&](const uint32_t (&w)[16], char* row0, int64_t row_pitch, int rows_live) {
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {                            // rows 0-15, then rows 16-31 of the warp
          if ((lane >> 4) == hr) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              st_shared_v4(stg + (lane & 15) * 64 + ((k ^ ((lane >> 1) & 3)) << 4), w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int r = i * 8 + sr;
            const uint4 v = ld_shared_v4(stg + r * 64 + ((sk ^ ((r >> 1) & 3)) << 4));
            if (hr * 16 + r < rows_live) *reinterpret_cast<uint4*>(row0 + (hr * 16 + r) * row_pitch + sk * 16) = v;
          }
          __syncwarp();
        }
      };
      const int rows_live = p.heads - quarter * 32;                 // rows of this warp that exist
      char* out_w = reinterpret_cast<char*>(reinterpret_cast<TQ*>(p.out) + ((int64_t)seq * p.heads + quarter * 32) * kMlaDV +
                                            half * 256 + wg * OC);
      char* po_w = reinterpret_cast<char*>(p.part_o + ((int64_t)slot * kMlaHeads + quarter * 32) * kMlaDV + half * 256 + wg * OC);
#pragma unroll 1
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t ov[32];
        tmem_ld_32x32(t_o + c * 32, ov);
        tmem_ld_wait();
        if (pc.whole) {
          uint32_t w[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            Vec16<TQ> two;      // only the first two elements are used
            two.e[0] = from_f32<TQ>(__uint_as_float(ov[2 * e]) * inv);
            two.e[1] = from_f32<TQ>(__uint_as_float(ov[2 * e + 1]) * inv);
            w[e] = two.raw.x;
          }
          turn_and_store(w, out_w + c * 32 * sizeof(TQ), kMlaDV * sizeof(TQ), rows_live);
        } else {
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {
            uint32_t w[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) w[e] = __float_as_uint(__uint_as_float(ov[hc * 16 + e]) * inv);
            turn_and_store(w, po_w + (c * 32 + hc * 16) * 4, kMlaDV * 4, 32);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ofree);
      g0 += pc.n;
      ++a;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(20000);      // let copies in flight land before the CTA leaves
    if (threadIdx.x == 0 && p.status) *p.status = *abort_flag;
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kMlaTmemCols);
  }
}


// Merges the pieces of every sequence that a range boundary cut:
//   out = sum_c 2^(lse_c - M) O_c / sum_c 2^(lse_c - M).
// A cut sequence ends as the first piece of exactly one range, and that range's blocks merge it:
// one warp per head (blockIdx.y picks 8 of the heads), a lane owns 16 of the 512 columns.  Piece 0
// sits in the slot the schedule recorded; piece i > 0 is the first piece of the i-th range after it.
template <typename TQ>
__global__ void __launch_bounds__(256)
mla_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, const int4* __restrict__ sched,
                 const int2* __restrict__ seq_info, TQ* __restrict__ out, int heads) {
  dependency_wait();                             // partials and schedule come from the kernels before
  const int4 sc = sched[blockIdx.x];
  if (sc.y == 0 || sc.z == sc.x) return;        // the first piece starts a sequence, or does not finish it
  const int b = sc.x;
  const int2 info = seq_info[b];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int h = blockIdx.y * 8 + warp;
  if (info.y <= 1 || h >= heads) return;
  auto slot_of = [&](int c) { return c == 0 ? info.x : 2 * ((info.x >> 1) + c); };
  float m = -INFINITY;
  for (int c = lane; c < info.y; c += 32) m = fmaxf(m, part_lse[(int64_t)slot_of(c) * kMlaHeads + h]);
  m = warp_max(m);
  float denom = 0.f;
  float4 acc[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
  for (int c = 0; c < info.y; ++c) {
    const int slot = slot_of(c);
    const float lse = part_lse[(int64_t)slot * kMlaHeads + h];
    const float w = lse == -INFINITY ? 0.f : exp2f(lse - m);
    denom += w;
    const float4* src = reinterpret_cast<const float4*>(part_o + ((int64_t)slot * kMlaHeads + h) * kMlaDV) + lane;
#pragma unroll
    for (int k = 0; k < 4; ++k) {               // 512-byte rows of the warp: columns 128 k + 4 lane
      const float4 v = src[k * 32];
      acc[k].x = fmaf(w, v.x, acc[k].x); acc[k].y = fmaf(w, v.y, acc[k].y);
      acc[k].z = fmaf(w, v.z, acc[k].z); acc[k].w = fmaf(w, v.w, acc[k].w);
    }
  }
  const float inv = denom > 0.f ? 1.0f / denom : 0.f;
  TQ* o = out + ((int64_t)b * heads + h) * kMlaDV + lane * 4;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    Vec16<TQ> v;                                // the first four elements are used: 8 bytes
    v.e[0] = from_f32<TQ>(acc[k].x * inv); v.e[1] = from_f32<TQ>(acc[k].y * inv);
    v.e[2] = from_f32<TQ>(acc[k].z * inv); v.e[3] = from_f32<TQ>(acc[k].w * inv);
    *reinterpret_cast<uint2*>(o + k * 128) = make_uint2(v.raw.x, v.raw.y);
  }
}

// ---- host ---------------------------------------------------------------------------------------
namespace {
inline int64_t up256(int64_t v) { return (v + 255) / 256 * 256; }
struct MlaWorkspace {
  int64_t sched, seq_info, seq_max_ts, q_scale, qv, qlo, part_lse, part_o, total;
};
MlaWorkspace mla_workspace_layout(int64_t batch, int workers) {
  MlaWorkspace w;
  int64_t off = 0;
  w.sched = off;      off += up256((int64_t)workers * 16);
  w.seq_info = off;   off += up256(batch * 8);
  w.seq_max_ts = off; off += up256(batch * 4);
  w.q_scale = off;    off += up256(batch * kMlaHeads * 4);
  w.qv = off;         off += up256(batch * kMlaQvBytes);
  w.qlo = off;        off += up256(batch * kMlaQloBytes);
  w.part_lse = off;   off += up256((int64_t)2 * workers * kMlaHeads * 4);
  w.part_o = off;     off += up256((int64_t)2 * workers * kMlaHeads * kMlaDV * 4);
  w.total = off;
  return w;
}
}  // namespace

bool mla_persistent_supported(int64_t batch) { return batch > 0 && batch <= kMlaSchedMaxBatch && sm_count() >= 2; }

int64_t mla_persistent_workspace_bytes(int64_t batch) {
  return batch > 0 ? mla_workspace_layout(batch, sm_count() / 2).total + 256 : 0;      // + room to align the base
}

template <typename TQ>
static int mla_persistent_launch_t(const CUtensorMap& tm_kv, const CUtensorMap& tm_q, const MlaPrepParams& pp,
                                   const MlaSchedParams& sp, const int2* seq_info, cudaStream_t s) {
  mla_prepare_kernel<TQ><<<(unsigned)(5 * pp.batch + 1), 256, 0, s>>>(pp);
  TL_LAUNCH_CHECK("mla_prepare_kernel");
  // the decode and merge kernels are launched with programmatic stream serialization: each starts
  // while its predecessor runs and waits inside (dependency_wait) before it reads the predecessor's output
  cudaLaunchAttribute overlap[1];
  overlap[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  overlap[0].val.programmaticStreamSerializationAllowed = 1;
  auto kernel = mla_decode_persistent_kernel<TQ>;
  TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmemP));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pp.workers));
  cfg.blockDim = dim3(kMlaThreads);
  cfg.dynamicSmemBytes = kMlaSmemP;
  cfg.stream = s;
  cfg.attrs = overlap;
  cfg.numAttrs = 1;
  TL_CUDA(cudaLaunchKernelEx(&cfg, kernel, tm_kv, tm_q, sp));
  count_launch();
  cudaLaunchConfig_t mcfg = {};
  mcfg.gridDim = dim3((unsigned)pp.workers, (unsigned)((pp.heads + 7) / 8));
  mcfg.blockDim = dim3(256);
  mcfg.stream = s;
  mcfg.attrs = overlap;
  mcfg.numAttrs = 1;
  TL_CUDA(cudaLaunchKernelEx(&mcfg, mla_merge_kernel<TQ>, (const float*)sp.part_o, (const float*)sp.part_lse,
                             (const int4*)sp.sched, seq_info, (TQ*)sp.out, (int)pp.heads));
  count_launch();
  return TL_B200_OK;
}

int mla_persistent_launch(const void* q, const void* kv_cache, const float* kv_scale, const int32_t* block_table,
                          const int32_t* cache_seqlens, void* out, int64_t batch, int64_t heads, int64_t page_size,
                          int64_t max_pages_per_seq, int64_t num_pages, float softmax_scale, int q_dtype,
                          void* workspace, cudaStream_t stream) {
  const int workers = sm_count() / 2;
  const MlaWorkspace w = mla_workspace_layout(batch, workers);
  char* ws = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(workspace) + 255u) & ~(uintptr_t)255u);

  CUtensorMap tm_kv, tm_q;
  {
    uint64_t dims[2] = {(uint64_t)kMlaD, (uint64_t)(num_pages * page_size)};
    uint64_t strides[1] = {(uint64_t)kMlaD};
    uint32_t box[2] = {128u, (uint32_t)kMlaBN};
    int rc = make_tensor_map(&tm_kv, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, kv_cache, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    uint64_t dims[2] = {128u, (uint64_t)(batch * kMlaSlabs * kMlaHeads)};
    uint64_t strides[1] = {128u};
    uint32_t box[2] = {128u, (uint32_t)kMlaHeads};
    int rc = make_tensor_map(&tm_q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, ws + w.qv, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  MlaPrepParams pp;
  pp.q = q; pp.kv_scale = kv_scale; pp.block_table = block_table; pp.seqlens = cache_seqlens;
  pp.qv = reinterpret_cast<uint8_t*>(ws + w.qv); pp.qlo = reinterpret_cast<uint8_t*>(ws + w.qlo);
  pp.q_scale = reinterpret_cast<float*>(ws + w.q_scale); pp.seq_max_ts = reinterpret_cast<float*>(ws + w.seq_max_ts);
  pp.sched = reinterpret_cast<int4*>(ws + w.sched); pp.seq_info = reinterpret_cast<int2*>(ws + w.seq_info);
  pp.batch = (int)batch; pp.heads = (int)heads; pp.page_size = (int)page_size; pp.max_pages = (int)max_pages_per_seq;
  pp.workers = workers;
  pp.len_cap = mla_len_cap(max_pages_per_seq, num_pages, page_size); pp.num_pages = (int)num_pages;
  MlaSchedParams sp;
  sp.qlo = pp.qlo; sp.q_scale = pp.q_scale; sp.seq_max_ts = pp.seq_max_ts; sp.kv_scale = kv_scale;
  sp.block_table = block_table; sp.seqlens = cache_seqlens; sp.sched = pp.sched; sp.out = out;
  sp.part_o = reinterpret_cast<float*>(ws + w.part_o); sp.part_lse = reinterpret_cast<float*>(ws + w.part_lse);
  sp.batch = (int)batch; sp.heads = (int)heads; sp.page_size = (int)page_size; sp.max_pages = (int)max_pages_per_seq;
  sp.len_cap = pp.len_cap; sp.num_pages = pp.num_pages;
  sp.scale_log2 = softmax_scale * 1.4426950408889634f;
  sp.status = device_status_word();
  if (q_dtype == TL_BF16) return mla_persistent_launch_t<__nv_bfloat16>(tm_kv, tm_q, pp, sp, pp.seq_info, stream);
  return mla_persistent_launch_t<__half>(tm_kv, tm_q, pp, sp, pp.seq_info, stream);
}

}  // namespace tl
