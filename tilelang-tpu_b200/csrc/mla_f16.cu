// MLA decode on tcgen05 for 16-bit (bf16 / fp16) latent caches: the reference's own MLA program
// (tpu_demo/ppl/deepseek_mla/mla_decode.py:9-121: fp16, dense cache, separate Q / Q_pe / KV / K_pe tensors)
// and the paged 16-bit form of examples/deepseek_mla/example_mla_decode_paged.py:20-97 at the DeepSeek shape
// (latent 512 + rope 64, V = the first 512 columns), with its variable kv-head count and several query tokens
// per sequence (:99-256).
//
//   S = scale * Q K^T (576 columns), P = online softmax (fp32 statistics, P rounded to the cache type before
//   the second product, as the program does), O += P K[:, :512], O / l at the end.
//
// One CTA pair per (sequence, kv head); each CTA owns 256 of the 512 output columns (the fp32 O accumulator of
// 128 rows x 512 columns alone would fill tensor memory) and both compute S.  The M = 128 rows of the MMAs are
// the (query token, head of the group) pairs of the kv head.  A key tile is 64 tokens: nine 128-byte column
// slabs (72 KB) per stage, two stages (loaded in two parts, and the MMA thread issues S and P V in the order they
// become ready: see there).  The same shared-memory image is the K-major operand of S = Q K^T and the
// MN-major operand of O += P V.  Q does not fit beside two stages in shared memory (147 KB), so its first 256
// columns live in tensor memory (128 columns, the A operand comes from there) and the other 320 in shared
// memory (80 KB).  Tensor memory: S/P buffers [0,64) and [64,128), Q [128,256), O [256,512).
// Warp 0: TMA, warp 1: MMA issue, warp 2: tensor-memory allocation, warps 4-7: softmax and epilogue (one thread
// per row, all 64 tokens of a tile).  Every wait is bounded.
#include "sm100.cuh"

namespace tl {
using namespace sm100;

int mla_order_launch(const int* seqlens, int* order, int batch, cudaStream_t s);     // mla_decode.cu

constexpr int kFD = 576, kFDV = 512, kFRows = 128, kFBN = 64;
constexpr int kFSlabs = 9;                        // 64-column slabs of a 576-column row
constexpr int kFQTmemCols = 128;                  // columns 0..255 of Q as packed pairs
constexpr int kFQSmemSlabs = 5;                   // columns 256..575 of Q
constexpr int kFStageBytes = kFSlabs * kFBN * 128;            // 72 KB
constexpr int kFStages = 2;
constexpr int kFQBytes = kFQSmemSlabs * kFRows * 128;         // 80 KB
constexpr int kFOffKV = kFQBytes;
constexpr int kFOffBar = kFOffKV + kFStages * kFStageBytes;
constexpr int kFSmem = kFOffBar + 256 + 1024;
constexpr int kFThreads = 256;
constexpr int kFColS = 0, kFColQ = 128, kFColO = 256;

struct MlaF16Params {
  const void* q;               // rows of q_row_elems elements; row of (b, i, head) = ((b * s_q + i) * h_q + head)
  const int* block_table;      // [batch, max_pages]; nullptr: dense cache, sequence b starts at row b * dense_len
  const int* seqlens;          // [batch]; nullptr: every sequence holds dense_len tokens
  void* out;                   // [batch, s_q, h_q, 512]
  int batch, s_q, h_q, h_kv, group;      // group = h_q / h_kv heads per kv head; rows used = s_q * group <= 128
  int page_size, max_pages, num_pages, len_cap, dense_len;
  int q_row_elems;             // 576 (one tensor) or 512 (Q and Q_pe are two tensors)
  int split;                   // 1: the rope columns (512..575) come from the second pair of tensor maps
  int fmt;                     // kFmtF16 / kFmtBF16
  float scale_log2;
  int splits;                  // CTA pairs per (sequence, kv head); > 1: each writes a normalised fp32 partial + its log2-sum-exp
  float* part_o;               // [units * splits][128][512]
  float* part_lse;             // [units * splits][128]
  const int* order;            // sequences, longest first (nullptr: batch order)
  int* status;
};

template <typename T>
__global__ void __launch_bounds__(kFThreads, 1)
mla_decode_f16_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_qpe,
                      const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_kpe,
                      const MlaF16Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t sm_q = base;
  const uint32_t sm_kv = base + kFOffKV;
  const uint32_t bar0 = base + kFOffBar;
  const uint32_t bar_kvfull = bar0;                 // [2]
  const uint32_t bar_kvempty = bar0 + 16;           // [2]
  const uint32_t bar_sfull = bar0 + 32;             // [2]
  const uint32_t bar_pfull = bar0 + 48;             // [2]
  const uint32_t bar_pvdone = bar0 + 64;            // [2]
  const uint32_t bar_qfull = bar0 + 80;             // columns 256.. of Q have landed in shared memory
  const uint32_t bar_qtmem = bar0 + 88;             // columns 0..255 of Q are in tensor memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + kFOffBar + 96);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int half = blockIdx.x & 1;
  const int slot = blockIdx.x >> 1;                 // which (sequence, kv head, split) this CTA pair takes
  // CTAs are dealt the sequences longest first when the launch had scratch for the order: the long ones start early
  const int rank = slot / p.splits, split = slot % p.splits;
  const int b = p.order ? __ldg(p.order + rank / p.h_kv) : rank / p.h_kv, kvh = rank % p.h_kv;
  const int unit = b * p.h_kv + kvh;
  const int piece = unit * p.splits + split;        // where its partial goes
  const int rows_used = p.s_q * p.group;
  const int seqlen = p.seqlens ? min(max(__ldg(p.seqlens + b), 0), p.len_cap) : p.dense_len;
  // this CTA pair's contiguous share of the sequence's key tiles
  const int tiles_all = (seqlen + kFBN - 1) / kFBN;
  const int per_split = (tiles_all + p.splits - 1) / p.splits;
  const int t0 = min(split * per_split, tiles_all);
  const int n_tiles = min(tiles_all - t0, per_split);
  const int* table = p.block_table ? p.block_table + (int64_t)b * p.max_pages : nullptr;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_kvfull + 8 * i, 2);         // a stage arrives in two parts
      mbar_init(bar_kvempty + 8 * i, 1);
      mbar_init(bar_sfull + 8 * i, 1);
      mbar_init(bar_pfull + 8 * i, 4);
      mbar_init(bar_pvdone + 8 * i, 1);
    }
    mbar_init(bar_qfull, 1);
    mbar_init(bar_qtmem, 4);
    mbar_fence_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_kv);
    if (p.split) {
      prefetch_tensormap(&tm_qpe);
      prefetch_tensormap(&tm_kpe);
    }
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  auto stage_addr = [&](int s) { return sm_kv + s * kFStageBytes; };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && n_tiles > 0) {
      bool ok = true;
      // columns 256..575 of the query rows of this kv head: one box per query token (its `group` heads)
      const int box_rows = p.s_q == 1 ? kFRows : p.group;
      mbar_expect_tx(bar_qfull, (uint32_t)(p.s_q * box_rows * 128 * kFQSmemSlabs));
      for (int i = 0; i < p.s_q; ++i) {
        const int qrow = (b * p.s_q + i) * p.h_q + kvh * p.group;
        for (int s = 0; s < kFQSmemSlabs; ++s) {
          const uint32_t dst = sm_q + s * (kFRows * 128) + i * p.group * 128;
          if (p.split && s == 4) tma_load_2d(dst, &tm_qpe, bar_qfull, 0, qrow);
          else tma_load_2d(dst, &tm_q, bar_qfull, 256 + 64 * s, qrow);
        }
      }
      // A stage is loaded in two parts.  The five slabs that P V of this CTA does not read (the other CTA's half of the
      // V columns and the rope slab) are free as soon as S of the tile before last has retired, the four V slabs only
      // when its P V has: the first part's transfer runs under that tile's softmax and P V.
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        const int tok = (t0 + j) * kFBN;
        int row;
        if (table) {
          const int page = __ldg(table + tok / p.page_size);
          // a page id outside the cache reads row 0; the softmax masks the tile
          row = (unsigned)page < (unsigned)p.num_pages ? page * p.page_size + tok % p.page_size : 0;
        } else {
          row = b * p.dense_len + tok;
        }
        const uint32_t full = bar_kvfull + 8 * st;
        // the cache row of (token, kv head) starts at column kvh * 576 of the flattened [tokens, h_kv * 576] view
        const int col0 = kvh * (p.split ? kFDV : kFD);
        auto load_slab = [&](int sl) {
          const uint32_t dst = stage_addr(st) + sl * (kFBN * 128);
          if (p.split && sl == 8) tma_load_2d(dst, &tm_kpe, full, kvh * 64, row);
          else tma_load_2d(dst, &tm_kv, full, col0 + 64 * sl, row);
        };
        if (j >= 2 && !(ok = mbar_wait(bar_sfull + 8 * st, ((j - 2) >> 1) & 1, abort_flag))) break;   // S(j - 2) has retired
        mbar_expect_tx(full, 5 * kFBN * 128);
#pragma unroll
        for (int sl = 0; sl < kFSlabs; ++sl)
          if (sl < 4 * half || sl >= 4 * half + 4) load_slab(sl);
        if (!(ok = mbar_wait(bar_kvempty + 8 * st, ((j >> 1) & 1) ^ 1, abort_flag))) break;           // P V(j - 2) has retired
        mbar_expect_tx(full, 4 * kFBN * 128);
#pragma unroll
        for (int sl = 0; sl < 4; ++sl) load_slab(4 * half + sl);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // Two chains share the tensor pipe: S(t) needs the load of tile t, which can only start when P V(t-2) has retired
    // (two stages), and P V(t) needs the softmax of tile t.  Issued in a fixed order (S(t+1) before P V(t)) every P V
    // queues behind an S that is still waiting for its load, and a tile costs the load latency plus all its MMAs.
    // Here the thread issues whichever of the two is ready (P V first), so the chains of even and odd tiles interleave.
    if (elect_one() && n_tiles > 0) {
      const uint32_t idesc_s = make_idesc(p.fmt, p.fmt, false, false, kFRows, kFBN);
      const uint32_t idesc_o = make_idesc(p.fmt, p.fmt, false, true, kFRows, 256);
      const uint64_t q_desc = smem_desc_sw128(sm_q, 16, 1024), k_desc = smem_desc_sw128(sm_kv, 16, 1024);
      const uint64_t v_desc = smem_desc_sw128(sm_kv, kFBN * 128, 1024);
      auto issue_s = [&](int j) {               // the stage of tile j has landed
        const int st = j & 1;
        const uint64_t kd = desc_at(k_desc, st * kFStageBytes);
        const uint32_t d = tmem_base + kFColS + (j & 1) * kFBN;
        // columns 0..255: Q from tensor memory (8 columns of packed pairs per 16-element step)
#pragma unroll
        for (int kk = 0; kk < 16; ++kk)
          mma_f16_ts(d, tmem_base + kFColQ + kk * 8, desc_at(kd, (kk / 4) * (kFBN * 128) + (kk % 4) * 32), idesc_s,
                     kk ? 1u : 0u);
        // columns 256..575: Q from shared memory
#pragma unroll
        for (int kk = 16; kk < 36; ++kk)
          mma_f16_ss(d, desc_at(q_desc, ((kk - 16) / 4) * (kFRows * 128) + (kk % 4) * 32),
                     desc_at(kd, (kk / 4) * (kFBN * 128) + (kk % 4) * 32), idesc_s, 1u);
        mma_commit(bar_sfull + 8 * (j & 1));
      };
      auto issue_pv = [&](int j) {              // P(j) is in tensor memory
        // V: this CTA's 256 columns = slabs [4 half, 4 half + 4) of the stage, MN-major (slabs 8 KB apart)
        const uint64_t vd = desc_at(v_desc, (j & 1) * kFStageBytes + (4 * half) * (kFBN * 128));
        const uint32_t pa = tmem_base + kFColS + (j & 1) * kFBN;
#pragma unroll
        for (int kk = 0; kk < kFBN / 16; ++kk)
          mma_f16_ts(tmem_base + kFColO, pa + kk * 8, desc_at(vd, kk * 2048), idesc_o, (j | kk) ? 1u : 0u);
        mma_commit(bar_pvdone + 8 * (j & 1));
        mma_commit(bar_kvempty + 8 * (j & 1));
      };
      bool ok = mbar_wait(bar_qfull, 0, abort_flag) && mbar_wait(bar_qtmem, 0, abort_flag);
      int next_s = 0, next_pv = 0;              // S(t) goes into the buffer and stage of t - 2: at most two ahead of P V
      uint32_t spins = 0;
      unsigned long long t_idle = 0;
      while (ok && next_pv < n_tiles) {
        if (next_pv < next_s && mbar_try_wait(bar_pfull + 8 * (next_pv & 1), (next_pv >> 1) & 1)) {
          tc_fence_after_sync();
          issue_pv(next_pv++);
          spins = 0;
        } else if (next_s < n_tiles && next_s < next_pv + 2 && mbar_try_wait(bar_kvfull + 8 * (next_s & 1), (next_s >> 1) & 1)) {
          tc_fence_after_sync();
          issue_s(next_s++);
          spins = 0;
        } else if ((++spins & 63u) == 0) {      // nothing ready: a bounded wait, as everywhere
          if (*abort_flag) ok = false;
          else if (spins == 64u) t_idle = global_timer_ns();
          else if (global_timer_ns() - t_idle > kWaitBudgetNs) { *abort_flag = kStatusWaitTimeout; ok = false; }
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ Q to tensor memory, softmax, epilogue
    const int quarter = warp % 4;
    const int r = quarter * 32 + lane;               // row = TMEM lane = (query token, head of the group)
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const bool row_live = r < rows_used;
    const int qi = row_live ? r / p.group : 0, g = row_live ? r % p.group : 0;
    const int64_t grow = ((int64_t)b * p.s_q + qi) * p.h_q + kvh * p.group + g;       // row of q and of out
    bool ok = true;
    if (n_tiles > 0) {
      const uint4* qrow = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.q) + grow * p.q_row_elems);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {                  // 64 columns = 32 words per store
        uint32_t words[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 v = row_live ? __ldg(qrow + c * 8 + i) : make_uint4(0, 0, 0, 0);
          words[4 * i] = v.x; words[4 * i + 1] = v.y; words[4 * i + 2] = v.z; words[4 * i + 3] = v.w;
        }
        tmem_st_32x32(tmem_base + kFColQ + c * 32 + lane_off, words);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_qtmem);
    }
    // a query token i of s_q sees the keys up to seqlen - s_q + i (the causal rule of the paged example)
    const int row_len = row_live ? max(seqlen - (p.s_q - 1 - qi), 0) : 0;
    float m_used = -INFINITY, row_sum = 0.f;
    const uint32_t t_o = tmem_base + kFColO + lane_off;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const uint32_t t_s = tmem_base + kFColS + (j & 1) * kFBN + lane_off;
      int page_ok = 1;
      if (table) page_ok = (unsigned)__ldg(table + (t0 + j) * kFBN / p.page_size) < (unsigned)p.num_pages;
      ok = mbar_wait(bar_sfull + 8 * (j & 1), (j >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t sv[64];
      tmem_ld_32x64(t_s, sv);
      tmem_ld_wait_for(sv);
      const int valid = page_ok ? row_len - (t0 + j) * kFBN : 0;      // tokens of this tile the row may see
      float m_tile = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        if (c >= valid) sv[c] = __float_as_uint(-INFINITY);
        m_tile = fmaxf(m_tile, __uint_as_float(sv[c]));
      }
      m_tile *= p.scale_log2;
      const float m_new = fmaxf(m_used, m_tile);
      // the maximum in use may lag the true one by up to 8 binades: P stays below 2^8, O is rescaled rarely
      const bool grow_now = (m_used == -INFINITY) ? (m_new != -INFINITY) : (m_new - m_used > 8.0f);
      if (j > 0 && __any_sync(0xffffffffu, grow_now && m_used != -INFINITY)) {
        ok = mbar_wait(bar_pvdone + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        const float alpha = (grow_now && m_used != -INFINITY) ? ex2_approx(m_used - m_new) : 1.0f;
        row_sum *= alpha;
#pragma unroll 1
        for (int c = 0; c < 256 / 32; ++c) {
          uint32_t ov[32];
          tmem_ld_32x32(t_o + c * 32, ov);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
          tmem_st_32x32(t_o + c * 32, ov);
        }
        tmem_st_wait();
      }
      if (grow_now) m_used = m_new;
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
      uint32_t packed[32];
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float p0 = ex2_approx(fmaf(__uint_as_float(sv[c]), p.scale_log2, -m_safe));
        const float p1 = ex2_approx(fmaf(__uint_as_float(sv[c + 1]), p.scale_log2, -m_safe));
        sum += p0 + p1;
        Vec16<T> two;                                 // the first two elements are used
        two.e[0] = from_f32<T>(p0);
        two.e[1] = from_f32<T>(p1);
        packed[c >> 1] = two.raw.x;
      }
      row_sum += sum;
      tmem_st_32x32(t_s, packed);                     // P over the first half of its own S buffer
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pfull + 8 * (j & 1));
    }
    // epilogue: 256 output columns of the row; with several splits a normalised fp32 partial and its log2-sum-exp
    T* out = reinterpret_cast<T*>(p.out) + grow * kFDV + half * 256;
    float* po = p.splits > 1 ? p.part_o + ((int64_t)piece * kFRows + r) * kFDV + half * 256 : nullptr;
    if (n_tiles == 0) {
      if (p.splits > 1) {
        if (half == 0) p.part_lse[(int64_t)piece * kFRows + r] = -INFINITY;      // the merge gives this piece no weight
      } else if (row_live) {
        for (int c = 0; c < 256 / 8; ++c) reinterpret_cast<uint4*>(out)[c] = make_uint4(0, 0, 0, 0);
      }
    } else if (ok) {
      ok = mbar_wait(bar_pvdone + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after_sync();
        const float inv = row_sum > 0.f ? 1.0f / row_sum : 0.f;
        if (p.splits > 1 && half == 0)
          p.part_lse[(int64_t)piece * kFRows + r] = row_sum > 0.f ? m_used + log2f(row_sum) : -INFINITY;
#pragma unroll 1
        for (int c = 0; c < 256 / 32; ++c) {
          uint32_t ov[32];
          tmem_ld_32x32(t_o + c * 32, ov);
          tmem_ld_wait();
          if (p.splits > 1) {
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              *reinterpret_cast<float4*>(po + c * 32 + e) =
                  make_float4(__uint_as_float(ov[e]) * inv, __uint_as_float(ov[e + 1]) * inv, __uint_as_float(ov[e + 2]) * inv,
                              __uint_as_float(ov[e + 3]) * inv);
          } else if (row_live) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              Vec16<T> v;
#pragma unroll
              for (int i = 0; i < 8; ++i) v.e[i] = from_f32<T>(__uint_as_float(ov[e + i]) * inv);
              *reinterpret_cast<uint4*>(out + c * 32 + e) = v.raw;
            }
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(20000);      // let copies and MMAs in flight land before the CTA leaves
    if (threadIdx.x == 0 && p.status) *p.status = *abort_flag;
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// Merges the `splits` partials of every (sequence, kv head): out = sum_c 2^(lse_c - M) O_c / sum_c 2^(lse_c - M).
// One warp per row, a lane owns 16 of the 512 columns.
template <typename T>
__global__ void __launch_bounds__(256)
mla_f16_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, T* __restrict__ out, int splits,
                     int s_q, int h_q, int h_kv, int group) {
  const int unit = blockIdx.x, b = unit / h_kv, kvh = unit % h_kv;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int r = blockIdx.y * 8 + warp;
  if (r >= s_q * group) return;
  const int64_t grow = ((int64_t)b * s_q + r / group) * h_q + kvh * group + r % group;
  float m = -INFINITY;
  for (int c = 0; c < splits; ++c) m = fmaxf(m, part_lse[((int64_t)unit * splits + c) * kFRows + r]);
  float denom = 0.f;
  float4 acc[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c = 0; c < splits; ++c) {
    const int64_t piece = (int64_t)unit * splits + c;
    const float lse = part_lse[piece * kFRows + r];
    if (lse == -INFINITY) continue;                      // a piece without visible keys (its partial was not written)
    const float w = exp2f(lse - m);
    denom += w;
    const float4* src = reinterpret_cast<const float4*>(part_o + (piece * kFRows + r) * kFDV) + lane;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float4 v = src[k * 32];
      acc[k].x = fmaf(w, v.x, acc[k].x); acc[k].y = fmaf(w, v.y, acc[k].y);
      acc[k].z = fmaf(w, v.z, acc[k].z); acc[k].w = fmaf(w, v.w, acc[k].w);
    }
  }
  const float inv = denom > 0.f ? 1.0f / denom : 0.f;
  T* o = out + grow * kFDV + lane * 4;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    Vec16<T> v;                                // the first four elements are used: 8 bytes
    v.e[0] = from_f32<T>(acc[k].x * inv); v.e[1] = from_f32<T>(acc[k].y * inv);
    v.e[2] = from_f32<T>(acc[k].z * inv); v.e[3] = from_f32<T>(acc[k].w * inv);
    *reinterpret_cast<uint2*>(o + k * 128) = make_uint2(v.raw.x, v.raw.y);
  }
}

// ---- host ---------------------------------------------------------------------------------------
// Splits per (sequence, kv head): about three CTAs per SM in total (short CTAs even out sequences of different
// lengths), at most 8; fewer when the scratch is too small.
int mla_f16_splits(int64_t units, int64_t workspace_bytes) {
  int splits = (int)((3 * sm_count() + 2 * units - 1) / (2 * units));
  if (splits > 8) splits = 8;
  while (splits > 1 && units * splits * kFRows * (kFDV + 1) * 4 + units * 4 + 768 > workspace_bytes) --splits;
  return splits < 1 ? 1 : splits;
}

// Scratch that lets mla_f16_splits() choose freely for `units` (sequence, kv head) pairs.
int64_t mla_f16_workspace_bytes(int64_t units) {
  if (units <= 0) return 0;
  int64_t splits = (3 * sm_count() + 2 * units - 1) / (2 * units);
  if (splits > 8) splits = 8;
  if (splits <= 1) return 0;
  return units * splits * kFRows * (kFDV + 1) * 4 + units * 4 + 1024;      // partials, their log-sum-exp, the sequence order
}

bool mla_f16_shape_ok(int64_t s_q, int64_t h_q, int64_t h_kv, int64_t d, int64_t dv) {
  if (d != kFD || dv != kFDV || h_kv <= 0 || h_q % h_kv != 0 || s_q <= 0) return false;
  const int64_t group = h_q / h_kv;
  if (s_q * group > kFRows) return false;
  return s_q == 1 || group % 8 == 0;       // a query token's rows must start on an 8-row swizzle group
}

// q: [batch, s_q, h_q, q_row] (q_row = 576, or 512 with q_pe [batch, s_q, h_q, 64]); cache: [tokens, h_kv, 576]
// (or [tokens, h_kv, 512] with k_pe [tokens, h_kv, 64]); tokens = num_pages * page_size, or batch * dense_len.
int mla_f16_launch(const void* q, const void* q_pe, const void* kv, const void* k_pe, const int32_t* block_table,
                   const int32_t* seqlens, void* out, int64_t batch, int64_t s_q, int64_t h_q, int64_t h_kv,
                   int64_t total_tokens, int64_t page_size, int64_t max_pages, int64_t num_pages, int64_t dense_len,
                   float softmax_scale, int dtype, cudaStream_t stream, void* workspace, int64_t workspace_bytes) {
  const bool split = q_pe != nullptr;
  const int64_t group = h_q / h_kv;
  const CUtensorMapDataType dt = dtype == TL_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const uint32_t q_box_rows = (uint32_t)(s_q == 1 ? kFRows : group);
  CUtensorMap tm_q, tm_qpe, tm_kv, tm_kpe;
  const int64_t q_row = split ? kFDV : kFD, kv_row = h_kv * (split ? kFDV : kFD);
  auto encode = [&](CUtensorMap* m, const void* ptr, int64_t cols, int64_t rows, uint32_t box_rows) {
    uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
    uint64_t strides[1] = {(uint64_t)cols * 2};
    uint32_t box[2] = {64u, box_rows};
    return make_tensor_map(m, dt, 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  int rc = encode(&tm_q, q, q_row, batch * s_q * h_q, q_box_rows);
  if (rc) return rc;
  rc = encode(&tm_kv, kv, kv_row, total_tokens, (uint32_t)kFBN);
  if (rc) return rc;
  if (split) {
    rc = encode(&tm_qpe, q_pe, 64, batch * s_q * h_q, q_box_rows);
    if (rc) return rc;
    rc = encode(&tm_kpe, k_pe, h_kv * 64, total_tokens, (uint32_t)kFBN);
    if (rc) return rc;
  } else {
    tm_qpe = tm_q;
    tm_kpe = tm_kv;
  }
  MlaF16Params p;
  p.q = q; p.block_table = block_table; p.seqlens = seqlens; p.out = out;
  p.batch = (int)batch; p.s_q = (int)s_q; p.h_q = (int)h_q; p.h_kv = (int)h_kv; p.group = (int)group;
  p.page_size = (int)page_size; p.max_pages = (int)max_pages; p.num_pages = (int)num_pages;
  {
    const int64_t cap = (max_pages < num_pages ? max_pages : num_pages) * page_size;
    p.len_cap = (int)(cap < 0x7fffffc0ll ? cap : 0x7fffffc0ll);
  }
  p.dense_len = (int)dense_len;
  p.q_row_elems = (int)q_row;
  p.split = split ? 1 : 0;
  p.fmt = dtype == TL_BF16 ? kFmtBF16 : kFmtF16;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = device_status_word();
  // Few (sequence, kv head) units leave SMs idle: with scratch from the caller every unit is cut into `splits`
  // contiguous shares of its key tiles (split-KV as in examples/deepseek_mla/example_mla_decode_paged.py:99-221) and a
  // second kernel merges the normalised partials by their log-sum-exp.
  const int64_t units = batch * h_kv;
  p.splits = workspace ? mla_f16_splits(units, workspace_bytes) : 1;
  p.part_o = nullptr; p.part_lse = nullptr; p.order = nullptr;
  if (p.splits > 1) {
    char* ws = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(workspace) + 255u) & ~(uintptr_t)255u);
    p.part_lse = reinterpret_cast<float*>(ws);
    p.part_o = reinterpret_cast<float*>(ws + ((units * p.splits * kFRows * 4 + 255) / 256) * 256);
    if (seqlens) {             // sequences of different lengths: the longest first
      int* order = reinterpret_cast<int*>(reinterpret_cast<char*>(p.part_o) + units * p.splits * kFRows * kFDV * 4);
      rc = mla_order_launch(seqlens, order, (int)batch, stream);
      if (rc) return rc;
      p.order = order;
    }
  }
  const unsigned grid = (unsigned)(2 * units * p.splits);
  if (dtype == TL_BF16) {
    auto kernel = mla_decode_f16_kernel<__nv_bfloat16>;
    TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFSmem));
    kernel<<<grid, kFThreads, kFSmem, stream>>>(tm_q, tm_qpe, tm_kv, tm_kpe, p);
  } else {
    auto kernel = mla_decode_f16_kernel<__half>;
    TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFSmem));
    kernel<<<grid, kFThreads, kFSmem, stream>>>(tm_q, tm_qpe, tm_kv, tm_kpe, p);
  }
  TL_LAUNCH_CHECK("mla_decode_f16_kernel");
  if (p.splits > 1) {
    const dim3 mgrid((unsigned)units, (unsigned)((s_q * group + 7) / 8));
    if (dtype == TL_BF16)
      mla_f16_merge_kernel<__nv_bfloat16><<<mgrid, 256, 0, stream>>>(p.part_o, p.part_lse, (__nv_bfloat16*)out, p.splits, (int)s_q,
                                                                   (int)h_q, (int)h_kv, (int)group);
    else
      mla_f16_merge_kernel<__half><<<mgrid, 256, 0, stream>>>(p.part_o, p.part_lse, (__half*)out, p.splits, (int)s_q, (int)h_q,
                                                           (int)h_kv, (int)group);
    TL_LAUNCH_CHECK("mla_f16_merge_kernel");
  }
  return TL_B200_OK;
}

}  // namespace tl
