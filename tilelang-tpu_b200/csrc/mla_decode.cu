// MLA decode (one query token per sequence) over a PAGED latent KV cache.
//
//   scores[h,t] = softmax_scale * q[h,:] . K[t,:]        K[t,:] = cache[t,:] (* scale[t] for FP8)
//   out[h,:]    = softmax(scores)[h,:] . K[:, :dv]        (V is the first dv columns of the latent)
//
// Paged semantics follow examples/deepseek_mla/example_mla_decode_paged.py:20-97,259-308 of the
// reference (block table int32 [batch, max_pages], cache_seqlens int32 [batch], tail tokens of the
// last page masked); the FP8 cache with one fp32 scale per token is the benchmark's extension.
//
// tcgen05 kernel (e4m3 cache, d = 576, dv = 512, <= 128 heads, page size a multiple of 64).  The
// cache bytes are used by the tensor core exactly as they sit in HBM: TMA drops each 64-token
// page slice into shared memory (128-byte swizzle, 128-column slabs) and the SAME image is the
// K-major operand of S = Q K^T and the MN-major operand of O += P V, so nothing is ever
// de-quantised elementwise.  The per-token scale multiplies the S columns after the first MMA
// and the P columns before the second.  Q (bf16/fp16) and P are each split into two e4m3 terms
// (value + residual, one scale per head for Q), so both products keep ~8 mantissa bits; Q's
// residual term and P live in tensor memory and enter the MMAs as the A operand from there.
// The fp32 O accumulator for 128 heads x 512 columns alone would fill tensor memory, so two CTAs
// share a sequence, each owning 256 output columns (S is computed by both).
//
// Two kernels run this arithmetic.  The one in this file takes one CTA pair per sequence, longest
// sequence first (a small pre-kernel orders them; scratch: one int32 per sequence), and cuts the
// query inside every CTA; it needs almost no workspace and serves the allocation-free entry point.
// mla_persistent.cu holds the persistent, work-balanced kernel that the large workspace selects.
//
// Other shapes / cache dtypes run a one-thread-per-(sequence, head) FMA kernel.
#include "mla_common.cuh"

#include <algorithm>
#include <type_traits>

namespace tl {

struct MlaParams {
  const void* q;               // [batch, heads, 576]
  const float* kv_scale;       // [num_pages * page_size]
  const int* block_table;      // [batch, max_pages]
  const int* seqlens;          // [batch]
  const int* order;            // [batch] sequence ids, longest first
  void* out;                   // [batch, heads, 512]
  int batch, heads, page_size, max_pages;
  int len_cap, num_pages;      // bounds for the lengths and page ids read on the device
  float scale_log2;
  int* status;
};

__global__ void mla_order_kernel(const int* __restrict__ seqlens, int* __restrict__ order, int batch) {
  for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < batch; b += gridDim.x * blockDim.x) {
    const int len = seqlens[b];
    int rank = 0;
    for (int o = 0; o < batch; ++o) {
      const int lo = seqlens[o];
      rank += (lo > len) || (lo == len && o < b);
    }
    order[rank] = b;
  }
}

// order[rank] = sequence, longest first (ties: lower index first); every entry of order[0, batch) is written
int mla_order_launch(const int* seqlens, int* order, int batch, cudaStream_t s) {
  mla_order_kernel<<<(unsigned)((batch + 255) / 256), 256, 0, s>>>(seqlens, order, batch);
  TL_LAUNCH_CHECK("mla_order_kernel");
  return TL_B200_OK;
}

template <typename TQ>
__global__ void __launch_bounds__(kMlaThreads, 1)
mla_decode_fp8_kernel(const __grid_constant__ CUtensorMap tm_kv, const MlaParams p) {
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
  const uint32_t bar_qready = bar_pvdone + 16;
  // the two softmax warpgroups meet on mbarriers (bounded waits), never on bar.sync
  const uint32_t bar_xch = bar_qready + 8;                   // [2 tile parities]
  const uint32_t bar_pre = bar_xch + 16;
  const uint32_t bar_post = bar_pre + 8;
  const uint32_t bar_qpark = bar_post + 8;                   // all residual bytes of Q are parked
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + kMlaOffBar + 8 * (2 * kMlaStages + 12));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // exchange area of the two softmax warpgroups: [2 tile parities][2 warpgroups][128 rows] floats
  float* exch = reinterpret_cast<float*>(base_ptr + kMlaOffBar + 1024);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int b = p.order[blockIdx.x >> 1];
  const int half = blockIdx.x & 1;
  const int seqlen = mla_len(p.seqlens, b, p.len_cap);
  const int n_tiles = (seqlen + kMlaBN - 1) / kMlaBN;
  const int* table = p.block_table + (int64_t)b * p.max_pages;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kMlaStages; ++s) {
      mbar_init(bar_kvfull + 8 * s, 1);
      mbar_init(bar_kvempty + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_sfull + 8 * i, 1);
      mbar_init(bar_pfull + 8 * i, kMlaSoftmaxWarps);
      mbar_init(bar_pvdone + 8 * i, 1);
    }
    mbar_init(bar_qready, kMlaSoftmaxWarps);
    mbar_init(bar_xch, kMlaSoftmaxWarps);
    mbar_init(bar_xch + 8, kMlaSoftmaxWarps);
    mbar_init(bar_pre, kMlaSoftmaxWarps);
    mbar_init(bar_post, kMlaSoftmaxWarps);
    mbar_init(bar_qpark, kMlaSoftmaxWarps);
    mbar_fence_init();
    prefetch_tensormap(&tm_kv);
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j % kMlaStages;
        const uint32_t ph = (j / kMlaStages) & 1;
        if (!(ok = mbar_wait(bar_kvempty + 8 * st, ph ^ 1, abort_flag))) break;
        if (j == 1 && !(ok = mbar_wait(bar_qready, 0, abort_flag))) break;   // stages 1-2 park Q's residual until then
        const int tok = j * kMlaBN;
        const int page = __ldg(table + tok / p.page_size);
        // row of the flattened cache; a page id outside the cache reads row 0 and the softmax masks the tile
        const int row = mla_page_ok(page, p.num_pages) ? page * p.page_size + tok % p.page_size : 0;
        const uint32_t full = bar_kvfull + 8 * st;
        mbar_expect_tx(full, kMlaStageBytes);
#pragma unroll
        for (int s = 0; s < kMlaSlabs; ++s)           // columns 576..639 of the last slab are out of range: zero fill
          tma_load_2d(stage_addr(st) + s * (kMlaBN * 128), &tm_kv, full, s * 128, row);
        bulk_load(stage_addr(st) + kMlaTile, p.kv_scale + row, kMlaBN * 4, full);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // S runs two tiles ahead of P V:  S(0) S(1) | PV(0) S(2) | PV(1) S(3) | ...
    if (elect_one() && n_tiles > 0) {
      const uint32_t idesc_s = make_idesc(kFmtE4M3, kFmtE4M3, false, false, kMlaHeads, kMlaBN);
      const uint32_t idesc_o = make_idesc(kFmtE4M3, kFmtE4M3, false, true, kMlaHeads, 256);
      // descriptors are built once; every MMA's operands are a constant byte offset further on
      const uint64_t q_desc = smem_desc_sw128(sm_q, 16, 1024), k_desc = smem_desc_sw128(sm_kv, 16, 1024);
      const uint64_t v_desc = smem_desc_sw128(sm_kv, kMlaBN * 128, 1024);
      bool ok = true;
      auto issue_s = [&](int j) {
        const int st = j % kMlaStages;
        if (!(ok = mbar_wait(bar_kvfull + 8 * st, (j / kMlaStages) & 1, abort_flag))) return;
        tc_fence_after_sync();
        const uint64_t kd = desc_at(k_desc, st * (kMlaTile + 1024));        // this stage, K-major view
        const uint32_t d = tmem_base + kMlaColS + (j & 1) * kMlaBN;
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
        mma_commit(bar_sfull + 8 * (j & 1));
      };
      ok = mbar_wait(bar_qready, 0, abort_flag);
      if (ok) issue_s(0);
      if (ok && n_tiles > 1) issue_s(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (!(ok = mbar_wait(bar_pfull + 8 * (j & 1), (j >> 1) & 1, abort_flag))) break;
        tc_fence_after_sync();
        const uint64_t vd = desc_at(v_desc, (j % kMlaStages) * (kMlaTile + 1024) + (2 * half) * (kMlaBN * 128));
        const uint32_t pa = tmem_base + kMlaColS + (j & 1) * kMlaBN;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          // A: P row = [value(64 tokens) | residual(64 tokens)] in 32 columns, 8 columns per step.
          // B: this half's 256 V columns = two 128-column slabs (8 KB apart), 32 tokens = 4 KB per
          // step; the residual steps reuse the same tokens.
          mma_f8_ts(tmem_base + kMlaColO, pa + kk * 8, desc_at(vd, (kk & 1) * 4096), idesc_o, (j | kk) ? 1u : 0u);
        }
        mma_commit(bar_pvdone + 8 * (j & 1));
        mma_commit(bar_kvempty + 8 * (j % kMlaStages));
        if (j + 2 < n_tiles) issue_s(j + 2);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ Q quantisation, softmax, epilogue
    const int wg = (warp - 4) / 4;                // 0: tokens 0-31 of a tile, 1: tokens 32-63
    const int quarter = warp % 4;
    const int h = quarter * 32 + lane;            // head = TMEM lane
    const int st_id = threadIdx.x - 128;          // 0..255 among the softmax threads
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    // (1) quantise the 128 query rows: q ~ (v + r) * q_scale with v, r in e4m3.  A warp takes
    //     one row at a time so the global reads are coalesced: 36 units of 16 columns, lanes 0-31
    //     take units 0-31, lanes 0-3 also units 32-35.  The value term goes straight to its place in
    //     shared memory; the residual of columns 0..511 is parked in key/value stages 1-2 (the
    //     producer fills them only after this phase) and moved to tensor memory by the row's owner.
    float* q_scales = exch + 1040;                                   // 128 floats
    constexpr int kLoPitch = 528;                                    // 512 + 16: conflict-free 16-byte reads
    uint8_t* park = base_ptr + (stage_addr(1) - base);
    auto quant16 = [](const float (&f)[16], uint32_t (&val)[4], uint32_t (&res)[4]) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        val[w] = pack_e4m3x4(f[4 * w], f[4 * w + 1], f[4 * w + 2], f[4 * w + 3]);
        const float2 a = e4m3x2_to_float2(val[w]), c = e4m3x2_to_float2(val[w] >> 16);
        res[w] = pack_e4m3x4(f[4 * w] - a.x, f[4 * w + 1] - a.y, f[4 * w + 2] - c.x, f[4 * w + 3] - c.y);
      }
    };
    for (int r = warp - 4; r < kMlaHeads; r += kMlaSoftmaxWarps) {
      const bool live = r < p.heads;
      const uint4* qrow = reinterpret_cast<const uint4*>(reinterpret_cast<const TQ*>(p.q) + ((int64_t)b * p.heads + r) * kMlaD);
      Vec16<TQ> in[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) in[i].raw = make_uint4(0, 0, 0, 0);
      if (live) {
        in[0].raw = __ldg(qrow + 2 * lane);
        in[1].raw = __ldg(qrow + 2 * lane + 1);
        if (lane < 4) {
          in[2].raw = __ldg(qrow + 64 + 2 * lane);
          in[3].raw = __ldg(qrow + 65 + 2 * lane);
        }
      }
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(to_f32(in[i].e[e])));
      amax = fmaxf(warp_max(amax), 1e-10f);
      const float inv = 448.0f / amax;
      if (lane == 0) q_scales[r] = amax / 448.0f;
#pragma unroll
      for (int u2 = 0; u2 < 2; ++u2) {
        if (u2 == 1 && lane >= 4) break;
        const int unit = u2 == 0 ? lane : 32 + lane;                 // 16 columns = 16 bytes of e4m3
        float f[16];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          f[e] = to_f32(in[2 * u2].e[e]) * inv;
          f[8 + e] = to_f32(in[2 * u2 + 1].e[e]) * inv;
        }
        uint32_t val[4], res[4];
        quant16(f, val, res);
        const int slab = unit / 8, c = unit % 8;
        const uint32_t row_addr = sm_q + slab * (kMlaHeads * 128) + r * 128;
        st_shared_v4(row_addr + ((c ^ (r & 7)) << 4), val[0], val[1], val[2], val[3]);
        if (slab == 4)
          st_shared_v4(row_addr + (((c + 4) ^ (r & 7)) << 4), res[0], res[1], res[2], res[3]);
        else
          *reinterpret_cast<uint4*>(park + r * kLoPitch + unit * 16) = make_uint4(res[0], res[1], res[2], res[3]);
      }
    }
    fence_proxy_async_smem();                    // the value term is read by the tensor core from shared memory
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_qpark);
    bool ok = mbar_wait(bar_qpark, 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    const float q_scale = q_scales[h];
    if (wg == 1 && ok) {
      // residual term of columns 0..511 of row h -> tensor memory, 32 words per store
#pragma unroll 1
      for (int c128 = 0; c128 < 4; ++c128) {
        uint32_t words[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 v = *reinterpret_cast<const uint4*>(park + h * kLoPitch + (c128 * 8 + i) * 16);
          words[4 * i] = v.x; words[4 * i + 1] = v.y; words[4 * i + 2] = v.z; words[4 * i + 3] = v.w;
        }
        tmem_st_32x32(tmem_base + kMlaColQlo + c128 * 32 + lane_off, words);
      }
      tmem_st_wait();
      tc_fence_before_sync();
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_qready);
    // (2) largest token scale of the sequence: P is multiplied by 32 * scale[t] / max_scale before
    //     it is cut to e4m3, which keeps it inside (0, 256]
    float max_ts = 0.f;
    const int tok_end = seqlen;
    // four tokens per load: a page holds a multiple of 64 tokens, so a group of four never straddles pages
#pragma unroll 4
    for (int t = st_id * 4; t < tok_end; t += kMlaSoftmaxThreads * 4) {
      const int page = __ldg(table + t / p.page_size);
      if (!mla_page_ok(page, p.num_pages)) continue;           // masked tile
      const float4 v = __ldg(reinterpret_cast<const float4*>(p.kv_scale + (int64_t)page * p.page_size + t % p.page_size));
      max_ts = fmaxf(max_ts, v.x);                              // slots past the end hold arbitrary bytes
      if (t + 1 < tok_end) max_ts = fmaxf(max_ts, v.y);
      if (t + 2 < tok_end) max_ts = fmaxf(max_ts, v.z);
      if (t + 3 < tok_end) max_ts = fmaxf(max_ts, v.w);
    }
    max_ts = warp_max(max_ts);
    {
      float* pre = exch + 1024;                     // its own 8 floats, apart from the per-tile area
      if (lane == 0) { pre[warp - 4] = max_ts; mbar_arrive(bar_pre); }
      ok = mbar_wait(bar_pre, 0, abort_flag) && ok;
      ok = __all_sync(0xffffffffu, ok);
      max_ts = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) max_ts = fmaxf(max_ts, pre[i]);
    }
    constexpr float kPScale = 32.0f;
    const float ts_norm = max_ts > 0.f ? kPScale / max_ts : kPScale;
    const float s_scale = q_scale * p.scale_log2;

    // (3) online softmax: a row is shared by one thread of each warpgroup (32 tokens each)
    float m_used = -INFINITY, row_sum = 0.f;
    const uint32_t t_o = tmem_base + kMlaColO + wg * 128 + lane_off;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const uint32_t t_s = tmem_base + kMlaColS + (j & 1) * kMlaBN + lane_off;
      const int tile_page = __ldg(table + j * kMlaBN / p.page_size);                 // on its way during the wait
      ok = mbar_wait(bar_sfull + 8 * (j & 1), (j >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t sv[32];
      tmem_ld_32x32(t_s + wg * 32, sv);
      tmem_ld_wait();
      const float4* ts4 = reinterpret_cast<const float4*>(base_ptr + (stage_addr(j % kMlaStages) - base) + kMlaTile) + wg * 8;
      // tokens of this half tile that exist; none if the tile's page id is outside the cache
      const int valid = mla_page_ok(tile_page, p.num_pages) ? seqlen - j * kMlaBN - wg * 32 : 0;
      // sp = acc * token_scale (packed pairs); the per-head factor s_scale > 0 is applied inside the
      // exponent, so the row maximum can be taken on sp
      float2 sp[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 t = ts4[i];
        sp[2 * i] = mul2(make_float2(__uint_as_float(sv[4 * i]), __uint_as_float(sv[4 * i + 1])), make_float2(t.x, t.y));
        sp[2 * i + 1] = mul2(make_float2(__uint_as_float(sv[4 * i + 2]), __uint_as_float(sv[4 * i + 3])), make_float2(t.z, t.w));
      }
      if (valid < 32) {                                      // last tile of the sequence only
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (c >= valid) reinterpret_cast<float*>(sp)[c] = -INFINITY;
      }
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        m4[0] = fmaxf(m4[0], sp[i].x); m4[1] = fmaxf(m4[1], sp[i].y);
        m4[2] = fmaxf(m4[2], sp[i + 1].x); m4[3] = fmaxf(m4[3], sp[i + 1].y);
      }
      float* ex = exch + (j & 1) * 256;
      ex[wg * 128 + h] = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_xch + 8 * (j & 1));
      ok = mbar_wait(bar_xch + 8 * (j & 1), (j >> 1) & 1, abort_flag);   // also: all of S is in registers now
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const float m_tile = fmaxf(ex[h], ex[128 + h]) * s_scale;
      const float m_new = fmaxf(m_used, m_tile);
      // e4m3 has little dynamic range (largest 448, smallest normal 2^-6), so P is kept in (0, 8] -
      // the running maximum may lag by at most three binades - and scaled by kPScale = 32 before it
      // is cut to its two e4m3 terms
      const bool grow = (j == 0) || (m_new - m_used > 3.0f);
      if (j > 0 && __any_sync(0xffffffffu, grow && m_used != -INFINITY)) {
        ok = mbar_wait(bar_pvdone + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        const float alpha = (grow && m_used != -INFINITY) ? ex2_approx(m_used - m_new) : 1.0f;
        row_sum *= alpha;
#pragma unroll 1
        for (int c = 0; c < 128 / 32; ++c) {
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
      uint32_t hi[8], lo[8];
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
      for (int i = 0; i < 8; ++i) {
        const float4 t = ts4[i];
        const float2 a0 = fma2(sp[2 * i], k2, nm2), a1 = fma2(sp[2 * i + 1], k2, nm2);
        const float2 p0 = make_float2(ex2_approx(a0.x), ex2_approx(a0.y));
        const float2 p1 = make_float2(ex2_approx(a1.x), ex2_approx(a1.y));
        sum2a = add2(sum2a, p0);
        sum2b = add2(sum2b, p1);
        float2 w0 = mul2(p0, mul2(make_float2(t.x, t.y), n2));
        float2 w1 = mul2(p1, mul2(make_float2(t.z, t.w), n2));
        if (valid < 32) {        // token scales of slots past the end are arbitrary bytes
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
      tmem_st_32x8(t_s + wg * 8, hi);
      tmem_st_32x8(t_s + 16 + wg * 8, lo);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pfull + 8 * (j & 1));
    }
    // (4) epilogue: each warpgroup writes 128 of this CTA's 256 output columns
    TQ* out = reinterpret_cast<TQ*>(p.out) + ((int64_t)b * p.heads + h) * kMlaDV + half * 256 + wg * 128;
    if (n_tiles == 0) {
      if (h < p.heads)                        // an empty sequence: zeros
        for (int c = 0; c < 128 / 8; ++c) reinterpret_cast<uint4*>(out)[c] = make_uint4(0, 0, 0, 0);
    } else {
      ok = ok && mbar_wait(bar_pvdone + 8 * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      float* ex = exch + 512;
      ex[wg * 128 + h] = row_sum;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_post);
      ok = mbar_wait(bar_post, 0, abort_flag) && ok;
      ok = __all_sync(0xffffffffu, ok);
      const float total = ex[h] + ex[128 + h];
      if (ok) {
        tc_fence_after_sync();
        const float inv = total > 0.f ? max_ts / (kPScale * total) : 0.f;     // undo the P normalisation
#pragma unroll 1
        for (int c = 0; c < 128 / 32; ++c) {
          uint32_t ov[32];
          tmem_ld_32x32(t_o + c * 32, ov);
          tmem_ld_wait();
          if (h < p.heads) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              Vec16<TQ> v;
#pragma unroll
              for (int i = 0; i < 8; ++i) v.e[i] = from_f32<TQ>(__uint_as_float(ov[e + i]) * inv);
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
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
    if (threadIdx.x == 0 && p.status) *p.status = *abort_flag;
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kMlaTmemCols);
  }
}

// =================================================================================
// FMA kernel: one thread per (sequence, head); any d / dv <= 512, any page size, cache in
// e4m3 (+ per-token scale), fp16 or bf16.
// =================================================================================
template <typename T> __device__ __forceinline__ float cache_f32(const T* p) { return to_f32(*p); }
template <> __device__ __forceinline__ float cache_f32<__nv_fp8_e4m3>(const __nv_fp8_e4m3* p) { return float(*p); }

struct MlaRowParams {
  const void *q, *cache;
  const float* kv_scale;
  const int *block_table, *seqlens;
  void* out;
  int batch, heads, d, dv, page_size, max_pages;
  int len_cap, num_pages;
  int s_q, h_kv;               // query tokens per sequence and kv heads (1, 1 in the single-token MLA form)
  float scale;
};

template <typename TQ, typename TC, int MAXDV>
__global__ void __launch_bounds__(128)
mla_rows_kernel(const MlaRowParams p) {
  // one thread per (sequence, query token, head); q and out are [batch, s_q, heads, .], the cache [tokens, h_kv, d]
  const int idx = blockIdx.x * 128 + threadIdx.x;
  if (idx >= p.batch * p.s_q * p.heads) return;
  const int b = idx / (p.s_q * p.heads);
  const int qi = (idx / p.heads) % p.s_q, kvh = (idx % p.heads) / (p.heads / p.h_kv);
  const TQ* q = (const TQ*)p.q + (int64_t)idx * p.d;
  const int* table = p.block_table + (int64_t)b * p.max_pages;
  // query token qi of s_q sees the keys up to len - s_q + qi (examples/deepseek_mla/example_mla_decode_paged.py:266-274)
  const int seqlen = max(mla_len(p.seqlens, b, p.len_cap) - (p.s_q - 1 - qi), 0);
  float acc[MAXDV];
#pragma unroll
  for (int i = 0; i < MAXDV; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int t = 0; t < seqlen; ++t) {
    const int page = table[t / p.page_size];
    if (!mla_page_ok(page, p.num_pages)) continue;             // a page id outside the cache: its tokens are masked
    const int64_t row = (int64_t)page * p.page_size + t % p.page_size;
    const TC* kr = (const TC*)p.cache + (row * p.h_kv + kvh) * p.d;
    const float ts = p.kv_scale ? p.kv_scale[row] : 1.f;
    float s = 0.f;
    for (int i = 0; i < p.d; ++i) s = fmaf(to_f32(q[i]), cache_f32<TC>(kr + i), s);
    s *= ts * p.scale;
    const float m_new = fmaxf(m, s);
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float pj = expf(s - m_new);
    l = l * alpha + pj;
    const float w = pj * ts;
#pragma unroll
    for (int i = 0; i < MAXDV; ++i)
      if (i < p.dv) acc[i] = fmaf(w, cache_f32<TC>(kr + i), acc[i] * alpha);
    m = m_new;
  }
  TQ* out = (TQ*)p.out + (int64_t)idx * p.dv;
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < MAXDV; ++i)
    if (i < p.dv) out[i] = from_f32<TQ>(acc[i] * inv);
}

template <typename TQ, typename TC>
static int launch_mla_rows(const MlaRowParams& p, cudaStream_t s) {
  const unsigned grid = (unsigned)((p.batch * p.s_q * p.heads + 127) / 128);
  if (p.dv <= 64) mla_rows_kernel<TQ, TC, 64><<<grid, 128, 0, s>>>(p);
  else mla_rows_kernel<TQ, TC, 512><<<grid, 128, 0, s>>>(p);
  TL_LAUNCH_CHECK("mla_rows_kernel");
  return TL_B200_OK;
}

template <typename TQ>
static int launch_mla_rows_cache(const MlaRowParams& p, int cache_dtype, cudaStream_t s) {
  switch (cache_dtype) {
    case TL_E4M3: return launch_mla_rows<TQ, __nv_fp8_e4m3>(p, s);
    case TL_F16: return launch_mla_rows<TQ, __half>(p, s);
    case TL_BF16: return launch_mla_rows<TQ, __nv_bfloat16>(p, s);
    default: return fail(TL_B200_EINVAL, "mla_decode_paged: unsupported cache dtype %d", cache_dtype);
  }
}

}  // namespace tl

using namespace tl;

extern "C" int64_t tl_b200_mla_decode_paged_workspace_bytes(int64_t batch) {
  return batch > 0 ? ((batch * 4 + 255) / 256) * 256 : 0;
}

extern "C" int64_t tl_b200_mla_decode_paged_split_workspace_bytes(int64_t batch, int64_t max_pages_per_seq,
                                                                 int64_t page_size) {
  if (batch <= 0 || max_pages_per_seq <= 0 || page_size <= 0) return 0;
  int64_t need = tl_b200_mla_decode_paged_workspace_bytes(batch);
  if (mla_persistent_supported(batch)) need = std::max(need, mla_persistent_workspace_bytes(batch));   // FP8 cache
  return std::max(need, mla_f16_workspace_bytes(batch));                                               // 16-bit cache, split-KV
}

extern "C" int tl_b200_mla_decode_paged(const void* q, const void* kv_cache, const float* kv_scale,
                                        const int32_t* block_table, const int32_t* cache_seqlens, void* out,
                                        int64_t batch, int64_t heads, int64_t d, int64_t dv, int64_t page_size,
                                        int64_t max_pages_per_seq, int64_t num_pages, float softmax_scale, int q_dtype,
                                        int cache_dtype, void* workspace, int64_t workspace_bytes, void* stream) {
  TL_REQUIRE(batch >= 0 && heads >= 0 && d > 0 && dv > 0 && page_size > 0 && max_pages_per_seq >= 0 && num_pages >= 0,
             "mla_decode_paged: bad size");
  TL_REQUIRE(dv <= d, "mla_decode_paged: dv (%lld) exceeds d (%lld)", (long long)dv, (long long)d);
  if (batch == 0 || heads == 0) return TL_B200_OK;
  TL_REQUIRE(q && kv_cache && block_table && cache_seqlens && out, "mla_decode_paged: null tensor pointer");
  TL_REQUIRE(q_dtype == TL_BF16 || q_dtype == TL_F16, "mla_decode_paged: q/out must be bfloat16 or float16");
  TL_REQUIRE(cache_dtype != TL_E4M3 || kv_scale, "mla_decode_paged: an e4m3 cache needs per-token scales");
  TL_REQUIRE(batch < (1 << 24) && num_pages * page_size < (1ll << 31), "mla_decode_paged: size too large");
  cudaStream_t s = (cudaStream_t)stream;
  const bool tc = cache_dtype == TL_E4M3 && d == kMlaD && dv == kMlaDV && heads <= kMlaHeads && page_size % kMlaBN == 0 &&
                  aligned16(q) && aligned16(out) && aligned16(kv_cache) && aligned16(kv_scale);
  if (tc) {
    // with the large workspace: the persistent, work-balanced kernel; with the small one: one CTA pair per sequence
    if (workspace && mla_persistent_supported(batch) && workspace_bytes >= mla_persistent_workspace_bytes(batch))
      return mla_persistent_launch(q, kv_cache, kv_scale, block_table, cache_seqlens, out, batch, heads, page_size,
                                   max_pages_per_seq, num_pages, softmax_scale, q_dtype, workspace, s);
    TL_REQUIRE(workspace && workspace_bytes >= tl_b200_mla_decode_paged_workspace_bytes(batch),
               "mla_decode_paged: workspace of %lld bytes required (tl_b200_mla_decode_paged_workspace_bytes)",
               (long long)tl_b200_mla_decode_paged_workspace_bytes(batch));
    CUtensorMap tm;
    uint64_t dims[2] = {(uint64_t)kMlaD, (uint64_t)(num_pages * page_size)};
    uint64_t strides[1] = {(uint64_t)kMlaD};
    uint32_t box[2] = {128u, (uint32_t)kMlaBN};
    int rc = make_tensor_map(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, kv_cache, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    int* order = reinterpret_cast<int*>(workspace);
    mla_order_kernel<<<(unsigned)((batch + 255) / 256), 256, 0, s>>>(cache_seqlens, order, (int)batch);
    TL_LAUNCH_CHECK("mla_order_kernel");
    MlaParams p;
    p.q = q; p.kv_scale = kv_scale; p.block_table = block_table; p.seqlens = cache_seqlens; p.order = order; p.out = out;
    p.batch = (int)batch; p.heads = (int)heads; p.page_size = (int)page_size; p.max_pages = (int)max_pages_per_seq;
    p.len_cap = mla_len_cap(max_pages_per_seq, num_pages, page_size); p.num_pages = (int)num_pages;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.status = device_status_word();
    const unsigned grid = (unsigned)(2 * batch);
    if (q_dtype == TL_BF16) {
      auto kernel = mla_decode_fp8_kernel<__nv_bfloat16>;
      TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmem));
      kernel<<<grid, kMlaThreads, kMlaSmem, s>>>(tm, p);
    } else {
      auto kernel = mla_decode_fp8_kernel<__half>;
      TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmem));
      kernel<<<grid, kMlaThreads, kMlaSmem, s>>>(tm, p);
    }
    TL_LAUNCH_CHECK("mla_decode_fp8_kernel");
    return TL_B200_OK;
  }
  // 16-bit cache of the query's type at the DeepSeek shape: the tcgen05 kernel of mla_f16.cu (no workspace)
  if (cache_dtype == q_dtype && mla_f16_shape_ok(1, heads, 1, d, dv) && page_size % kMlaBN == 0 && aligned16(q) &&
      aligned16(out) && aligned16(kv_cache))
    return mla_f16_launch(q, nullptr, kv_cache, nullptr, block_table, cache_seqlens, out, batch, 1, heads, 1,
                          num_pages * page_size, page_size, max_pages_per_seq, num_pages, 0, softmax_scale, q_dtype, s,
                          workspace, workspace_bytes);
  TL_REQUIRE(dv <= 512, "mla_decode_paged: dv above 512 is not supported");
  MlaRowParams rp;
  rp.q = q; rp.cache = kv_cache; rp.kv_scale = kv_scale; rp.block_table = block_table; rp.seqlens = cache_seqlens;
  rp.out = out; rp.batch = (int)batch; rp.heads = (int)heads; rp.d = (int)d; rp.dv = (int)dv;
  rp.page_size = (int)page_size; rp.max_pages = (int)max_pages_per_seq; rp.scale = softmax_scale;
  rp.len_cap = mla_len_cap(max_pages_per_seq, num_pages, page_size); rp.num_pages = (int)num_pages;
  rp.s_q = 1; rp.h_kv = 1;
  if (q_dtype == TL_BF16) return launch_mla_rows_cache<__nv_bfloat16>(rp, cache_dtype, s);
  return launch_mla_rows_cache<__half>(rp, cache_dtype, s);
}

// Several query tokens per sequence and several kv heads (examples/deepseek_mla/example_mla_decode_paged.py:99-256):
// q [batch, s_q, h_q, d], cache [num_pages, page_size, h_kv, d] of the same 16-bit type, out [batch, s_q, h_q, dv];
// head h reads kv head h / (h_q / h_kv); query token i sees the keys up to len - s_q + i.
extern "C" int tl_b200_mla_decode_paged_gqa(const void* q, const void* kv_cache, const int32_t* block_table,
                                            const int32_t* cache_seqlens, void* out, int64_t batch, int64_t s_q,
                                            int64_t h_q, int64_t h_kv, int64_t d, int64_t dv, int64_t page_size,
                                            int64_t max_pages_per_seq, int64_t num_pages, float softmax_scale, int dtype,
                                            void* stream) {
  TL_REQUIRE(batch >= 0 && s_q > 0 && h_q > 0 && h_kv > 0 && d > 0 && dv > 0 && page_size > 0 && max_pages_per_seq >= 0 &&
                 num_pages >= 0, "mla_decode_paged_gqa: bad size");
  TL_REQUIRE(h_q % h_kv == 0, "mla_decode_paged_gqa: h_q (%lld) must be a multiple of h_kv (%lld)", (long long)h_q, (long long)h_kv);
  TL_REQUIRE(dv <= d && dv <= 512, "mla_decode_paged_gqa: dv must not exceed d or 512");
  if (batch == 0) return TL_B200_OK;
  TL_REQUIRE(q && kv_cache && block_table && cache_seqlens && out, "mla_decode_paged_gqa: null tensor pointer");
  TL_REQUIRE(dtype == TL_BF16 || dtype == TL_F16, "mla_decode_paged_gqa: bfloat16 or float16");
  TL_REQUIRE(batch * s_q * h_q < (1ll << 31) && num_pages * page_size * h_kv < (1ll << 31), "mla_decode_paged_gqa: size too large");
  cudaStream_t s = (cudaStream_t)stream;
  if (mla_f16_shape_ok(s_q, h_q, h_kv, d, dv) && page_size % kMlaBN == 0 && aligned16(q) && aligned16(out) && aligned16(kv_cache))
    return mla_f16_launch(q, nullptr, kv_cache, nullptr, block_table, cache_seqlens, out, batch, s_q, h_q, h_kv,
                          num_pages * page_size, page_size, max_pages_per_seq, num_pages, 0, softmax_scale, dtype, s);
  MlaRowParams rp;
  rp.q = q; rp.cache = kv_cache; rp.kv_scale = nullptr; rp.block_table = block_table; rp.seqlens = cache_seqlens;
  rp.out = out; rp.batch = (int)batch; rp.heads = (int)h_q; rp.d = (int)d; rp.dv = (int)dv;
  rp.page_size = (int)page_size; rp.max_pages = (int)max_pages_per_seq; rp.scale = softmax_scale;
  rp.len_cap = mla_len_cap(max_pages_per_seq, num_pages, page_size); rp.num_pages = (int)num_pages;
  rp.s_q = (int)s_q; rp.h_kv = (int)h_kv;
  if (dtype == TL_BF16) return launch_mla_rows_cache<__nv_bfloat16>(rp, dtype, s);
  return launch_mla_rows_cache<__half>(rp, dtype, s);
}

// =================================================================================
// Allocation-free variant of the tensor-core path.
//
// Some callers cannot allocate device memory at the point where they decode: a serving loop
// whose memory pool is fully handed out to the KV cache, a plugin that runs inside someone
// else's allocator lock, or a host that forbids cudaMalloc once warm-up is over.  For them the
// one piece of scratch this kernel needs (the longest-first ordering of the sequences) lives in
// a fixed array inside the library image instead of a caller-provided workspace.  Every GPU
// that loads the library holds these 16 KB until the process exits.
// =================================================================================
namespace tl {
constexpr int kMlaNoAllocMaxBatch = 4096;
static __device__ __align__(256) int g_mla_order_scratch[kMlaNoAllocMaxBatch];

// In host code the array's name is only a handle for the runtime, not a device address, so the
// address is looked up once per device (with that device current) and cached.
constexpr int kMaxDevices = 64;
static std::atomic<int*> g_mla_order_ptr[kMaxDevices] = {};     // host threads may make their first calls together
}  // namespace tl

extern "C" int tl_b200_mla_decode_paged_noalloc(const void* q, const void* kv_cache, const float* kv_scale,
                                                const int32_t* block_table, const int32_t* cache_seqlens,
                                                void* out, int64_t batch, int64_t heads, int64_t page_size,
                                                int64_t max_pages_per_seq, int64_t num_pages, float softmax_scale,
                                                int q_dtype, void* stream) {
  TL_REQUIRE(batch >= 0 && heads >= 0 && page_size > 0 && max_pages_per_seq >= 0 && num_pages >= 0,
             "mla_decode_paged_noalloc: bad size");
  TL_REQUIRE(batch <= kMlaNoAllocMaxBatch,
             "mla_decode_paged_noalloc: batch %lld exceeds the built-in scratch (%d sequences); use "
             "tl_b200_mla_decode_paged with a caller-provided workspace", (long long)batch, kMlaNoAllocMaxBatch);
  if (batch == 0 || heads == 0) return TL_B200_OK;
  TL_REQUIRE(q && kv_cache && kv_scale && block_table && cache_seqlens && out,
             "mla_decode_paged_noalloc: null tensor pointer");
  TL_REQUIRE(q_dtype == TL_BF16 || q_dtype == TL_F16, "mla_decode_paged_noalloc: q/out must be bfloat16 or float16");
  TL_REQUIRE(heads <= kMlaHeads && page_size % kMlaBN == 0,
             "mla_decode_paged_noalloc: needs heads <= 128 and a page size that is a multiple of 64");
  TL_REQUIRE(num_pages * page_size < (1ll << 31), "mla_decode_paged_noalloc: cache too large");
  TL_REQUIRE(aligned16(q) && aligned16(out) && aligned16(kv_cache) && aligned16(kv_scale),
             "mla_decode_paged_noalloc: tensors must be 16-byte aligned");
  int dev = 0;
  TL_CUDA(cudaGetDevice(&dev));
  TL_REQUIRE(dev >= 0 && dev < kMaxDevices, "mla_decode_paged_noalloc: device index %d out of range", dev);
  int* order = g_mla_order_ptr[dev].load(std::memory_order_acquire);
  if (order == nullptr) {
    TL_CUDA(cudaGetSymbolAddress((void**)&order, g_mla_order_scratch));
    g_mla_order_ptr[dev].store(order, std::memory_order_release);       // every thread looks up the same address
  }
  cudaStream_t s = (cudaStream_t)stream;
  CUtensorMap tm;
  uint64_t dims[2] = {(uint64_t)kMlaD, (uint64_t)(num_pages * page_size)};
  uint64_t strides[1] = {(uint64_t)kMlaD};
  uint32_t box[2] = {128u, (uint32_t)kMlaBN};
  int rc = make_tensor_map(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, kv_cache, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  // every entry of order[0, batch) is rewritten by this launch, so nothing has to be cleared
  mla_order_kernel<<<(unsigned)((batch + 255) / 256), 256, 0, s>>>(cache_seqlens, order, (int)batch);
  TL_LAUNCH_CHECK("mla_order_kernel");
  MlaParams p;
  p.q = q; p.kv_scale = kv_scale; p.block_table = block_table; p.seqlens = cache_seqlens; p.order = order; p.out = out;
  p.batch = (int)batch; p.heads = (int)heads; p.page_size = (int)page_size; p.max_pages = (int)max_pages_per_seq;
  p.len_cap = mla_len_cap(max_pages_per_seq, num_pages, page_size); p.num_pages = (int)num_pages;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  // The host-visible status word is created by tl_b200_init (or by an earlier call of another entry
  // point); this path allocates nothing, so without it a kernel that gives up a wait cannot say so.
  p.status = device_status_word_if_created();
  if (q_dtype == TL_BF16) {
    auto kernel = mla_decode_fp8_kernel<__nv_bfloat16>;
    TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmem));
    kernel<<<(unsigned)(2 * batch), kMlaThreads, kMlaSmem, s>>>(tm, p);
  } else {
    auto kernel = mla_decode_fp8_kernel<__half>;
    TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmem));
    kernel<<<(unsigned)(2 * batch), kMlaThreads, kMlaSmem, s>>>(tm, p);
  }
  TL_LAUNCH_CHECK("mla_decode_fp8_kernel");
  return TL_B200_OK;
}
