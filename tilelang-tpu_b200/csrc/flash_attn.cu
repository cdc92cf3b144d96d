// FlashAttention forward on bshd tensors  O = softmax(scale * Q K^T + mask) V.
//
// tcgen05 kernel (bf16 / fp16, head_dim 64 or 128): one CTA owns 256 query rows of one
// (batch, head) as two 128-row "lanes".  Both lanes share every K/V tile that TMA brings into a
// 4-stage shared-memory ring, which halves L2 traffic per flop, and they ping-pong on the tensor
// core: while one lane's softmax warpgroup works on its scores, the MMA thread runs the other
// lane's S = Q K^T or O += P V.  S, P and O all live in tensor memory: every lane has two S
// buffers, so S runs two key tiles ahead of P V, and the softmax threads write P (16-bit) over the
// S buffer it came from, which the second MMA reads as its A operand straight from tensor memory.
// Softmax runs in the log2 domain with one thread per query row, fp32 statistics, and rescales O
// only when a row maximum grows by more than 2^8 (the stale maximum is exact algebraically and
// keeps P below 2^8, far inside bf16/fp32 range).
//
// Masking is expressed as a per-row key limit (keys [0, limit) are visible):
//   mode 0: limit = seq_kv                       (no mask)
//   mode 1: limit = q + 1                        (causal, tril; the check function of the demo)
//   mode 2: limit = ceil((q / bm + 1) * bm / bn) * bn, capped at seq_kv
//           (what the reference TPU program computes: a shortened KV loop and NO mask inside
//            the last tile, tpu_demo/flashattn/tpu_test_flashattn_bf16.py:116-118)
// Everything else (other dtypes, head dims, tiny shapes) runs a one-thread-per-row FMA kernel,
// which also serves the dense MLA decode program.
#include "sm100.cuh"
#include "mla_common.cuh"

#include <type_traits>

namespace tl {
using namespace sm100;

struct AttnParams {
  void* o;
  int batch, heads, seq_q, seq_kv, dim;
  float scale_log2;          // scale * log2(e)
  int mode, prog_bm, prog_bn;
  int in_fmt;
  int* status;
};

__device__ __forceinline__ int key_limit(int q, int mode, int bm, int bn, int seq_kv) {
  if (mode == 1) return min(q + 1, seq_kv);
  if (mode == 2) {
    long long blocks = ((long long)(q / bm + 1) * bm + bn - 1) / bn;
    long long lim = blocks * bn;
    return (int)(lim < seq_kv ? lim : seq_kv);
  }
  return seq_kv;
}

// =================================================================================
// tcgen05 kernel
// =================================================================================
constexpr int kFaBM = 128;       // rows per lane
constexpr int kFaBN = 64;        // keys per tile
constexpr int kFaStages = 4;     // K ring and V ring, each
constexpr int kFaThreads = 384;  // warp 0 TMA, warp 1 MMA, warp 2 TMEM alloc, warps 4-7 / 8-11 softmax

template <int HD> struct FaCfg {
  static constexpr int kSlabs = HD / 64;
  static constexpr int kQLane = kFaBM * HD * 2;           // one lane of Q
  static constexpr int kKV = kFaBN * HD * 2;              // one K or V tile
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = 2 * kQLane;
  static constexpr int kOffV = kOffK + kFaStages * kKV;
  static constexpr int kOffBar = kOffV + kFaStages * kKV;
  static constexpr int kSmemBytes = kOffBar + 256 + 1024;
  static constexpr int kTmemCols = 512;
  // lane l: two S buffers of 64 fp32 columns at l*128 + buf*64 (P, 16-bit, is written over the
  // first 32 columns of the S buffer it came from); O at 256 + l*HD
  static constexpr int kColS = 0;
  static constexpr int kColO = 256;
};

template <int HD, typename T>
__global__ void __launch_bounds__(kFaThreads, 1)
flash_attn_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  using Cfg = FaCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t sm_q = base + Cfg::kOffQ, sm_k = base + Cfg::kOffK, sm_v = base + Cfg::kOffV;
  const uint32_t bar0 = base + Cfg::kOffBar;
  // barrier map (8 bytes each)
  const uint32_t bar_q = bar0;
  const uint32_t bar_kfull = bar0 + 8;                       // [stages]
  const uint32_t bar_kempty = bar_kfull + 8 * kFaStages;
  const uint32_t bar_vfull = bar_kempty + 8 * kFaStages;
  const uint32_t bar_vempty = bar_vfull + 8 * kFaStages;
  const uint32_t bar_sfull = bar_vempty + 8 * kFaStages;     // [2 lanes][2 buffers]
  // P-ready and PV-retired barriers are per S buffer as well: a thread can only reach the next
  // tile of the same buffer after the previous phase has completed, so phases never overlap
  const uint32_t bar_pfull = bar_sfull + 32;                 // [2 lanes][2 buffers]
  const uint32_t bar_pvdone = bar_pfull + 32;                // [2 lanes][2 buffers]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + Cfg::kOffBar + 8 * (1 + 4 * kFaStages + 12));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane_id = threadIdx.x % 32;
  // longest rows first: with a causal mask the last query tiles have the most keys
  const int q_tiles = gridDim.x;
  const int q_tile = q_tiles - 1 - blockIdx.x;
  const int head = blockIdx.y, b = blockIdx.z;
  const int q0 = q_tile * 2 * kFaBM;

  // number of key tiles each lane needs
  int n_lane[2];
#pragma unroll
  for (int l = 0; l < 2; ++l) {
    const int first = q0 + l * kFaBM;
    if (first >= p.seq_q) { n_lane[l] = 0; continue; }
    const int last = min(first + kFaBM, p.seq_q) - 1;
    const int lim = key_limit(last, p.mode, p.prog_bm, p.prog_bn, p.seq_kv);   // limit grows with q
    n_lane[l] = (lim + kFaBN - 1) / kFaBN;
  }
  const int n_total = max(n_lane[0], n_lane[1]);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_q, 1);
    for (int s = 0; s < kFaStages; ++s) {
      mbar_init(bar_kfull + 8 * s, 1);
      mbar_init(bar_kempty + 8 * s, 1);
      mbar_init(bar_vfull + 8 * s, 1);
      mbar_init(bar_vempty + 8 * s, 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar_sfull + 8 * i, 1);
      mbar_init(bar_pfull + 8 * i, kFaBM / 32);  // one arrival per softmax warp of the lane
      mbar_init(bar_pvdone + 8 * i, 1);
    }
    mbar_fence_init();
    // Q and the first ring of K and V tiles are requested here, before the CTA meets for the tensor
    // memory allocation: fresh stages need no empty-wait, and only this thread has seen the barriers.
    mbar_expect_tx(bar_q, 2 * Cfg::kQLane);
#pragma unroll
    for (int l = 0; l < 2; ++l)
#pragma unroll
      for (int s = 0; s < Cfg::kSlabs; ++s)
        tma_load_4d(sm_q + l * Cfg::kQLane + s * (kFaBM * 128), &tm_q, bar_q, s * 64, head, q0 + l * kFaBM, b);
    for (int j = 0; j < min(n_total, kFaStages); ++j) {
      mbar_expect_tx(bar_kfull + 8 * j, Cfg::kKV);
#pragma unroll
      for (int s = 0; s < Cfg::kSlabs; ++s)
        tma_load_4d(sm_k + j * Cfg::kKV + s * (kFaBN * 128), &tm_k, bar_kfull + 8 * j, s * 64, head, j * kFaBN, b);
      mbar_expect_tx(bar_vfull + 8 * j, Cfg::kKV);
#pragma unroll
      for (int s = 0; s < Cfg::kSlabs; ++s)
        tma_load_4d(sm_v + j * Cfg::kKV + s * (kFaBN * 128), &tm_v, bar_vfull + 8 * j, s * 64, head, j * kFaBN, b);
    }
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      bool ok = true;
      for (int j = kFaStages; j < n_total && ok; ++j) {      // the first ring was requested during set-up
        const int st = j % kFaStages;
        const uint32_t ph = (j / kFaStages) & 1;
        if (!(ok = mbar_wait(bar_kempty + 8 * st, ph ^ 1, abort_flag))) break;
        mbar_expect_tx(bar_kfull + 8 * st, Cfg::kKV);
#pragma unroll
        for (int s = 0; s < Cfg::kSlabs; ++s)
          tma_load_4d(sm_k + st * Cfg::kKV + s * (kFaBN * 128), &tm_k, bar_kfull + 8 * st, s * 64, head, j * kFaBN, b);
        if (!(ok = mbar_wait(bar_vempty + 8 * st, ph ^ 1, abort_flag))) break;
        mbar_expect_tx(bar_vfull + 8 * st, Cfg::kKV);
#pragma unroll
        for (int s = 0; s < Cfg::kSlabs; ++s)
          tma_load_4d(sm_v + st * Cfg::kKV + s * (kFaBN * 128), &tm_v, bar_vfull + 8 * st, s * 64, head, j * kFaBN, b);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // Per lane S runs two key tiles ahead of P V, so a lane's softmax never waits for the tensor
    // core:  S(0) S(1) | PV(0) S(2) | PV(1) S(3) | ...   (lane 0 and lane 1 interleaved)
    if (elect_one() && n_total > 0) {
      const uint32_t idesc_s = make_idesc(p.in_fmt, p.in_fmt, false, false, kFaBM, kFaBN);   // S = Q K^T
      const uint32_t idesc_o = make_idesc(p.in_fmt, p.in_fmt, false, true, kFaBM, HD);       // O += P V
      bool ok = mbar_wait(bar_q, 0, abort_flag);

      // descriptors are built once; every MMA's operands are a constant byte offset further on
      const uint64_t q_desc = smem_desc_sw128(sm_q, 16, 1024), k_desc = smem_desc_sw128(sm_k, 16, 1024);
      const uint64_t v_desc = smem_desc_sw128(sm_v, kFaBN * 128, 1024);
      auto s_col = [&](int l, int j) { return tmem_base + Cfg::kColS + l * 128 + (j & 1) * kFaBN; };
      auto issue_s = [&](int l, int j) {       // S_l(j) = Q_l K_j^T, K dimension = head dim
        const uint64_t a0 = desc_at(q_desc, l * Cfg::kQLane), b0 = desc_at(k_desc, (j % kFaStages) * Cfg::kKV);
        const uint32_t d = s_col(l, j);
#pragma unroll
        for (int s = 0; s < Cfg::kSlabs; ++s)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_f16_ss(d, desc_at(a0, s * (kFaBM * 128) + kk * 32), desc_at(b0, s * (kFaBN * 128) + kk * 32), idesc_s,
                       (s | kk) ? 1u : 0u);
        mma_commit(bar_sfull + 8 * (2 * l + (j & 1)));
      };
      auto issue_pv = [&](int l, int j) {      // O_l += P_l(j) V_j; P comes from tensor memory
        const uint64_t b0 = desc_at(v_desc, (j % kFaStages) * Cfg::kKV);
        const uint32_t d = tmem_base + Cfg::kColO + l * HD, a = s_col(l, j);
#pragma unroll
        for (int kk = 0; kk < kFaBN / 16; ++kk)
          // A: 16 keys of P = 8 columns of packed 16-bit pairs.  B: V tile, 64-column slabs
          // (leading offset), 8-key groups 1 KB apart, 16 keys = 2 KB
          mma_f16_ts(d, a + kk * 8, desc_at(b0, kk * 2048), idesc_o, (j | kk) ? 1u : 0u);
        mma_commit(bar_pvdone + 8 * (2 * l + (j & 1)));
      };
      auto last_lane = [&](int j) { return j < n_lane[1] ? 1 : 0; };   // issue order is lane 0, lane 1
      auto issue_s_both = [&](int j) {         // S(j) of every lane that needs it, then free the K stage
        const int st = j % kFaStages;
        if (!(ok = mbar_wait(bar_kfull + 8 * st, (j / kFaStages) & 1, abort_flag))) return;
        tc_fence_after_sync();
        for (int l = 0; l < 2; ++l)
          if (j < n_lane[l]) issue_s(l, j);
        mma_commit(bar_kempty + 8 * st);
      };
      (void)last_lane;

      if (ok) issue_s_both(0);
      if (ok && n_total > 1) issue_s_both(1);
      for (int j = 0; j < n_total && ok; ++j) {
        const int st = j % kFaStages;
        const uint32_t ph = (j / kFaStages) & 1;
        if (!(ok = mbar_wait(bar_vfull + 8 * st, ph, abort_flag))) break;
        for (int l = 0; l < 2 && ok; ++l) {
          if (j < n_lane[l]) {
            if (!(ok = mbar_wait(bar_pfull + 8 * (2 * l + (j & 1)), (j >> 1) & 1, abort_flag))) break;
            tc_fence_after_sync();
            issue_pv(l, j);
          }
        }
        if (!ok) break;
        mma_commit(bar_vempty + 8 * st);
        if (j + 2 < n_total) issue_s_both(j + 2);     // reuses the S buffers whose P was just consumed
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- softmax + epilogue
    const int l = (warp - 4) / 4;                 // lane 0: warps 4-7, lane 1: warps 8-11
    const int quarter = warp % 4;
    const int r = quarter * 32 + lane_id;         // row inside the lane = TMEM lane
    const int q = q0 + l * kFaBM + r;
    const int n = n_lane[l];
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t t_s0 = tmem_base + Cfg::kColS + l * 128 + lane_off;
    const uint32_t t_o = tmem_base + Cfg::kColO + l * HD + lane_off;
    const int limit = q < p.seq_q ? key_limit(q, p.mode, p.prog_bm, p.prog_bn, p.seq_kv) : 0;
    float m_used = -INFINITY, row_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n; ++j) {
      const uint32_t t_s = t_s0 + (j & 1) * kFaBN;
      ok = mbar_wait(bar_sfull + 8 * (2 * l + (j & 1)), (j >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t sv[64];
      tmem_ld_32x64(t_s, sv);
      tmem_ld_wait();
      const int k0 = j * kFaBN;
      if (k0 + kFaBN > limit) {
#pragma unroll
        for (int c = 0; c < 64; ++c)
          if (k0 + c >= limit) sv[c] = 0xff800000u;          // -inf
      }
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 64; c += 4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) m4[e] = fmaxf(m4[e], __uint_as_float(sv[c + e]));
      }
      const float m_tile = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      const float m_new = fmaxf(m_used, m_tile * p.scale_log2);
      const bool grow = (j == 0) || (m_new - m_used > 8.0f);
      if (j > 0 && __any_sync(0xffffffffu, grow && m_used != -INFINITY)) {
        // O is rescaled only after the previous P V of this lane has retired
        ok = mbar_wait(bar_pvdone + 8 * (2 * l + ((j - 1) & 1)), ((j - 1) >> 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        const float alpha = (grow && m_used != -INFINITY) ? ex2_approx(m_used - m_new) : 1.0f;
        row_sum *= alpha;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
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
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[32];
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        const float p0 = ex2_approx(fmaf(__uint_as_float(sv[c]), p.scale_log2, -m_safe));
        const float p1 = ex2_approx(fmaf(__uint_as_float(sv[c + 1]), p.scale_log2, -m_safe));
        sum4[(c >> 1) & 3] += p0 + p1;
        if constexpr (std::is_same<T, __nv_bfloat16>::value) {
          __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          packed[c >> 1] = *reinterpret_cast<uint32_t*>(&h);
        } else {
          __half2 h = __floats2half2_rn(p0, p1);
          packed[c >> 1] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      row_sum += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      tmem_st_32x32(t_s, packed);        // P over the first half of its own S buffer
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane_id == 0) mbar_arrive(bar_pfull + 8 * (2 * l + (j & 1)));
    }
    // epilogue: O / row_sum -> global
    if (ok && n > 0) {
      ok = mbar_wait(bar_pvdone + 8 * (2 * l + ((n - 1) & 1)), ((n - 1) >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after_sync();
        const float inv = row_sum > 0.f ? 1.0f / row_sum : 0.f;
        // A thread owns a row, so storing straight from registers would touch 32 different lines per
        // instruction.  The warp's 32 rows are laid out in the lane's Q tile (no MMA reads it any more),
        // 16-byte units XOR-swizzled by the row, and stored whole rows at a time.
        constexpr int UPR = HD * 2 / 16;                     // 16-byte units per output row
        const uint32_t stg = sm_q + l * Cfg::kQLane + quarter * (32 * HD * 2);
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t ov[32];
          tmem_ld_32x32(t_o + c * 32, ov);
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              Vec16<T> two;      // only the first two elements are used
              two.e[0] = from_f32<T>(__uint_as_float(ov[8 * k + 2 * e]) * inv);
              two.e[1] = from_f32<T>(__uint_as_float(ov[8 * k + 2 * e + 1]) * inv);
              w[e] = two.raw.x;
            }
            const int u = c * 4 + k;
            st_shared_v4(stg + lane_id * (HD * 2) + ((u ^ (lane_id & (UPR - 1))) << 4), w[0], w[1], w[2], w[3]);
          }
        }
        __syncwarp();
        const int row0 = q0 + l * kFaBM + quarter * 32;      // first row of this warp
        char* out_w = reinterpret_cast<char*>(reinterpret_cast<T*>(p.o) + (((int64_t)b * p.seq_q + row0) * p.heads + head) * HD);
        const int64_t row_pitch = (int64_t)p.heads * HD * sizeof(T);
#pragma unroll
        for (int i = 0; i < UPR; ++i) {
          const int idx = i * 32 + lane_id, rr = idx / UPR, u = idx % UPR;
          const uint4 v = ld_shared_v4(stg + rr * (HD * 2) + ((u ^ (rr & (UPR - 1))) << 4));
          if (row0 + rr < p.seq_q) *reinterpret_cast<uint4*>(out_w + rr * row_pitch + u * 16) = v;
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
    if (threadIdx.x == 0 && p.status) *p.status = *abort_flag;
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// =================================================================================
// One-thread-per-row FMA kernel: any dtype, any head dim up to MAXD, optional second
// (positional) dot product, strided layouts.  Serves small / odd attention shapes and the
// dense MLA decode program.
// =================================================================================
struct RowAttnParams {
  const void *q, *q2, *k, *k2, *v;
  void* o;
  // element strides: q/q2/o indexed by (batch, query, head); k/k2/v by (batch, key, head)
  int64_t q_sb, q_sq, q_sh, q2_sb, q2_sq, q2_sh, o_sb, o_sq, o_sh;
  int64_t k_sb, k_sk, k_sh, k2_sb, k2_sk, k2_sh, v_sb, v_sk, v_sh;
  int batch, heads, seq_q, seq_kv, d1, d2, dv;
  float scale;
  int mode, prog_bm, prog_bn;
};

template <typename T, int MAXD>
__global__ void __launch_bounds__(128)
attn_rows_kernel(const RowAttnParams p) {
  const int64_t row = (int64_t)blockIdx.x * 128 + threadIdx.x;
  const int64_t total = (int64_t)p.batch * p.heads * p.seq_q;
  if (row >= total) return;
  const int q = (int)(row % p.seq_q);
  const int h = (int)((row / p.seq_q) % p.heads);
  const int b = (int)(row / ((int64_t)p.seq_q * p.heads));
  const T* qp = (const T*)p.q + b * p.q_sb + q * p.q_sq + h * p.q_sh;
  const T* q2p = p.q2 ? (const T*)p.q2 + b * p.q2_sb + q * p.q2_sq + h * p.q2_sh : nullptr;
  const T* kb = (const T*)p.k + b * p.k_sb + h * p.k_sh;
  const T* k2b = p.k2 ? (const T*)p.k2 + b * p.k2_sb + h * p.k2_sh : nullptr;
  const T* vb = (const T*)p.v + b * p.v_sb + h * p.v_sh;
  const int limit = key_limit(q, p.mode, p.prog_bm, p.prog_bn, p.seq_kv);
  float acc[MAXD];
#pragma unroll
  for (int d = 0; d < MAXD; ++d) acc[d] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int j = 0; j < limit; ++j) {
    float s = 0.f;
    const T* kr = kb + j * p.k_sk;
    for (int d = 0; d < p.d1; ++d) s = fmaf(to_f32(qp[d]), to_f32(kr[d]), s);
    if (q2p) {
      const T* k2r = k2b + j * p.k2_sk;
      for (int d = 0; d < p.d2; ++d) s = fmaf(to_f32(q2p[d]), to_f32(k2r[d]), s);
    }
    s *= p.scale;
    const float m_new = fmaxf(m, s);
    const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float pj = expf(s - m_new);
    l = l * alpha + pj;
    // the programs round P to the tile dtype before the second matmul
    const float pr = to_f32(from_f32<T>(pj));
    const T* vr = vb + j * p.v_sk;
#pragma unroll
    for (int d = 0; d < MAXD; ++d)
      if (d < p.dv) acc[d] = fmaf(pr, to_f32(vr[d]), acc[d] * alpha);
    m = m_new;
  }
  T* op = (T*)p.o + b * p.o_sb + q * p.o_sq + h * p.o_sh;
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int d = 0; d < MAXD; ++d)
    if (d < p.dv) op[d] = from_f32<T>(acc[d] * inv);
}

template <typename T>
static int launch_rows(const RowAttnParams& p, cudaStream_t s) {
  const int64_t total = (int64_t)p.batch * p.heads * p.seq_q;
  const unsigned grid = (unsigned)((total + 127) / 128);
  if (p.dv <= 32) attn_rows_kernel<T, 32><<<grid, 128, 0, s>>>(p);
  else if (p.dv <= 128) attn_rows_kernel<T, 128><<<grid, 128, 0, s>>>(p);
  else if (p.dv <= 512) attn_rows_kernel<T, 512><<<grid, 128, 0, s>>>(p);
  else return fail(TL_B200_EUNSUP, "attention: value dim %d exceeds 512", p.dv);
  TL_LAUNCH_CHECK("attn_rows_kernel");
  return TL_B200_OK;
}

static int launch_rows_dtype(const RowAttnParams& p, int dtype, cudaStream_t s) {
  switch (dtype) {
    case TL_F32: return launch_rows<float>(p, s);
    case TL_F16: return launch_rows<__half>(p, s);
    case TL_BF16: return launch_rows<__nv_bfloat16>(p, s);
    default: return fail(TL_B200_EINVAL, "attention: unsupported dtype %d", dtype);
  }
}

template <int HD, typename T>
static int launch_fa_tc(const void* q, const void* k, const void* v, void* o, int batch, int seq_q, int seq_kv,
                        int heads, float scale, int mode, int bm, int bn, cudaStream_t s) {
  const bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
  const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap tq, tk, tv;
  auto make = [&](CUtensorMap* m, const void* ptr, int seq, int box_rows) {
    uint64_t dims[4] = {(uint64_t)HD, (uint64_t)heads, (uint64_t)seq, (uint64_t)batch};
    uint64_t strides[3] = {(uint64_t)HD * 2, (uint64_t)heads * HD * 2, (uint64_t)seq * heads * HD * 2};
    uint32_t box[4] = {64u, 1u, (uint32_t)box_rows, 1u};
    return make_tensor_map(m, dt, 4, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  int rc;
  if ((rc = make(&tq, q, seq_q, kFaBM))) return rc;
  if ((rc = make(&tk, k, seq_kv, kFaBN))) return rc;
  if ((rc = make(&tv, v, seq_kv, kFaBN))) return rc;
  AttnParams p;
  p.o = o;
  p.batch = batch; p.heads = heads; p.seq_q = seq_q; p.seq_kv = seq_kv; p.dim = HD;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.mode = mode; p.prog_bm = bm > 0 ? bm : 1; p.prog_bn = bn > 0 ? bn : 1;
  p.in_fmt = is_bf16 ? kFmtBF16 : kFmtF16;
  p.status = device_status_word();
  auto kernel = flash_attn_tcgen05_kernel<HD, T>;
  TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FaCfg<HD>::kSmemBytes));
  dim3 grid((seq_q + 2 * kFaBM - 1) / (2 * kFaBM), heads, batch);
  kernel<<<grid, kFaThreads, FaCfg<HD>::kSmemBytes, s>>>(tq, tk, tv, p);
  TL_LAUNCH_CHECK("flash_attn_tcgen05_kernel");
  return TL_B200_OK;
}

}  // namespace tl

using namespace tl;

extern "C" int tl_b200_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, int64_t batch,
                                      int64_t seq_q, int64_t seq_kv, int64_t heads, int64_t dim, float scale,
                                      int mask_mode, int block_m, int block_n, int dtype, void* stream) {
  TL_REQUIRE(batch >= 0 && seq_q >= 0 && seq_kv >= 0 && heads >= 0 && dim >= 0, "flash_attn_fwd: negative size");
  TL_REQUIRE(mask_mode >= 0 && mask_mode <= 2, "flash_attn_fwd: mask_mode must be 0, 1 or 2");
  TL_REQUIRE(mask_mode != 2 || (block_m > 0 && block_n > 0), "flash_attn_fwd: block mask needs block sizes");
  TL_REQUIRE(mask_mode == 0 || seq_q == seq_kv, "flash_attn_fwd: a causal mask needs seq_q == seq_kv");
  if (batch == 0 || seq_q == 0 || heads == 0 || dim == 0) return TL_B200_OK;
  TL_REQUIRE(q && k && v && o, "flash_attn_fwd: null tensor pointer");
  TL_REQUIRE(seq_kv > 0, "flash_attn_fwd: no keys");
  TL_REQUIRE(batch < 65536 && heads < 65536 && seq_q < (1ll << 30) && seq_kv < (1ll << 30), "flash_attn_fwd: size too large");
  cudaStream_t s = (cudaStream_t)stream;
  const bool tc = (dtype == TL_BF16 || dtype == TL_F16) && (dim == 64 || dim == 128) && aligned16(q) && aligned16(k) &&
                  aligned16(v) && aligned16(o) && seq_q >= 64;
  if (tc) {
    const int B = (int)batch, SQ = (int)seq_q, SK = (int)seq_kv, H = (int)heads;
    if (dtype == TL_BF16) {
      if (dim == 128) return launch_fa_tc<128, __nv_bfloat16>(q, k, v, o, B, SQ, SK, H, scale, mask_mode, block_m, block_n, s);
      return launch_fa_tc<64, __nv_bfloat16>(q, k, v, o, B, SQ, SK, H, scale, mask_mode, block_m, block_n, s);
    }
    if (dim == 128) return launch_fa_tc<128, __half>(q, k, v, o, B, SQ, SK, H, scale, mask_mode, block_m, block_n, s);
    return launch_fa_tc<64, __half>(q, k, v, o, B, SQ, SK, H, scale, mask_mode, block_m, block_n, s);
  }
  RowAttnParams p{};
  p.q = q; p.k = k; p.v = v; p.o = o; p.q2 = nullptr; p.k2 = nullptr;
  const int64_t hd = heads * dim;
  p.q_sb = seq_q * hd; p.q_sq = hd; p.q_sh = dim;
  p.o_sb = seq_q * hd; p.o_sq = hd; p.o_sh = dim;
  p.k_sb = seq_kv * hd; p.k_sk = hd; p.k_sh = dim;
  p.v_sb = seq_kv * hd; p.v_sk = hd; p.v_sh = dim;
  p.batch = (int)batch; p.heads = (int)heads; p.seq_q = (int)seq_q; p.seq_kv = (int)seq_kv;
  p.d1 = (int)dim; p.d2 = 0; p.dv = (int)dim;
  p.scale = scale; p.mode = mask_mode; p.prog_bm = block_m > 0 ? block_m : 1; p.prog_bn = block_n > 0 ? block_n : 1;
  return launch_rows_dtype(p, dtype, s);
}

extern "C" int tl_b200_mla_decode_dense(const void* q, const void* q_pe, const void* kv, const void* k_pe, void* out,
                                        int64_t batch, int64_t heads, int64_t seq_kv, int64_t dim, int64_t pe_dim,
                                        float scale, int dtype, void* stream) {
  TL_REQUIRE(batch >= 0 && heads >= 0 && seq_kv >= 0 && dim >= 0 && pe_dim >= 0, "mla_decode_dense: negative size");
  if (batch == 0 || heads == 0 || dim == 0) return TL_B200_OK;
  TL_REQUIRE(q && kv && out && (pe_dim == 0 || (q_pe && k_pe)), "mla_decode_dense: null tensor pointer");
  TL_REQUIRE(seq_kv > 0, "mla_decode_dense: no keys");
  // DeepSeek shape (latent 512 + rope 64, up to 128 heads) in a 16-bit type: the tcgen05 kernel, with the identity
  // as its page table; Q / Q_pe and KV / K_pe stay separate tensors
  if ((dtype == TL_BF16 || dtype == TL_F16) && dim == 512 && pe_dim == 64 && heads <= 128 && aligned16(q) && aligned16(q_pe) &&
      aligned16(kv) && aligned16(k_pe) && aligned16(out) && batch * seq_kv < (1ll << 31))
    return mla_f16_launch(q, q_pe, kv, k_pe, nullptr, nullptr, out, batch, 1, heads, 1, batch * seq_kv, 0, 0, 0, seq_kv,
                          scale, dtype, (cudaStream_t)stream);
  RowAttnParams p{};
  p.q = q; p.q2 = pe_dim ? q_pe : nullptr; p.k = kv; p.k2 = pe_dim ? k_pe : nullptr; p.v = kv; p.o = out;
  // Q[b,h,1,dim], Q_pe[b,h,1,pe], KV[b,s,1,dim], K_pe[b,s,1,pe], Out[b,h,1,dim]; one shared kv head
  p.q_sb = heads * dim; p.q_sq = 0; p.q_sh = dim;
  p.q2_sb = heads * pe_dim; p.q2_sq = 0; p.q2_sh = pe_dim;
  p.o_sb = heads * dim; p.o_sq = 0; p.o_sh = dim;
  p.k_sb = seq_kv * dim; p.k_sk = dim; p.k_sh = 0;
  p.k2_sb = seq_kv * pe_dim; p.k2_sk = pe_dim; p.k2_sh = 0;
  p.v_sb = seq_kv * dim; p.v_sk = dim; p.v_sh = 0;
  p.batch = (int)batch; p.heads = (int)heads; p.seq_q = 1; p.seq_kv = (int)seq_kv;
  p.d1 = (int)dim; p.d2 = (int)pe_dim; p.dv = (int)dim;
  p.scale = scale; p.mode = 0; p.prog_bm = 1; p.prog_bn = 1;
  return launch_rows_dtype(p, dtype, (cudaStream_t)stream);
}
