// FP8 (e4m3) GEMM with 128-granular fp32 scales:
//   C[m,n] = sum over 128-wide K blocks kb of  sa[m,kb] * sb[n/128,kb] * (A8[m,kb] . B8[n,kb])
// A8 [M,K] row-major e4m3 with one scale per row per K block, B8 [N,K] row-major e4m3 with one
// scale per 128x128 block, C bf16 or fp32.  Semantics of the block-scaled program
// examples/deepseek_deepgemm/example_deepgemm_fp8_2xAcc.py:66-81: the tensor core produces an
// fp32 partial product per K block, which is "promoted" into a separate fp32 accumulator with
// the product of the two scales.
//
// Persistent warp-specialised kernel: TMA ring (6 stages of 128x128 A and B bytes, 128-byte
// swizzle) -> tcgen05.mma kind::f8f6f4 into one of four partial accumulators in tensor memory ->
// eight promotion warps (64 columns of 32 rows each) pull the partial with tcgen05.ld and do the scaled
// accumulation in registers while the tensor core already fills the next partials.  The promotion is a
// dependent chain per warp (wait for the partial, load, hand the buffer back, multiply in): a warp fetches its
// share with a single load, one round trip to tensor memory per K block.
//
// PAIR = true runs the same pipeline on CTA pairs (two CTAs of a cluster on neighbouring SMs, cta_group::2): a tile
// is 256 x 128, each CTA owns 128 of its rows (its own partials, promotion warps and output rows) and loads only 64
// of the 128 B rows; the MMAs (M = 256, N = 128), issued by the even CTA, read B from both shared memories.  A
// 128 x 128 e4m3 tile reads 128 bytes of shared memory per clock, all there is; the pair needs 96.
#include "sm100.cuh"

namespace tl {
using namespace sm100;

constexpr int kF8BM = 128, kF8BN = 128, kF8BK = 128;
constexpr int kF8Stages = 6;           // one CTA per tile; pairs: 8 stages of 24 KB
constexpr int kF8Cols = 64;           // columns of a partial per promotion warp (32: sixteen warps, measured 4% slower at the C4 shape, on one CTA and on pairs)
constexpr int kF8PromoWarps = 4 * (kF8BN / kF8Cols);        // 8: four lane quarters x two column groups
constexpr int kF8PromoWarp0 = 4;      // warp 0 TMEM alloc + TMA, warp 1 MMA, warps 4.. promotion/epilogue
constexpr int kF8Threads = (kF8PromoWarp0 + kF8PromoWarps) * 32;
constexpr int kF8Acc = 4;             // partial accumulators in tensor memory (4 x 128 columns)
constexpr int kF8TmemCols = kF8Acc * kF8BN;

__device__ __forceinline__ bool aligned16_dev(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct F8Params {
  void* c;
  const float* sa;      // [M, K/128]
  const float* sb;      // [ceil(N/128), K/128]
  int m, n, k, kblocks;
  int tiles_m, tiles_n;
  int* status;
};

template <bool PAIR> struct F8Cfg {
  static constexpr int kStages = PAIR ? 8 : kF8Stages;
  static constexpr int kBRows = PAIR ? kF8BN / 2 : kF8BN;       // B rows one CTA loads
  static constexpr int kStageA = kF8BM * kF8BK;
  static constexpr int kStageB = kBRows * kF8BK;
  static constexpr int kTileM = PAIR ? 2 * kF8BM : kF8BM;       // rows of C per tile
  static constexpr int kSmem = kStages * (kStageA + kStageB) + 1024 + 256;
};

template <typename TOut, bool PAIR>
__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_blockscale_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                           const F8Params p) {
  using Cfg = F8Cfg<PAIR>;
  constexpr int STAGES = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t smem_a = base;
  const uint32_t smem_b = base + STAGES * Cfg::kStageA;
  uint8_t* tail = base_ptr + STAGES * (Cfg::kStageA + Cfg::kStageB);
  const uint32_t bar_full = smem_u32(tail);
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES;
  const uint32_t bar_tempty = bar_tfull + 8 * kF8Acc;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8 * (2 * STAGES + 2 * kF8Acc));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;          // pairs: rank 0 issues the MMAs
  const int unit = PAIR ? blockIdx.x / 2 : blockIdx.x;          // tiles are dealt to CTAs, or to pairs
  const int units = PAIR ? gridDim.x / 2 : gridDim.x;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < kF8Acc; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      // one arrival per promotion warp; pairs: the even CTA's barrier collects both CTAs' warps
      mbar_init(bar_tempty + 8 * a, PAIR ? 2 * kF8PromoWarps : kF8PromoWarps);
    }
    mbar_fence_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
  }
  if (warp == 0) {
    if constexpr (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_slot), kF8TmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), kF8TmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if constexpr (PAIR) cluster_sync_all();     // both CTAs' barriers and tensor memory exist before anything is signalled
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // tiles walk 8 row-blocks per column-block so resident tiles share operands in L2
  auto coords = [&](int tile, int& tm, int& tn) {
    constexpr int G = 8;
    const int per_group = G * p.tiles_n;
    const int group = tile / per_group;
    const int first_m = group * G;
    const int rows = min(G, p.tiles_m - first_m);
    const int in_group = tile - group * per_group;
    tm = first_m + in_group % rows;
    tn = in_group / rows;
  };

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = unit; tile < num_tiles && ok; tile += units) {
        int tm, tn;
        coords(tile, tm, tn);
        const int a_row = tm * Cfg::kTileM + (int)rank * kF8BM;
        const int b_row = tn * kF8BN + (int)rank * Cfg::kBRows;
        for (int kb = 0; kb < p.kblocks; ++kb) {
          if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag))) break;
          if constexpr (PAIR) {
            // the even CTA's barrier counts the bytes of both CTAs' loads
            if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * (Cfg::kStageA + Cfg::kStageB));
            const uint32_t full = map_to_cta(bar_full + 8 * stage, 0);
            tma_load_2d_pair(smem_a + stage * Cfg::kStageA, &tm_a, full, kb * kF8BK, a_row);
            tma_load_2d_pair(smem_b + stage * Cfg::kStageB, &tm_b, full, kb * kF8BK, b_row);
          } else {
            const uint32_t full = bar_full + 8 * stage;
            mbar_expect_tx(full, Cfg::kStageA + Cfg::kStageB);
            tma_load_2d(smem_a + stage * Cfg::kStageA, &tm_a, full, kb * kF8BK, a_row);
            tma_load_2d(smem_b + stage * Cfg::kStageB, &tm_b, full, kb * kF8BK, b_row);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1 && rank == 0) {
    if (elect_one()) {
      const uint32_t idesc = make_idesc(kFmtE4M3, kFmtE4M3, false, false, Cfg::kTileM, kF8BN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t it = 0;                       // K blocks issued so far: selects the partial accumulator
      bool ok = true;
      for (int tile = unit; tile < num_tiles && ok; tile += units) {
        for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
          const uint32_t buf = it % kF8Acc;
          if (!(ok = mbar_wait(bar_tempty + 8 * buf, ((it / kF8Acc) & 1) ^ 1, abort_flag))) break;
          if (!(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag))) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_a + stage * Cfg::kStageA;
          const uint32_t b_addr = smem_b + stage * Cfg::kStageB;
#pragma unroll
          for (int kk = 0; kk < kF8BK / 32; ++kk) {      // K = 32 per instruction for 8-bit operands
            const uint64_t a_desc = smem_desc_sw128(a_addr + kk * 32, 16, 1024);
            const uint64_t b_desc = smem_desc_sw128(b_addr + kk * 32, 16, 1024);
            if constexpr (PAIR) mma_f8_ss_pair(tmem_base + buf * kF8BN, a_desc, b_desc, idesc, kk ? 1u : 0u);
            else mma_f8_ss(tmem_base + buf * kF8BN, a_desc, b_desc, idesc, kk ? 1u : 0u);
          }
          if constexpr (PAIR) {                          // the stage and the partial are signalled in both CTAs
            mma_commit_pair(bar_empty + 8 * stage);
            mma_commit_pair(map_to_cta(bar_empty + 8 * stage, 1));
            mma_commit_pair(bar_tfull + 8 * buf);
            mma_commit_pair(map_to_cta(bar_tfull + 8 * buf, 1));
          } else {
            mma_commit(bar_empty + 8 * stage);
            mma_commit(bar_tfull + 8 * buf);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp >= kF8PromoWarp0) {
    const int wg = (warp - kF8PromoWarp0) / 4;   // column group
    const int quarter = warp % 4;             // the tensor-memory lanes a warp may touch follow from warp % 4
    const int r = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    TOut* c = reinterpret_cast<TOut*>(p.c);
    const bool vec_ok = ((int64_t)p.n * sizeof(TOut)) % 16 == 0 && (reinterpret_cast<uintptr_t>(p.c) & 15u) == 0;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = unit; tile < num_tiles && ok; tile += units) {
      int tm, tn;
      coords(tile, tm, tn);
      const int row = tm * Cfg::kTileM + (int)rank * kF8BM + r;
      const float* sa_row = p.sa + (int64_t)(row < p.m ? row : 0) * p.kblocks;
      const float* sb_row = p.sb + (int64_t)tn * p.kblocks;
      float2 acc2[kF8Cols / 2];                // fp32 accumulators, updated two at a time
#pragma unroll
      for (int j = 0; j < kF8Cols / 2; ++j) acc2[j] = make_float2(0.f, 0.f);
      float* acc = reinterpret_cast<float*>(acc2);
      // Per K block: wait for the partial, ONE 64-column load (a single round trip to tensor memory), hand the
      // buffer back to the tensor core, then multiply the partial in.  The scales of a row are fetched four K
      // blocks at a time (16-byte loads, one group ahead): every thread reads its own row of `sa`, so each scalar
      // load would cost a warp 32 sectors.
      const bool quads = (p.kblocks % 4 == 0) && aligned16_dev(p.sa) && aligned16_dev(p.sb);
      auto scales_at = [&](int kb) {
        float4 a, b;
        if (quads) {
          a = __ldg(reinterpret_cast<const float4*>(sa_row + kb));
          b = __ldg(reinterpret_cast<const float4*>(sb_row + kb));
        } else {
          const int n = p.kblocks - kb;
          a = make_float4(__ldg(sa_row + kb), n > 1 ? __ldg(sa_row + kb + 1) : 0.f, n > 2 ? __ldg(sa_row + kb + 2) : 0.f,
                          n > 3 ? __ldg(sa_row + kb + 3) : 0.f);
          b = make_float4(__ldg(sb_row + kb), n > 1 ? __ldg(sb_row + kb + 1) : 0.f, n > 2 ? __ldg(sb_row + kb + 2) : 0.f,
                          n > 3 ? __ldg(sb_row + kb + 3) : 0.f);
        }
        return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w);
      };
      float4 sc_next = scales_at(0);
      for (int kb0 = 0; kb0 < p.kblocks && ok; kb0 += 4) {
        const float4 sc = sc_next;
        if (kb0 + 4 < p.kblocks) sc_next = scales_at(kb0 + 4);
        const float sc_of[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (kb0 + q >= p.kblocks) break;
          const uint32_t buf = it % kF8Acc;
          ok = mbar_wait(bar_tfull + 8 * buf, (it / kF8Acc) & 1, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          uint32_t v[kF8Cols];
          if constexpr (kF8Cols == 64) tmem_ld_32x64(tmem_base + buf * kF8BN + wg * kF8Cols + lane_off, reinterpret_cast<uint32_t(&)[64]>(v));
          else tmem_ld_32x32(tmem_base + buf * kF8BN + wg * kF8Cols + lane_off, reinterpret_cast<uint32_t(&)[32]>(v));
          tmem_ld_wait_for(v);
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * buf, 0));
            else mbar_arrive(bar_tempty + 8 * buf);
          }
          const float2 sc2 = make_float2(sc_of[q], sc_of[q]);
#pragma unroll
          for (int j = 0; j < kF8Cols; j += 2)
            acc2[j / 2] = fma2(make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), sc2, acc2[j / 2]);
          ++it;
        }
      }
      if (!ok) break;
      const int col0 = tn * kF8BN + wg * kF8Cols;
      if (row < p.m && col0 < p.n) {
        TOut* dst = c + (int64_t)row * p.n + col0;
        const int valid = min(kF8Cols, p.n - col0);
        if (vec_ok && valid == kF8Cols) {
          if constexpr (sizeof(TOut) == 4) {
#pragma unroll
            for (int j = 0; j < kF8Cols; j += 4)
              *reinterpret_cast<float4*>(dst + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < kF8Cols; j += 8) {
              Vec16<TOut> o;
#pragma unroll
              for (int e = 0; e < 8; ++e) o.e[e] = from_f32<TOut>(acc[j + e]);
              *reinterpret_cast<uint4*>(dst + j) = o.raw;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < kF8Cols; ++j)
            if (j < valid) dst[j] = from_f32<TOut>(acc[j]);
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
  if constexpr (PAIR) {
    // neither CTA may leave (or free tensor memory) while the other can still read its shared memory or signal its barriers
    tc_fence_before_sync();
    cluster_sync_all();
  }
  if (warp == 2) {
    tc_fence_after_sync();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, kF8TmemCols);
    else tmem_dealloc(tmem_base, kF8TmemCols);
  }
}

template <typename TOut, bool PAIR>
static int launch_f8(const CUtensorMap& ta, const CUtensorMap& tb, const F8Params& p, cudaStream_t s) {
  auto kernel = gemm_fp8_blockscale_kernel<TOut, PAIR>;
  constexpr int smem = F8Cfg<PAIR>::kSmem;
  TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const int tiles = p.tiles_m * p.tiles_n;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  if (PAIR) {
    const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
    cfg.gridDim = dim3(2 * pairs);
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  } else {
    cfg.gridDim = dim3(tiles < sm_count() ? tiles : sm_count());
  }
  cfg.blockDim = dim3(kF8Threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  TL_CUDA(cudaLaunchKernelEx(&cfg, kernel, ta, tb, p));
  TL_LAUNCH_CHECK("gemm_fp8_blockscale_kernel");
  return TL_B200_OK;
}

}  // namespace tl

using namespace tl;

extern "C" int tl_b200_gemm_fp8_blockscale(const void* a, const void* b, const float* scales_a, const float* scales_b,
                                           void* c, int64_t m, int64_t n, int64_t k, int out_dtype, void* stream) {
  TL_REQUIRE(m >= 0 && n >= 0 && k >= 0, "gemm_fp8_blockscale: negative size");
  TL_REQUIRE(m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31), "gemm_fp8_blockscale: dimension exceeds 2^31");
  if (m == 0 || n == 0) return TL_B200_OK;
  TL_REQUIRE(a && b && c && scales_a && scales_b, "gemm_fp8_blockscale: null tensor pointer");
  TL_REQUIRE(k > 0 && k % 128 == 0, "gemm_fp8_blockscale: K (%lld) must be a positive multiple of 128 (one scale "
                                    "per 128-wide K block)", (long long)k);
  TL_REQUIRE(out_dtype == TL_BF16 || out_dtype == TL_F32, "gemm_fp8_blockscale: output must be bfloat16 or float32");
  TL_REQUIRE(aligned16(a) && aligned16(b), "gemm_fp8_blockscale: A and B must be 16-byte aligned");
  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {(uint64_t)k, (uint64_t)m};
    uint64_t strides[1] = {(uint64_t)k};
    uint32_t box[2] = {(uint32_t)kF8BK, (uint32_t)kF8BM};
    int rc = make_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  // CTA pairs (256 x 128 tiles) whenever every pair of SMs gets a tile
  const int64_t pair_tiles = ((m + 2 * kF8BM - 1) / (2 * kF8BM)) * ((n + kF8BN - 1) / kF8BN);
  const bool pair = pair_tiles >= sm_count() / 2;
  {
    uint64_t dims[2] = {(uint64_t)k, (uint64_t)n};
    uint64_t strides[1] = {(uint64_t)k};
    uint32_t box[2] = {(uint32_t)kF8BK, (uint32_t)(pair ? F8Cfg<true>::kBRows : kF8BN)};
    int rc = make_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  F8Params p;
  p.c = c; p.sa = scales_a; p.sb = scales_b;
  p.m = (int)m; p.n = (int)n; p.k = (int)k; p.kblocks = (int)(k / 128);
  const int tile_m = pair ? 2 * kF8BM : kF8BM;
  p.tiles_m = (int)((m + tile_m - 1) / tile_m);
  p.tiles_n = (int)((n + kF8BN - 1) / kF8BN);
  p.status = device_status_word();
  cudaStream_t s = (cudaStream_t)stream;
  if (pair) {
    if (out_dtype == TL_F32) return launch_f8<float, true>(ta, tb, p, s);
    return launch_f8<__nv_bfloat16, true>(ta, tb, p, s);
  }
  if (out_dtype == TL_F32) return launch_f8<float, false>(ta, tb, p, s);
  return launch_f8<__nv_bfloat16, false>(ta, tb, p, s);
}
