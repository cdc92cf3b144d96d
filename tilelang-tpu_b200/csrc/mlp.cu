// Front half of the gated MLP as one kernel:
//
//   out[M,N] = silu(x Wg^T) * (x Wu^T)        x [M,K], Wg and Wu [N,K] row-major, 16-bit
//
// The reference's MLP program (tpu_demo/ppl/mlp/mlp_bf16.py:10-139) runs, per tile, a gate GEMM and
// an up GEMM that round their results to the 16-bit type, SiLU and the product in fp32, one more
// rounding, and then the down GEMM.  Here the two GEMMs share the A tiles and the SiLU-product is
// the epilogue of the pair, so the two [M,N] intermediates and the separate SwiGLU pass over them
// (2 reads + 1 write of M*N elements) never touch HBM.  The roundings are kept where the program
// has them: the epilogue rounds both accumulators to the 16-bit type before the fp32 SiLU-product.
// The down projection is a plain GEMM (tl_b200_gemm with trans_b).
//
// tcgen05 kernel: persistent, warp-specialised like the GEMM of gemm.cu.  A stage of the TMA ring
// holds a 128x64 tile of x and, one behind the other, 128x64 tiles of Wg and Wu (48 KB, 4 stages): together they
// are ONE K-major B operand of 256 rows, so one thread issues one 128x256x16 MMA per K step and the gate and up
// accumulators come out side by side in tensor memory (256 columns), double-buffered (512 columns) so that the
// four epilogue warps work on one pair while the next tile's main loop runs.
//
// PAIR = true: the same on CTA pairs (cta_group::2, tiles of 256 rows x 128 output columns).  The B operand of the
// pair's MMA (M = 256, N = 256) takes its first 128 rows from the even CTA and the other 128 from the odd one, so
// the even CTA loads only the Wg tile and the odd CTA only the Wu tile (32 KB per stage and CTA, 6 stages).
#include "sm100.cuh"

#include <type_traits>

namespace tl {
using namespace sm100;

constexpr int kMlpBM = 128, kMlpBN = 128, kMlpBK = 64, kMlpStages = 4, kMlpThreads = 256;
constexpr int kMlpStageA = kMlpBM * kMlpBK * 2, kMlpStageB = kMlpBN * kMlpBK * 2;
constexpr int kMlpStage = kMlpStageA + 2 * kMlpStageB;

struct MlpParams {
  void* out;
  int m, n, k, tiles_m, tiles_n;
  int in_fmt;
  int* status;
};

// Same grouped rasterisation as the GEMM: 8 row blocks per column block.
__device__ __forceinline__ void mlp_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int G = 8;
  const int per_group = G * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * G;
  const int rows = min(G, tiles_m - first_m);
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % rows;
  tn = in_group / rows;
}

template <typename T> __device__ __forceinline__ float round_through(float v) { return to_f32(from_f32<T>(v)); }

template <bool PAIR> struct MlpCfg {
  static constexpr int kStages = PAIR ? 6 : kMlpStages;
  static constexpr int kStage = PAIR ? kMlpStageA + kMlpStageB : kMlpStage;   // a pair's CTA holds x and ONE weight tile
  static constexpr int kTileM = PAIR ? 2 * kMlpBM : kMlpBM;
  static constexpr int kSmem = kStages * kStage + 1024 + 256;
};

template <typename T, bool PAIR>
__global__ void __launch_bounds__(kMlpThreads, 1)
mlp_gate_up_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_g,
                           const __grid_constant__ CUtensorMap tm_u, const MlpParams p) {
  using Cfg = MlpCfg<PAIR>;
  constexpr int STAGES = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;          // swizzle atoms need 1024-byte alignment
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  uint8_t* tail = base_ptr + STAGES * Cfg::kStage;
  const uint32_t bar_full = smem_u32(tail);                   // full[S], empty[S], tfull[2], tempty[2]
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int num_kb = (p.k + kMlpBK - 1) / kMlpBK;
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
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, PAIR ? 8 : 4);      // one arrival per epilogue warp (pairs: of both CTAs)
    }
    mbar_fence_init();
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_g);
    prefetch_tensormap(&tm_u);
  }
  if (warp == 2) {
    if constexpr (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_slot), 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), 512);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if constexpr (PAIR) cluster_sync_all();     // both CTAs' barriers and tensor memory exist before anything is signalled
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = unit; tile < num_tiles && ok; tile += units) {
        int tm, tn;
        mlp_tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int x_row = tm * Cfg::kTileM + (int)rank * kMlpBM;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag))) break;
          const uint32_t st = base + stage * Cfg::kStage;
          if constexpr (PAIR) {
            // the even CTA's barrier counts the bytes of both CTAs' loads; the even CTA brings Wg, the odd one Wu
            if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * Cfg::kStage);
            const uint32_t full = map_to_cta(bar_full + 8 * stage, 0);
            tma_load_2d_pair(st, &tm_x, full, kb * kMlpBK, x_row);
            tma_load_2d_pair(st + kMlpStageA, rank == 0 ? &tm_g : &tm_u, full, kb * kMlpBK, tn * kMlpBN);
          } else {
            const uint32_t full = bar_full + 8 * stage;
            mbar_expect_tx(full, Cfg::kStage);
            tma_load_2d(st, &tm_x, full, kb * kMlpBK, x_row);
            tma_load_2d(st + kMlpStageA, &tm_g, full, kb * kMlpBK, tn * kMlpBN);
            tma_load_2d(st + kMlpStageA + kMlpStageB, &tm_u, full, kb * kMlpBK, tn * kMlpBN);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1 && rank == 0) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      // N = 256: gate columns [0,128), up columns [128,256) of the accumulator
      const uint32_t idesc = make_idesc(p.in_fmt, p.in_fmt, false, false, Cfg::kTileM, 2 * kMlpBN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = unit; tile < num_tiles && ok; tile += units, ++local) {
        const int acc = local & 1;
        if (!(ok = mbar_wait(bar_tempty + 8 * acc, ((local >> 1) & 1) ^ 1, abort_flag))) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * 256;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag))) break;
          tc_fence_after_sync();
          const uint32_t st = base + stage * Cfg::kStage;
#pragma unroll
          for (int kk = 0; kk < kMlpBK / 16; ++kk) {
            // K-major operands: 8-row groups 1024 B apart, a K step of 16 elements is 32 B.  B is the Wg tile followed
            // by the Wu tile (one CTA: 256 rows in this shared memory; pairs: 128 rows in each CTA's)
            const uint64_t a_desc = smem_desc_sw128(st + kk * 32, 16, 1024);
            const uint64_t b_desc = smem_desc_sw128(st + kMlpStageA + kk * 32, 16, 1024);
            if constexpr (PAIR) mma_f16_ss_pair(d_tmem, a_desc, b_desc, idesc, (kb | kk) != 0 ? 1u : 0u);
            else mma_f16_ss(d_tmem, a_desc, b_desc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          if constexpr (PAIR) {                         // the stage is free in both CTAs once these MMAs retire
            mma_commit_pair(bar_empty + 8 * stage);
            mma_commit_pair(map_to_cta(bar_empty + 8 * stage, 1));
          } else {
            mma_commit(bar_empty + 8 * stage);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) {                                       // both accumulators complete
          if constexpr (PAIR) {
            mma_commit_pair(bar_tfull + 8 * acc);
            mma_commit_pair(map_to_cta(bar_tfull + 8 * acc, 1));
          } else {
            mma_commit(bar_tfull + 8 * acc);
          }
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue: SiLU(gate) * up
    const int quarter = warp - 4;                     // == warp % 4: TMEM lanes [32q, 32q+32)
    T* out = reinterpret_cast<T*>(p.out);
    const bool vec_ok = ((int64_t)p.n * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15u) == 0;
    int local = 0;
    bool ok = true;
    for (int tile = unit; tile < num_tiles && ok; tile += units, ++local) {
      int tm, tn;
      mlp_tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      const int acc = local & 1;
      ok = mbar_wait(bar_tfull + 8 * acc, (local >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);             // keep the warp together for the aligned loads
      if (!ok) break;
      tc_fence_after_sync();
      const int row = tm * Cfg::kTileM + (int)rank * kMlpBM + quarter * 32 + lane;
      const uint32_t t_gate = tmem_base + acc * 256 + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int cchunk = 0; cchunk < kMlpBN / 32; ++cchunk) {
        uint32_t g[32], u[32];
        tmem_ld_32x32(t_gate + cchunk * 32, g);
        tmem_ld_32x32(t_gate + 128 + cchunk * 32, u);
        tmem_ld_wait();
        const int col = tn * kMlpBN + cchunk * 32;
        if (row < p.m && col < p.n) {
          T* dst = out + (int64_t)row * p.n + col;
          const int valid = min(32, p.n - col);
          float r[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            // the program's gate and up GEMMs deliver 16-bit tiles; SiLU and the product run in fp32
            const float gv = round_through<T>(__uint_as_float(g[j])), uv = round_through<T>(__uint_as_float(u[j]));
            float th;                                       // same expression as the SwiGLU kernel: bit-identical results
            asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(0.5f * gv));
            r[j] = gv < -17.0f ? 0.0f * uv : uv * (0.5f * gv * (1.0f + th));
          }
          if (vec_ok && valid == 32) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              Vec16<T> v;
#pragma unroll
              for (int e = 0; e < 8; ++e) v.e[e] = from_f32<T>(r[j + e]);
              *reinterpret_cast<uint4*>(dst + j) = v.raw;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) dst[j] = from_f32<T>(r[j]);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * acc, 0));
        else mbar_arrive(bar_tempty + 8 * acc);
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(20000);      // let copies and MMAs in flight land
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
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
}

// =================================================================================
// Plain FMA kernel: fp32 / fp16 / bf16, any size and alignment.
// =================================================================================
template <typename T>
__global__ void __launch_bounds__(256)
mlp_gate_up_simt_kernel(const T* __restrict__ x, const T* __restrict__ wg, const T* __restrict__ wu, T* __restrict__ out,
                        int m, int n, int k) {
  constexpr int TS = 64, KT = 16;
  __shared__ float sx[KT][TS + 1], sg[KT][TS + 1], su[KT][TS + 1];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int m0 = blockIdx.y * TS, n0 = blockIdx.x * TS;
  float ag[4][4] = {}, au[4][4] = {};
  for (int k0 = 0; k0 < k; k0 += KT) {
    for (int i = threadIdx.x; i < TS * KT; i += 256) {
      const int r = i / KT, kk = i % KT, gk = k0 + kk;
      sx[kk][r] = (m0 + r < m && gk < k) ? to_f32(x[(int64_t)(m0 + r) * k + gk]) : 0.f;
      sg[kk][r] = (n0 + r < n && gk < k) ? to_f32(wg[(int64_t)(n0 + r) * k + gk]) : 0.f;
      su[kk][r] = (n0 + r < n && gk < k) ? to_f32(wu[(int64_t)(n0 + r) * k + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KT; ++kk) {
      float xv[4], gv[4], uv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { xv[i] = sx[kk][ty * 4 + i]; gv[i] = sg[kk][tx * 4 + i]; uv[i] = su[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          ag[i][j] = fmaf(xv[i], gv[j], ag[i][j]);
          au[i][j] = fmaf(xv[i], uv[j], au[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
      if (gm < m && gn < n) {
        const float gv = round_through<T>(ag[i][j]), uv = round_through<T>(au[i][j]);
        out[(int64_t)gm * n + gn] = from_f32<T>(uv * (gv / (1.0f + expf(-gv))));
      }
    }
}

template <typename T>
static int mlp_gate_up_tc(const void* x, const void* wg, const void* wu, void* out, int m, int n, int k, cudaStream_t s) {
  const bool is_bf16 = std::is_same<T, __nv_bfloat16>::value;
  const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap tx, tg, tu;
  auto make = [&](CUtensorMap* map, const void* ptr, int rows, int box_rows) {
    uint64_t dims[2] = {(uint64_t)k, (uint64_t)rows};
    uint64_t strides[1] = {(uint64_t)k * 2};
    uint32_t box[2] = {(uint32_t)kMlpBK, (uint32_t)box_rows};
    return make_tensor_map(map, dt, 2, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  int rc;
  if ((rc = make(&tx, x, m, kMlpBM))) return rc;
  if ((rc = make(&tg, wg, n, kMlpBN))) return rc;
  if ((rc = make(&tu, wu, n, kMlpBN))) return rc;
  MlpParams p;
  p.out = out;
  p.m = m; p.n = n; p.k = k;
  p.tiles_n = (n + kMlpBN - 1) / kMlpBN;
  p.in_fmt = is_bf16 ? kFmtBF16 : kFmtF16;
  p.status = device_status_word();
  // CTA pairs (tiles of 256 rows) whenever every pair of SMs gets a tile
  const int64_t pair_tiles = (int64_t)((m + 2 * kMlpBM - 1) / (2 * kMlpBM)) * p.tiles_n;
  const bool pair = pair_tiles >= sm_count() / 2;
  const int tile_m = pair ? 2 * kMlpBM : kMlpBM;
  p.tiles_m = (m + tile_m - 1) / tile_m;
  const int tiles = p.tiles_m * p.tiles_n;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  cfg.blockDim = dim3(kMlpThreads);
  cfg.stream = s;
  if (pair) {
    auto kernel = mlp_gate_up_tcgen05_kernel<T, true>;
    TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MlpCfg<true>::kSmem));
    const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
    cfg.gridDim = dim3(2 * pairs);
    cfg.dynamicSmemBytes = MlpCfg<true>::kSmem;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TL_CUDA(cudaLaunchKernelEx(&cfg, kernel, tx, tg, tu, p));
  } else {
    auto kernel = mlp_gate_up_tcgen05_kernel<T, false>;
    TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MlpCfg<false>::kSmem));
    cfg.gridDim = dim3(tiles < sm_count() ? tiles : sm_count());
    cfg.dynamicSmemBytes = MlpCfg<false>::kSmem;
    TL_CUDA(cudaLaunchKernelEx(&cfg, kernel, tx, tg, tu, p));
  }
  TL_LAUNCH_CHECK("mlp_gate_up_tcgen05_kernel");
  return TL_B200_OK;
}

template <typename T>
static int mlp_gate_up_simt(const void* x, const void* wg, const void* wu, void* out, int m, int n, int k, cudaStream_t s) {
  dim3 grid((n + 63) / 64, (m + 63) / 64);
  mlp_gate_up_simt_kernel<T><<<grid, 256, 0, s>>>((const T*)x, (const T*)wg, (const T*)wu, (T*)out, m, n, k);
  TL_LAUNCH_CHECK("mlp_gate_up_simt_kernel");
  return TL_B200_OK;
}

}  // namespace tl

using namespace tl;

extern "C" int tl_b200_mlp_gate_up(const void* x, const void* w_gate, const void* w_up, void* out, int64_t m, int64_t n,
                                   int64_t k, int dtype, void* stream) {
  TL_REQUIRE(m >= 0 && n >= 0 && k >= 0, "mlp_gate_up: negative size");
  TL_REQUIRE(m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31), "mlp_gate_up: dimension exceeds 2^31");
  if (m == 0 || n == 0) return TL_B200_OK;
  TL_REQUIRE(x && w_gate && w_up && out, "mlp_gate_up: null tensor pointer");
  TL_REQUIRE(k > 0, "mlp_gate_up: K must be positive");
  cudaStream_t s = (cudaStream_t)stream;
  const int M = (int)m, N = (int)n, K = (int)k;
  if (dtype == TL_F32) return mlp_gate_up_simt<float>(x, w_gate, w_up, out, M, N, K, s);
  TL_REQUIRE(dtype == TL_F16 || dtype == TL_BF16, "mlp_gate_up: unsupported dtype %d", dtype);
  const bool tma_ok = aligned16(x) && aligned16(w_gate) && aligned16(w_up) && K % 8 == 0;   // 16-byte row strides
  if (dtype == TL_BF16)
    return tma_ok ? mlp_gate_up_tc<__nv_bfloat16>(x, w_gate, w_up, out, M, N, K, s)
                  : mlp_gate_up_simt<__nv_bfloat16>(x, w_gate, w_up, out, M, N, K, s);
  return tma_ok ? mlp_gate_up_tc<__half>(x, w_gate, w_up, out, M, N, K, s)
                : mlp_gate_up_simt<__half>(x, w_gate, w_up, out, M, N, K, s);
}
