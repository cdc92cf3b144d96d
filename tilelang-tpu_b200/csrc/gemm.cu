// Dense GEMM  C[M,N] = A[M,K] * B  with fp32 accumulation.
//
// Large products run on CTA pairs (`gemm_pair_kernel` below: 256 x 256 tiles, cta_group::2); smaller ones on the
// one-CTA kernel described first.
//
// The 16-bit path is a persistent, warp-specialised tcgen05 kernel: TMA brings 128xBK tiles of A
// and BNxBK tiles of B into a shared-memory ring (128-byte swizzle), one thread issues
// tcgen05.mma into a double-buffered fp32 accumulator in tensor memory, and four epilogue warps
// drain the other accumulator (tcgen05.ld -> round -> global stores) while the next tile's main
// loop already runs.  B may be [K,N] row-major (MN-major operand, the layout of the reference
// matmul program) or [N,K] row-major (K-major, `transpose_B=True` of ppl_gemm).
// e4m3 operands (the plain, un-scaled FP8 form of ppl_gemm, src/target/codegen_ppl.cc:775-790) run the same
// kernel with `kind::f8f6f4`: every byte offset is the same, a stage simply holds twice the K elements.
// fp32 inputs and shapes TMA cannot describe use a plain shared-memory-tiled FMA kernel.
#include "sm100.cuh"

#include <type_traits>

namespace tl {
using namespace sm100;

// =================================================================================
// tcgen05 kernel
// =================================================================================
constexpr int kBM = 128;        // rows of C per tile = TMEM lanes
constexpr int kRowBytes = 128;   // K bytes per stage row: one 128-byte swizzle row (64 16-bit or 128 8-bit elements)
constexpr int kUmmaBytes = 32;  // K bytes of one tcgen05.mma (16 16-bit or 32 8-bit elements)
constexpr int kGemmThreads = 256;
constexpr int kEpiWarp0 = 4;    // warps 4..7 form the epilogue (warp%4 selects the TMEM lane quarter)
constexpr int kTilePair = 512;  // tile_n value that selects 256 x 256 tiles on CTA pairs

template <int BN> struct GemmCfg {
  static constexpr int kStageA = kBM * kRowBytes;
  static constexpr int kStageB = BN * kRowBytes;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kTmemCols = 2 * BN;                      // two accumulators
  static constexpr int kSmemBytes = kStages * (kStageA + kStageB) + 1024 /*alignment*/ + 256 /*barriers*/;
};

struct GemmParams {
  void* c;
  int64_t ldc;
  int m, n, k;
  int tiles_m, tiles_n;
  int c_is_f32;       // output element: 0 = same 16-bit type as the inputs, 1 = fp32
  int in_fmt;         // kFmtF16 / kFmtBF16 (16-bit operands), kFmtE4M3 (8-bit)
  int* status;
};

// Grouped rasterisation: consecutive tile ids walk 8 row-blocks before moving to the next
// column-block, so the tiles resident at one time share A rows and B columns in L2.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int G = 8;
  const int per_group = G * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * G;
  const int rows = min(G, tiles_m - first_m);
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % rows;
  tn = in_group / rows;
}

template <typename TOut>
__device__ __forceinline__ void store_row_chunk(TOut* dst, const uint32_t (&acc)[32], int valid, bool vec_ok) {
  if constexpr (sizeof(TOut) == 4) {
    if (vec_ok && valid == 32) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<uint4*>(dst + j) = make_uint4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < valid) dst[j] = __uint_as_float(acc[j]);
    }
  } else {
    if (vec_ok && valid == 32) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        Vec16<TOut> v;
#pragma unroll
        for (int e = 0; e < 8; ++e) v.e[e] = from_f32<TOut>(__uint_as_float(acc[j + e]));
        *reinterpret_cast<uint4*>(dst + j) = v.raw;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < valid) dst[j] = from_f32<TOut>(__uint_as_float(acc[j]));
    }
  }
}

template <int BN, bool B_MN_MAJOR, typename TOut, int EB>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::kStages;
  constexpr int kBK = kRowBytes / EB;          // K elements per stage (EB = bytes per operand element)
  constexpr int kSlabCols = kRowBytes / EB;    // MN-major B: columns per 128-byte slab
  constexpr int kSlabBytes = kBK * kRowBytes;  // ... and the bytes of one slab (kBK k-rows)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;          // swizzle atoms need 1024-byte alignment
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t smem_a = base;
  const uint32_t smem_b = base + STAGES * Cfg::kStageA;
  uint8_t* tail = base_ptr + STAGES * (Cfg::kStageA + Cfg::kStageB);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail);         // full[S], empty[S], tfull[2], tempty[2]
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const int num_kb = (p.k + kBK - 1) / kBK;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 4);      // one arrival per epilogue warp
    }
    mbar_fence_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
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
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag))) break;
          const uint32_t full = bar_full + 8 * stage;
          mbar_expect_tx(full, Cfg::kStageA + Cfg::kStageB);
          tma_load_2d(smem_a + stage * Cfg::kStageA, &tm_a, full, kb * kBK, tm * kBM);
          if constexpr (B_MN_MAJOR) {
            // B is [K,N]: slabs of 128 bytes of columns x kBK k-rows (8 KB for 16-bit, 16 KB for 8-bit operands)
#pragma unroll
            for (int j = 0; j < BN / kSlabCols; ++j)
              tma_load_2d(smem_b + stage * Cfg::kStageB + j * kSlabBytes, &tm_b, full, tn * BN + j * kSlabCols,
                          kb * kBK);
          } else {
            tma_load_2d(smem_b + stage * Cfg::kStageB, &tm_b, full, kb * kBK, tn * BN);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc(p.in_fmt, p.in_fmt, false, B_MN_MAJOR, kBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!(ok = mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag))) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag))) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_a + stage * Cfg::kStageA;
          const uint32_t b_addr = smem_b + stage * Cfg::kStageB;
#pragma unroll
          for (int kk = 0; kk < kRowBytes / kUmmaBytes; ++kk) {
            // A, K-major: 8-row groups are 1024 B apart; a K step is 32 B.
            const uint64_t a_desc = smem_desc_sw128(a_addr + kk * kUmmaBytes, 16, 1024);
            uint64_t b_desc;
            if constexpr (B_MN_MAJOR)
              // MN-major: slabs one slab apart (leading), 8-k-row groups 1 KB apart (stride);
              // a K step is 32 / EB k-rows of 128 B.
              b_desc = smem_desc_sw128(b_addr + kk * (kUmmaBytes / EB * kRowBytes), kSlabBytes, 1024);
            else
              b_desc = smem_desc_sw128(b_addr + kk * kUmmaBytes, 16, 1024);
            if constexpr (EB == 2) mma_f16_ss(d_tmem, a_desc, b_desc, idesc, (kb | kk) != 0 ? 1u : 0u);
            else mma_f8_ss(d_tmem, a_desc, b_desc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          mma_commit(bar_empty + 8 * stage);          // stage is free once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) mma_commit(bar_tfull + 8 * acc);      // accumulator complete
      }
    }
  } else if (warp >= kEpiWarp0) {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp - kEpiWarp0;             // == warp % 4: TMEM lanes [32q, 32q+32)
    TOut* c = reinterpret_cast<TOut*>(p.c);
    const bool vec_ok = (p.ldc * sizeof(TOut)) % 16 == 0 && (reinterpret_cast<uintptr_t>(p.c) & 15u) == 0;
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);             // keep the warp together for the aligned loads
      if (!ok) break;
      tc_fence_after_sync();
      const int row = tm * kBM + quarter * 32 + lane;
      const uint32_t t_addr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int cchunk = 0; cchunk < BN / 32; ++cchunk) {
        uint32_t v[32];
        tmem_ld_32x32(t_addr + cchunk * 32, v);
        tmem_ld_wait();
        const int col = tn * BN + cchunk * 32;
        if (row < p.m && col < p.n)
          store_row_chunk<TOut>(c + (int64_t)row * p.ldc + col, v, min(32, p.n - col), vec_ok);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag) {
    // Some wait gave up: let copies and MMAs that are still in flight land before the shared
    // and tensor memory they target is released, then report.
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
// The same kernel on CTA pairs: one 256 x 256 tile of C per two SMs
// =================================================================================
// Two CTAs of a cluster (neighbouring SMs) own rows [0,128) and [128,256) of the tile.  Each loads its 128 rows of A
// and only HALF of the tile's B (128 of the 256 N rows); the MMAs (cta_group::2, M = 256, N = 256), issued by one
// thread of the even CTA, read B from both shared memories.  Per SM that halves the B bytes fetched from L2 and read
// from shared memory per flop, and leaves room for six stages.  Barriers: the even CTA's `full` barrier counts the
// bytes of both CTAs' loads; `empty` and `tfull` exist in both CTAs and the issuing thread commits to each; the even
// CTA's `tempty` collects the eight epilogue warps of both.
struct GemmPairCfg {
  static constexpr int kBN = 256;                    // columns of the pair's tile
  static constexpr int kHalfN = kBN / 2;             // B rows held by one CTA
  static constexpr int kStageA = kBM * kRowBytes;
  static constexpr int kStageB = kHalfN * kRowBytes;
  static constexpr int kStages = 6;
  static constexpr int kTmemCols = 2 * kBN;
  static constexpr int kSmemBytes = kStages * (kStageA + kStageB) + 1024 + 256;
};

template <bool B_MN_MAJOR, typename TOut, int EB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const GemmParams p) {
  using Cfg = GemmPairCfg;
  constexpr int STAGES = Cfg::kStages;
  constexpr int BN = Cfg::kBN;
  constexpr int kBK = kRowBytes / EB;
  constexpr int kSlabCols = kRowBytes / EB;
  constexpr int kSlabBytes = kBK * kRowBytes;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  const uint32_t smem_a = base;
  const uint32_t smem_b = base + STAGES * Cfg::kStageA;
  uint8_t* tail = base_ptr + STAGES * (Cfg::kStageA + Cfg::kStageB);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail);         // full[S], empty[S], tfull[2], tempty[2]
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();                    // 0: issues the MMAs
  const int pair = blockIdx.x / 2, num_pairs = gridDim.x / 2;
  const int num_kb = (p.k + kBK - 1) / kBK;
  const int num_tiles = p.tiles_m * p.tiles_n;                // tiles of 256 x 256

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 8);      // one arrival per epilogue warp of both CTAs (used in the even CTA)
    }
    mbar_fence_init();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
  }
  if (warp == 2) {
    tmem_alloc_pair(smem_u32(tmem_slot), Cfg::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();                        // both CTAs' barriers and tensor memory exist before anything is signalled
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int row0 = tm * 2 * kBM + (int)rank * kBM;          // this CTA's rows of A
        const int col0 = tn * BN + (int)rank * Cfg::kHalfN;       // this CTA's rows of B (columns of C)
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag))) break;
          if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * (Cfg::kStageA + Cfg::kStageB));
          const uint32_t full = map_to_cta(bar_full + 8 * stage, 0);
          tma_load_2d_pair(smem_a + stage * Cfg::kStageA, &tm_a, full, kb * kBK, row0);
          if constexpr (B_MN_MAJOR) {
#pragma unroll
            for (int j = 0; j < Cfg::kHalfN / kSlabCols; ++j)
              tma_load_2d_pair(smem_b + stage * Cfg::kStageB + j * kSlabBytes, &tm_b, full, col0 + j * kSlabCols,
                               kb * kBK);
          } else {
            tma_load_2d_pair(smem_b + stage * Cfg::kStageB, &tm_b, full, kb * kBK, col0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1 && rank == 0) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    if (elect_one()) {
      const uint32_t idesc = make_idesc(p.in_fmt, p.in_fmt, false, B_MN_MAJOR, 2 * kBM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        if (!(ok = mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag))) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag))) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_a + stage * Cfg::kStageA;
          const uint32_t b_addr = smem_b + stage * Cfg::kStageB;
#pragma unroll
          for (int kk = 0; kk < kRowBytes / kUmmaBytes; ++kk) {
            const uint64_t a_desc = smem_desc_sw128(a_addr + kk * kUmmaBytes, 16, 1024);
            uint64_t b_desc;
            if constexpr (B_MN_MAJOR)
              b_desc = smem_desc_sw128(b_addr + kk * (kUmmaBytes / EB * kRowBytes), kSlabBytes, 1024);
            else
              b_desc = smem_desc_sw128(b_addr + kk * kUmmaBytes, 16, 1024);
            if constexpr (EB == 2) mma_f16_ss_pair(d_tmem, a_desc, b_desc, idesc, (kb | kk) != 0 ? 1u : 0u);
            else mma_f8_ss_pair(d_tmem, a_desc, b_desc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          mma_commit_pair(bar_empty + 8 * stage);                        // the stage is free in this CTA ...
          mma_commit_pair(map_to_cta(bar_empty + 8 * stage, 1));         // ... and in the other
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          mma_commit_pair(bar_tfull + 8 * acc);
          mma_commit_pair(map_to_cta(bar_tfull + 8 * acc, 1));
        }
      }
    }
  } else if (warp >= kEpiWarp0) {
    // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int quarter = warp - kEpiWarp0;
    TOut* c = reinterpret_cast<TOut*>(p.c);
    const bool vec_ok = (p.ldc * sizeof(TOut)) % 16 == 0 && (reinterpret_cast<uintptr_t>(p.c) & 15u) == 0;
    int local = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = tm * 2 * kBM + (int)rank * kBM + quarter * 32 + lane;
      const uint32_t t_addr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int cchunk = 0; cchunk < BN / 32; ++cchunk) {
        uint32_t v[32];
        tmem_ld_32x32(t_addr + cchunk * 32, v);
        tmem_ld_wait();
        const int col = tn * BN + cchunk * 32;
        if (row < p.m && col < p.n)
          store_row_chunk<TOut>(c + (int64_t)row * p.ldc + col, v, min(32, p.n - col), vec_ok);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * acc, 0));
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
    if (threadIdx.x == 0 && p.status) *p.status = *abort_flag;
    __syncthreads();
  }
  // neither CTA may leave (or free tensor memory) while the other can still read its shared memory or signal its barriers
  tc_fence_before_sync();
  cluster_sync_all();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
  }
}

// =================================================================================
// Plain FMA kernel: any of fp32 / fp16 / bf16, any size and alignment.
// =================================================================================
template <typename TIn, typename TOut, bool TRANS_B>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TIn* __restrict__ a, const TIn* __restrict__ b, TOut* __restrict__ c, int m, int n, int k) {
  constexpr int T = 64, KT = 16;
  __shared__ float sa[KT][T + 1];
  __shared__ float sb[KT][T + 1];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int m0 = blockIdx.y * T, n0 = blockIdx.x * T;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < k; k0 += KT) {
    for (int i = threadIdx.x; i < T * KT; i += 256) {
      int r = i / KT, kk = i % KT;             // A tile: rows of M, K contiguous
      int gm = m0 + r, gk = k0 + kk;
      sa[kk][r] = (gm < m && gk < k) ? to_f32(a[(int64_t)gm * k + gk]) : 0.f;
    }
    for (int i = threadIdx.x; i < T * KT; i += 256) {
      int kk, cidx;
      if (TRANS_B) { cidx = i / KT; kk = i % KT; } else { kk = i / T; cidx = i % T; }
      int gn = n0 + cidx, gk = k0 + kk;
      float v = 0.f;
      if (gn < n && gk < k) v = TRANS_B ? to_f32(b[(int64_t)gn * k + gk]) : to_f32(b[(int64_t)gk * n + gn]);
      sb[kk][cidx] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < KT; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { av[i] = sa[kk][ty * 4 + i]; bv[i] = sb[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
      if (gm < m && gn < n) c[(int64_t)gm * n + gn] = from_f32<TOut>(acc[i][j]);
    }
}

template <typename TIn, typename TOut>
static int launch_simt(const void* a, const void* b, void* c, int m, int n, int k, bool trans_b, cudaStream_t s) {
  dim3 grid((n + 63) / 64, (m + 63) / 64);
  if (trans_b)
    gemm_simt_kernel<TIn, TOut, true><<<grid, 256, 0, s>>>((const TIn*)a, (const TIn*)b, (TOut*)c, m, n, k);
  else
    gemm_simt_kernel<TIn, TOut, false><<<grid, 256, 0, s>>>((const TIn*)a, (const TIn*)b, (TOut*)c, m, n, k);
  TL_LAUNCH_CHECK("gemm_simt_kernel");
  return TL_B200_OK;
}

template <int BN, bool B_MN, typename TOut, int EB = 2>
static int launch_tc(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t s) {
  auto kernel = gemm_tcgen05_kernel<BN, B_MN, TOut, EB>;
  TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<BN>::kSmemBytes));
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kernel<<<grid, kGemmThreads, GemmCfg<BN>::kSmemBytes, s>>>(ta, tb, p);
  TL_LAUNCH_CHECK("gemm_tcgen05_kernel");
  return TL_B200_OK;
}

template <int BN, typename T16>
static int launch_tc_out(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, bool b_mn,
                         cudaStream_t s) {
  if (p.c_is_f32)
    return b_mn ? launch_tc<BN, true, float>(ta, tb, p, s) : launch_tc<BN, false, float>(ta, tb, p, s);
  return b_mn ? launch_tc<BN, true, T16>(ta, tb, p, s) : launch_tc<BN, false, T16>(ta, tb, p, s);
}

// e4m3 operands: out_kind 0 = fp32, 1 = bf16, 2 = fp16
template <int BN>
static int launch_tc_f8(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, bool b_mn, int out_kind,
                        cudaStream_t s) {
  if (out_kind == 0)
    return b_mn ? launch_tc<BN, true, float, 1>(ta, tb, p, s) : launch_tc<BN, false, float, 1>(ta, tb, p, s);
  if (out_kind == 1)
    return b_mn ? launch_tc<BN, true, __nv_bfloat16, 1>(ta, tb, p, s) : launch_tc<BN, false, __nv_bfloat16, 1>(ta, tb, p, s);
  return b_mn ? launch_tc<BN, true, __half, 1>(ta, tb, p, s) : launch_tc<BN, false, __half, 1>(ta, tb, p, s);
}


template <bool B_MN, typename TOut, int EB>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t s) {
  auto kernel = gemm_pair_kernel<B_MN, TOut, EB>;
  TL_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmPairCfg::kSmemBytes));
  const int tiles = p.tiles_m * p.tiles_n;
  const int pairs = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
  kernel<<<2 * pairs, kGemmThreads, GemmPairCfg::kSmemBytes, s>>>(ta, tb, p);      // cluster size 2 is a kernel attribute
  TL_LAUNCH_CHECK("gemm_pair_kernel");
  return TL_B200_OK;
}
template <typename T16>
static int launch_pair_out(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, bool b_mn, int out_kind,
                           cudaStream_t s) {
  if constexpr (std::is_same<T16, uint8_t>::value) {
    if (out_kind == 0) return b_mn ? launch_pair<true, float, 1>(ta, tb, p, s) : launch_pair<false, float, 1>(ta, tb, p, s);
    if (out_kind == 1)
      return b_mn ? launch_pair<true, __nv_bfloat16, 1>(ta, tb, p, s) : launch_pair<false, __nv_bfloat16, 1>(ta, tb, p, s);
    return b_mn ? launch_pair<true, __half, 1>(ta, tb, p, s) : launch_pair<false, __half, 1>(ta, tb, p, s);
  } else {
    if (p.c_is_f32) return b_mn ? launch_pair<true, float, 2>(ta, tb, p, s) : launch_pair<false, float, 2>(ta, tb, p, s);
    return b_mn ? launch_pair<true, T16, 2>(ta, tb, p, s) : launch_pair<false, T16, 2>(ta, tb, p, s);
  }
}

// T16 = uint8_t selects the e4m3 form (out_kind as above); otherwise the 16-bit operand type
template <typename T16>
static int gemm_tc(const void* a, const void* b, void* c, int m, int n, int k, bool trans_b, bool c_f32,
                   cudaStream_t s, int out_kind = 0, int tile_n = 0) {
  constexpr bool is_f8 = std::is_same<T16, uint8_t>::value;
  constexpr int EB = is_f8 ? 1 : 2;
  constexpr int kBK = kRowBytes / EB;
  const bool is_bf16 = std::is_same<T16, __nv_bfloat16>::value;
  const CUtensorMapDataType dt = is_f8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                       : (is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  // Tile width: the widest that still gives every SM a tile.
  int bn = 256;
  const int tiles_m = (m + kBM - 1) / kBM;
  auto tiles_for = [&](int w) { return (int64_t)tiles_m * ((n + w - 1) / w); };
  if (tiles_for(256) < sm_count()) bn = 128;
  if (bn == 128 && tiles_for(128) < sm_count()) bn = 64;
  if (tile_n == 64 || tile_n == 128 || tile_n == 256) bn = tile_n;     // the caller's choice (a tuned table)
  // 256 x 256 tiles on CTA pairs: the caller's choice, or the library's whenever every pair of SMs gets a tile
  const int64_t pair_tiles = (int64_t)((m + 2 * kBM - 1) / (2 * kBM)) * ((n + GemmPairCfg::kBN - 1) / GemmPairCfg::kBN);
  const bool pair = tile_n == kTilePair || (tile_n == 0 && pair_tiles >= sm_count() / 2);
  if (pair) bn = GemmPairCfg::kHalfN;                                  // width of the B box one CTA loads

  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {(uint64_t)k, (uint64_t)m};
    uint64_t strides[1] = {(uint64_t)k * EB};
    uint32_t box[2] = {(uint32_t)kBK, (uint32_t)kBM};
    int rc = make_tensor_map(&ta, dt, 2, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  if (trans_b) {   // B is [N,K]: K-major
    uint64_t dims[2] = {(uint64_t)k, (uint64_t)n};
    uint64_t strides[1] = {(uint64_t)k * EB};
    uint32_t box[2] = {(uint32_t)kBK, (uint32_t)bn};
    int rc = make_tensor_map(&tb, dt, 2, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  } else {         // B is [K,N]: MN-major, loaded as slabs of 128 bytes of columns
    uint64_t dims[2] = {(uint64_t)n, (uint64_t)k};
    uint64_t strides[1] = {(uint64_t)n * EB};
    uint32_t box[2] = {(uint32_t)(kRowBytes / EB), (uint32_t)kBK};
    int rc = make_tensor_map(&tb, dt, 2, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  GemmParams p;
  p.c = c;
  p.ldc = n;
  p.m = m; p.n = n; p.k = k;
  p.tiles_m = tiles_m;
  p.tiles_n = (n + bn - 1) / bn;
  p.c_is_f32 = c_f32 ? 1 : 0;
  p.in_fmt = is_f8 ? kFmtE4M3 : (is_bf16 ? kFmtBF16 : kFmtF16);
  p.status = device_status_word();
  const bool b_mn = !trans_b;
  if (pair) {
    p.tiles_m = (m + 2 * kBM - 1) / (2 * kBM);
    p.tiles_n = (n + GemmPairCfg::kBN - 1) / GemmPairCfg::kBN;
    return launch_pair_out<T16>(ta, tb, p, b_mn, out_kind, s);
  }
  if constexpr (is_f8) {
    if (bn < 128 && b_mn) bn = 128;       // an MN-major slab of 8-bit columns is 128 columns wide
    p.tiles_n = (n + bn - 1) / bn;
    switch (bn) {
      case 256: return launch_tc_f8<256>(ta, tb, p, b_mn, out_kind, s);
      case 128: return launch_tc_f8<128>(ta, tb, p, b_mn, out_kind, s);
      default: return launch_tc_f8<64>(ta, tb, p, b_mn, out_kind, s);
    }
  } else {
    switch (bn) {
      case 256: return launch_tc_out<256, T16>(ta, tb, p, b_mn, s);
      case 128: return launch_tc_out<128, T16>(ta, tb, p, b_mn, s);
      default: return launch_tc_out<64, T16>(ta, tb, p, b_mn, s);
    }
  }
}

}  // namespace tl

using namespace tl;

extern "C" int tl_b200_gemm(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int trans_b,
                            int in_dtype, int out_dtype, void* stream) {
  return tl_b200_gemm_tiled(a, b, c, m, n, k, trans_b, in_dtype, out_dtype, 0, stream);
}

extern "C" int tl_b200_gemm_tiled(const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k, int trans_b,
                                  int in_dtype, int out_dtype, int tile_n, void* stream) {
  TL_REQUIRE(tile_n == 0 || tile_n == 64 || tile_n == 128 || tile_n == 256 || tile_n == kTilePair,
             "gemm: tile_n must be 0, 64, 128, 256 or 512 (a 256 x 256 tile on a CTA pair)");
  TL_REQUIRE(m >= 0 && n >= 0 && k >= 0, "gemm: negative size");
  TL_REQUIRE(m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31), "gemm: dimension exceeds 2^31");
  if (m == 0 || n == 0) return TL_B200_OK;
  TL_REQUIRE(a && b && c, "gemm: null tensor pointer");
  TL_REQUIRE(k > 0, "gemm: K must be positive");
  TL_REQUIRE(out_dtype == in_dtype || out_dtype == TL_F32 ||
                 (in_dtype == TL_E4M3 && (out_dtype == TL_BF16 || out_dtype == TL_F16)),
             "gemm: output must be the input type or float32 (e4m3 operands: float32, bfloat16 or float16)");
  TL_REQUIRE(!(in_dtype == TL_E4M3 && out_dtype == TL_E4M3), "gemm: e4m3 operands need a float32, bfloat16 or float16 output");
  cudaStream_t s = (cudaStream_t)stream;
  const bool tb = trans_b != 0;
  const int M = (int)m, N = (int)n, K = (int)k;
  if (in_dtype == TL_F32) return launch_simt<float, float>(a, b, c, M, N, K, tb, s);
  if (in_dtype == TL_E4M3) {
    // plain (un-scaled) FP8 product: tensor cores only; TMA needs 16-byte aligned bases and row strides
    TL_REQUIRE(aligned16(a) && aligned16(b) && K % 16 == 0 && (tb || N % 16 == 0),
               "gemm: e4m3 operands need 16-byte aligned tensors, K %% 16 == 0 and (transposed B or N %% 16 == 0)");
    const int out_kind = out_dtype == TL_F32 ? 0 : (out_dtype == TL_BF16 ? 1 : 2);
    return gemm_tc<uint8_t>(a, b, c, M, N, K, tb, out_dtype == TL_F32, s, out_kind, tile_n);
  }
  TL_REQUIRE(in_dtype == TL_F16 || in_dtype == TL_BF16, "gemm: unsupported input dtype %d", in_dtype);
  // TMA needs 16-byte aligned bases and row strides
  const bool tma_ok = aligned16(a) && aligned16(b) && K % 8 == 0 && (tb || N % 8 == 0);
  if (tma_ok) {
    if (in_dtype == TL_BF16) return gemm_tc<__nv_bfloat16>(a, b, c, M, N, K, tb, out_dtype == TL_F32, s, 0, tile_n);
    return gemm_tc<__half>(a, b, c, M, N, K, tb, out_dtype == TL_F32, s, 0, tile_n);
  }
  if (in_dtype == TL_BF16) {
    if (out_dtype == TL_F32) return launch_simt<__nv_bfloat16, float>(a, b, c, M, N, K, tb, s);
    return launch_simt<__nv_bfloat16, __nv_bfloat16>(a, b, c, M, N, K, tb, s);
  }
  if (out_dtype == TL_F32) return launch_simt<__half, float>(a, b, c, M, N, K, tb, s);
  return launch_simt<__half, __half>(a, b, c, M, N, K, tb, s);
}
