// Microbenchmark: SM clocks per tcgen05.mma (M = 128, one K step) for N = 64 / 128 / 256, operands
// from shared memory (SS) or A from tensor memory (TS), kind::f16 (bf16, K = 16) and kind::f8f6f4
// (e4m3, K = 32).  One thread issues 1600 MMAs back to back into one accumulator; the time to issue
// them and the time until the last one has completed (tcgen05.commit -> mbarrier) are reported.
// The tile shapes of the attention kernels rest on these figures (N = 64 runs at 2/3 efficiency).
//
// Build and run (not part of the library):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -Iinclude -o mma_rate \
//        tilelang-tpu_b200/csrc/microbench/mma_rate.cu tilelang-tpu_b200/csrc/api.cu -lcuda && ./mma_rate
#include "../sm100.cuh"
#include <cstdio>
using namespace tl; using namespace tl::sm100;
template <int N, bool F8, bool TS>
__global__ void __launch_bounds__(128, 1) rate_kernel(unsigned long long* out, int iters) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  __shared__ uint32_t slot; __shared__ uint64_t bar;
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&slot), 512); tmem_relinquish(); }
  if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); mbar_fence_init(); }
  for (int i = threadIdx.x; i < 32768; i += 128) reinterpret_cast<uint32_t*>(smem_raw + (base - smem_u32(smem_raw)))[i] = 0;
  fence_proxy_async_smem();
  tc_fence_before_sync(); __syncthreads(); tc_fence_after_sync();
  const uint32_t tm = slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc(F8 ? kFmtE4M3 : kFmtBF16, F8 ? kFmtE4M3 : kFmtBF16, false, false, 128, N);
    const uint64_t a = smem_desc_sw128(base, 16, 1024), b = smem_desc_sw128(base + 65536, 16, 1024);
    volatile int abortf = 0;
    long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        if (TS) { if (F8) mma_f8_ts(tm, tm + 256 + kk * 8, desc_at(b, kk * 32), idesc, 1u); else mma_f16_ts(tm, tm + 256 + kk * 8, desc_at(b, kk * 32), idesc, 1u); }
        else { if (F8) mma_f8_ss(tm, desc_at(a, kk * 32), desc_at(b, kk * 32), idesc, 1u); else mma_f16_ss(tm, desc_at(a, kk * 32), desc_at(b, kk * 32), idesc, 1u); }
      }
    }
    long long t1 = clock64();
    mma_commit(smem_u32(&bar));
    mbar_wait(smem_u32(&bar), 0, &abortf);
    long long t2 = clock64();
    out[0] = (unsigned long long)(t1 - t0); out[1] = (unsigned long long)(t2 - t0);
  }
  tc_fence_before_sync(); __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after_sync(); tmem_dealloc(tm, 512); }
}
template <int N, bool F8, bool TS> void run(const char* name) {
  unsigned long long* d; cudaMalloc(&d, 16); unsigned long long h[2];
  auto k = rate_kernel<N, F8, TS>;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  const int iters = 200;
  k<<<1, 128, 200 * 1024>>>(d, iters); k<<<1, 128, 200 * 1024>>>(d, iters);
  cudaError_t e = cudaDeviceSynchronize();
  cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
  printf("%s N=%d: issue %.1f clk/MMA, complete %.1f clk/MMA (%s)\n", name, N, h[0] / (iters * 8.0), h[1] / (iters * 8.0), cudaGetErrorString(e));
  cudaFree(d);
}
int main() {
  run<64, false, false>("bf16 SS"); run<128, false, false>("bf16 SS"); run<256, false, false>("bf16 SS");
  run<64, false, true>("bf16 TS"); run<128, false, true>("bf16 TS"); run<256, false, true>("bf16 TS");
  run<64, true, false>("e4m3 SS"); run<128, true, false>("e4m3 SS"); run<256, true, false>("e4m3 SS");
  run<64, true, true>("e4m3 TS"); run<256, true, true>("e4m3 TS");
  return 0;
}
