// Library management entry points and the host-side error plumbing.
#include "common.cuh"
#include "sm100.cuh"

#include <mutex>

namespace tl {

static thread_local char g_error[1024] = "";
static std::atomic<int64_t> g_launches{0};
static int g_sm_count = 0;
static std::once_flag g_sm_once;

char* error_buffer() { return g_error; }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count() {
  std::call_once(g_sm_once, [] {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      g_sm_count = n;
    else
      g_sm_count = 148;
  });
  return g_sm_count;
}

// ---- tensor maps -------------------------------------------------------------------------------
// cuTensorMapEncodeTiled is fetched through the runtime's driver entry point query, so the
// library carries no link-time dependency on libcuda (it must load on machines without a GPU).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;
static std::once_flag g_encode_once;

int make_tensor_map(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    CUtensorMapSwizzle swizzle) {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = (EncodeTiledFn)fn;
  });
  if (!g_encode) return fail(TL_B200_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(TL_B200_EINVAL, "tensor map base address must be 16-byte aligned");
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) {
      gstrides[i] = strides_bytes[i];
      if (gstrides[i] % 16 != 0)
        return fail(TL_B200_EINVAL, "tensor map stride %llu is not a multiple of 16 bytes",
                    (unsigned long long)gstrides[i]);
    }
  }
  CUresult r = g_encode(map, type, (cuuint32_t)rank, const_cast<void*>(base), gdims, gstrides, gbox, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TL_B200_ECUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return TL_B200_OK;
}

// ---- device status word ----------------------------------------------------------------------
// Host-mapped so the host can read it without a device allocation or a copy.
static int* g_status_host = nullptr;
static std::atomic<int*> g_status_dev{nullptr};   // published once; read without the once-flag by paths that must not allocate
static std::once_flag g_status_once;

int* device_status_word() {
  std::call_once(g_status_once, [] {
    void* h = nullptr;
    if (cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
      g_status_host = (int*)h;
      g_status_host[0] = 0;
      void* d = nullptr;
      if (cudaHostGetDevicePointer(&d, h, 0) == cudaSuccess) g_status_dev.store((int*)d, std::memory_order_release);
    }
  });
  return g_status_dev.load(std::memory_order_acquire);
}

// The status word if some earlier call created it (tl_b200_init does), nullptr otherwise: for
// paths that must not allocate.
int* device_status_word_if_created() { return g_status_dev.load(std::memory_order_acquire); }

int take_device_status() {
  if (!g_status_host) return 0;
  int v = *(volatile int*)g_status_host;
  if (v) *(volatile int*)g_status_host = 0;
  return v;
}

// One warp waits, with the library's bounded wait, on a barrier that nothing ever arrives at: the wait
// runs out of its (short) budget, the abort flag is raised and the status word is written exactly as the
// tensor-core kernels do when one of their waits gives up.  No copy or MMA is in flight, nothing hangs.
__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long budget_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    sm100::mbar_init(sm100::smem_u32(&bar), 1);
    sm100::mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = sm100::mbar_wait_budget(sm100::smem_u32(&bar), 0, &abort_flag, budget_ns);
    if (!ok && status) *status = abort_flag;
  }
}

}  // namespace tl

extern "C" {

int tl_b200_selftest_bounded_wait(int64_t budget_us, void* stream) {
  TL_REQUIRE(budget_us >= 1 && budget_us <= 100000, "selftest_bounded_wait: budget must be 1 us .. 100 ms");
  int* status = tl::device_status_word();
  TL_REQUIRE(status != nullptr, "selftest_bounded_wait: the host-mapped status word could not be created");
  tl::bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, (unsigned long long)budget_us * 1000ull);
  TL_LAUNCH_CHECK("bounded_wait_selftest_kernel");
  return TL_B200_OK;
}

int tl_b200_init(int device) {
  int n = 0;
  TL_CUDA(cudaGetDeviceCount(&n));
  TL_REQUIRE(device >= 0 && device < n, "tl_b200_init: device %d out of range (%d visible)", device, n);
  TL_CUDA(cudaSetDevice(device));
  int major = 0, minor = 0;
  TL_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  TL_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device));
  if (major != 10)
    return tl::fail(TL_B200_EUNSUP,
                    "tl_b200_init: device %d is sm_%d%d; this library holds sm_100a code only", device,
                    major, minor);
  TL_CUDA(cudaFree(0));
  // created here, where allocating is allowed, so that entry points that must not allocate can still
  // report a kernel that gave up a bounded wait
  tl::device_status_word();
  return TL_B200_OK;
}

int tl_b200_version(void) { return TL_B200_VERSION; }

const char* tl_b200_last_error(void) { return tl::error_buffer(); }

int64_t tl_b200_launch_count(void) { return tl::g_launches.load(std::memory_order_relaxed); }

int tl_b200_device_status(void) {
  int v = tl::take_device_status();
  if (v) tl::fail(TL_B200_EDEVICE, "a kernel gave up a bounded wait (device status %d)", v);
  return v;
}

}  // extern "C"
