// Library management entry points and the host-side error plumbing.
#include "common.cuh"

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

}  // namespace tl

extern "C" {

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
  return TL_B200_OK;
}

int tl_b200_version(void) { return TL_B200_VERSION; }

const char* tl_b200_last_error(void) { return tl::error_buffer(); }

int64_t tl_b200_launch_count(void) { return tl::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
