// HBM-bound programs: RMSNorm, interleaved RoPE, SwiGLU, row reductions and the elementwise
// tile ops.  All of them make one pass over their inputs with 16-byte accesses; nothing here
// touches tensor cores.
#include "common.cuh"

#include <type_traits>

namespace tl {

constexpr int kThreads = 256;

// A VB-byte vector of T (VB = 16 or 32) with streaming / cached access.
template <typename T, int VB> struct VecT;
template <typename T> struct VecT<T, 16> {
  static constexpr int N = 16 / sizeof(T);
  Vec16<T> v;
  __device__ __forceinline__ T& operator[](int i) { return v.e[i]; }
  __device__ __forceinline__ void load_stream(const void* p) { v.raw = ld_stream16(p); }
  __device__ __forceinline__ void load_cached(const void* p) { v.raw = ld_cached16(p); }
  __device__ __forceinline__ void store_stream(void* p) { st_stream16(p, v.raw); }
};
template <typename T> struct VecT<T, 32> {
  static constexpr int N = 32 / sizeof(T);
  Vec32<T> v;
  __device__ __forceinline__ T& operator[](int i) { return v.e[i]; }
  __device__ __forceinline__ void load_stream(const void* p) { v = ld_stream32<T>(p); }
  __device__ __forceinline__ void load_cached(const void* p) { v = ld_cached32<T>(p); }
  __device__ __forceinline__ void store_stream(void* p) { st_stream32<T>(p, v); }
};

// Grid for a grid-stride kernel: exactly the CTAs that are resident at once (a multiple of the
// SM count), never more than the work needs.
template <typename K>
static unsigned resident_grid(K kernel, int64_t work_items, int per_cta) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0) != cudaSuccess || per_sm < 1)
    per_sm = 4;
  int64_t need = (work_items + per_cta - 1) / per_cta;
  int64_t cap = (int64_t)sm_count() * per_sm;
  if (need < 1) need = 1;
  return (unsigned)(need < cap ? need : cap);
}

// =================================================================================
// RMSNorm.  THREADS_PER_ROW threads own one row and keep it in registers between the
// sum-of-squares pass and the scaling pass, so every element is read once and written once.
// =================================================================================
template <typename T, int VB, int TPR, int VPT>
__global__ void __launch_bounds__(kThreads)
rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, int64_t rows,
               int nvec, float inv_cols, float eps) {
  dependency_wait();             // launched so that it may start under its predecessor's tail
  dependency_release();
  using V = VecT<T, VB>;
  constexpr int VN = V::N;
  constexpr int ROWS_PER_CTA = kThreads / TPR;
  __shared__ float partial[kThreads / 32];

  const int lane_in_row = threadIdx.x % TPR;
  const int row_in_cta = threadIdx.x / TPR;
  const int64_t row = (int64_t)blockIdx.x * ROWS_PER_CTA + row_in_cta;
  const bool live = row < rows;

  V v[VPT];
  float ss = 0.f;
  if (live) {
    const char* xr = reinterpret_cast<const char*>(x) + row * nvec * VB;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int c = lane_in_row + i * TPR;
      if (c < nvec) v[i].load_stream(xr + (int64_t)c * VB);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int c = lane_in_row + i * TPR;
      if (c < nvec) {
#pragma unroll
        for (int j = 0; j < VN; ++j) {
          float f = to_f32(v[i][j]);
          ss = fmaf(f, f, ss);
        }
      }
    }
  }
  ss = warp_sum(ss);
  if constexpr (TPR > 32) {
    constexpr int WPR = TPR / 32;  // warps per row
    const int warp = threadIdx.x / 32;
    if ((threadIdx.x & 31) == 0) partial[warp] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int k = 0; k < WPR; ++k) ss += partial[row_in_cta * WPR + k];
  }
  if (!live) return;
  const float r = rsqrtf(ss * inv_cols + eps);
  char* yr = reinterpret_cast<char*>(y) + row * nvec * VB;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    int c = lane_in_row + i * TPR;
    if (c < nvec) {
      V o;
      if (w != nullptr) {
        V wv;
        wv.load_cached(reinterpret_cast<const char*>(w) + (int64_t)c * VB);
#pragma unroll
        for (int j = 0; j < VN; ++j) o[j] = from_f32<T>(to_f32(v[i][j]) * r * to_f32(wv[j]));
      } else {
#pragma unroll
        for (int j = 0; j < VN; ++j) o[j] = from_f32<T>(to_f32(v[i][j]) * r);
      }
      o.store_stream(yr + (int64_t)c * VB);
    }
  }
}

// Any width, any alignment: one CTA per row, two scalar passes (the second one hits L2).
template <typename T>
__global__ void __launch_bounds__(kThreads)
rmsnorm_generic_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                       int64_t cols, float inv_cols, float eps) {
  __shared__ float partial[kThreads / 32];
  const T* xr = x + (int64_t)blockIdx.x * cols;
  T* yr = y + (int64_t)blockIdx.x * cols;
  float ss = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += kThreads) {
    float f = to_f32(xr[c]);
    ss = fmaf(f, f, ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x / 32] = ss;
  __syncthreads();
  ss = 0.f;
#pragma unroll
  for (int k = 0; k < kThreads / 32; ++k) ss += partial[k];
  const float r = rsqrtf(ss * inv_cols + eps);
  for (int64_t c = threadIdx.x; c < cols; c += kThreads) {
    float f = to_f32(xr[c]) * r;
    if (w != nullptr) f *= to_f32(w[c]);
    yr[c] = from_f32<T>(f);
  }
}

template <typename T, int VB, int TPR, int VPT>
static int launch_rmsnorm(const void* x, const void* w, void* y, int64_t rows, int nvec, float inv_cols,
                          float eps, cudaStream_t s) {
  constexpr int RPC = kThreads / TPR;
  int64_t grid = (rows + RPC - 1) / RPC;
  TL_CUDA(launch_overlapped(rmsnorm_kernel<T, VB, TPR, VPT>, dim3((unsigned)grid), dim3(kThreads), 0, s, (const T*)x,
                            (const T*)w, (T*)y, rows, nvec, inv_cols, eps));
  TL_LAUNCH_CHECK("rmsnorm_kernel");
  return TL_B200_OK;
}

// Rows up to 256 vectors are owned by one warp (no CTA-wide barrier at all); longer rows by a
// whole CTA.
template <typename T, int VB>
static int rmsnorm_vec(const void* x, const void* w, void* y, int64_t rows, int nv, float inv_cols, float eps,
                       cudaStream_t s) {
  if (nv <= 32) return launch_rmsnorm<T, VB, 32, 1>(x, w, y, rows, nv, inv_cols, eps, s);
  if (nv <= 64) return launch_rmsnorm<T, VB, 32, 2>(x, w, y, rows, nv, inv_cols, eps, s);
  // two vectors per thread: a row spread over more warps keeps more rows' loads in flight per SM than one warp
  // holding a whole row in registers (8192 x 4096 bf16: 31 -> 27 us inside the benchmark step)
  if (nv <= 128) return launch_rmsnorm<T, VB, 64, 2>(x, w, y, rows, nv, inv_cols, eps, s);
  if (nv <= 256) return launch_rmsnorm<T, VB, 128, 2>(x, w, y, rows, nv, inv_cols, eps, s);
  if (nv <= 512) return launch_rmsnorm<T, VB, 256, 2>(x, w, y, rows, nv, inv_cols, eps, s);
  if (nv <= 1024) return launch_rmsnorm<T, VB, 256, 4>(x, w, y, rows, nv, inv_cols, eps, s);
  return launch_rmsnorm<T, VB, 256, 8>(x, w, y, rows, nv, inv_cols, eps, s);
}

template <typename T>
static int rmsnorm_dispatch(const void* x, const void* w, void* y, int64_t rows, int64_t cols, float eps,
                            cudaStream_t s) {
  const float inv_cols = 1.0f / (float)cols;
  const int64_t row_bytes = cols * (int64_t)sizeof(T);
  TL_REQUIRE(rows < (1ll << 31), "rmsnorm: rows %lld too large", (long long)rows);
  if (row_bytes % 32 == 0 && row_bytes / 32 <= 2048 && aligned32(x) && aligned32(y) &&
      (w == nullptr || aligned32(w)))
    return rmsnorm_vec<T, 32>(x, w, y, rows, (int)(row_bytes / 32), inv_cols, eps, s);
  if (row_bytes % 16 == 0 && row_bytes / 16 <= 2048 && aligned16(x) && aligned16(y) &&
      (w == nullptr || aligned16(w)))
    return rmsnorm_vec<T, 16>(x, w, y, rows, (int)(row_bytes / 16), inv_cols, eps, s);
  rmsnorm_generic_kernel<T><<<(unsigned)rows, kThreads, 0, s>>>((const T*)x, (const T*)w, (T*)y, cols,
                                                                inv_cols, eps);
  TL_LAUNCH_CHECK("rmsnorm_generic_kernel");
  return TL_B200_OK;
}

// =================================================================================
// RoPE on interleaved pairs.  One 16-byte vector holds whole (even, odd) pairs, so a thread
// needs no neighbour's data.  Intermediate products are rounded to T exactly where the
// reference's tile ops round them (ppl_mul, ppl_mul_C, ppl_rope_add all work in tile dtype).
// =================================================================================
template <typename T> __device__ __forceinline__ float rnd(float v) { return to_f32(from_f32<T>(v)); }

// One output pair.  __fmul_rn / __fadd_rn keep the products and the sum as separate roundings
// (no FMA contraction), which is what separate tile ops produce; for 16-bit T each of them is
// additionally rounded to T.
template <typename T>
__device__ __forceinline__ void rope_pair(float xe, float xo, float ce, float co, float se, float so, T& oe,
                                          T& oo) {
  // out[2i]   = (x*cos)[2i]   + (-x*sin)[2i+1]
  // out[2i+1] = (x*cos)[2i+1] + ( x*sin)[2i]
  oe = from_f32<T>(__fadd_rn(rnd<T>(__fmul_rn(xe, ce)), rnd<T>(__fmul_rn(-xo, so))));
  oo = from_f32<T>(__fadd_rn(rnd<T>(__fmul_rn(xo, co)), rnd<T>(__fmul_rn(xe, se))));
}

// Packed form for 16-bit types: one 32-bit word holds an (even, odd) pair.  A bf16x2 / f16x2
// multiply rounds each exact product once to T, which is exactly the rounding of the separate
// tile multiplies, and costs no float conversion; only the final sum goes through fp32.
template <typename T> struct Pair16;
template <> struct Pair16<__nv_bfloat16> {
  using V2 = __nv_bfloat162;
  static __device__ __forceinline__ float lo(uint32_t w) { return __uint_as_float(w << 16); }
  static __device__ __forceinline__ float hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    V2 r = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
  }
};
template <> struct Pair16<__half> {
  using V2 = __half2;
  static __device__ __forceinline__ float lo(uint32_t w) { return __low2float(*reinterpret_cast<V2*>(&w)); }
  static __device__ __forceinline__ float hi(uint32_t w) { return __high2float(*reinterpret_cast<V2*>(&w)); }
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    V2 r = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&r);
  }
};
template <typename T>
__device__ __forceinline__ uint32_t rope_word(uint32_t x, uint32_t c, uint32_t s) {
  using P = Pair16<T>;
  using V2 = typename P::V2;
  V2 xc = __hmul2(*reinterpret_cast<V2*>(&x), *reinterpret_cast<V2*>(&c));   // (xe*ce, xo*co)
  V2 xs = __hmul2(*reinterpret_cast<V2*>(&x), *reinterpret_cast<V2*>(&s));   // (xe*se, xo*so)
  const uint32_t wc = *reinterpret_cast<uint32_t*>(&xc), ws = *reinterpret_cast<uint32_t*>(&xs);
  // out[2i] = (x*cos)[2i] + (-x*sin)[2i+1];  out[2i+1] = (x*cos)[2i+1] + (x*sin)[2i]
  return P::pack(__fadd_rn(P::lo(wc), -P::hi(ws)), __fadd_rn(P::hi(wc), P::lo(ws)));
}

template <typename T, int VB, int UNROLL>
__global__ void __launch_bounds__(kThreads)
rope_kernel(const T* __restrict__ x, const T* __restrict__ cos_tab, const T* __restrict__ sin_tab,
            T* __restrict__ out, uint32_t total_vec, uint32_t vec_per_row, uint32_t vec_per_table_row) {
  dependency_wait();             // launched so that it may start under its predecessor's tail
  dependency_release();
  using V = VecT<T, VB>;
  constexpr int VN = V::N;
  const uint32_t stride = gridDim.x * kThreads;
  const char* xb = reinterpret_cast<const char*>(x);
  const char* cb = reinterpret_cast<const char*>(cos_tab);
  const char* sb = reinterpret_cast<const char*>(sin_tab);
  char* ob = reinterpret_cast<char*>(out);
  // total_vec < 2^31, so base + u*stride cannot wrap before the bound check
  for (uint32_t base = blockIdx.x * kThreads + threadIdx.x; base < total_vec; base += stride * UNROLL) {
    V xa[UNROLL], ca[UNROLL], sa[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      uint32_t i = base + u * stride;
      if (i < total_vec) {
        // vec_per_table_row = vectors of x served by one table row (heads * vec_per_row)
        uint32_t t = (i / vec_per_table_row) * vec_per_row + i % vec_per_row;
        xa[u].load_stream(xb + (int64_t)i * VB);
        ca[u].load_cached(cb + (int64_t)t * VB);
        sa[u].load_cached(sb + (int64_t)t * VB);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      uint32_t i = base + u * stride;
      if (i < total_vec) {
        V o;
        if constexpr (sizeof(T) == 2) {
          const uint32_t* xw = reinterpret_cast<const uint32_t*>(&xa[u]);
          const uint32_t* cw = reinterpret_cast<const uint32_t*>(&ca[u]);
          const uint32_t* sw = reinterpret_cast<const uint32_t*>(&sa[u]);
          uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
          for (int p = 0; p < VB / 4; ++p) ow[p] = rope_word<T>(xw[p], cw[p], sw[p]);
        } else {
#pragma unroll
          for (int p = 0; p < VN; p += 2)
            rope_pair<T>(to_f32(xa[u][p]), to_f32(xa[u][p + 1]), to_f32(ca[u][p]), to_f32(ca[u][p + 1]),
                         to_f32(sa[u][p]), to_f32(sa[u][p + 1]), o[p], o[p + 1]);
        }
        o.store_stream(ob + (int64_t)i * VB);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
rope_generic_kernel(const T* __restrict__ x, const T* __restrict__ cos_tab, const T* __restrict__ sin_tab,
                    T* __restrict__ out, int64_t total_pairs, int64_t half_width,
                    int64_t rows_per_table_row) {
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < total_pairs; i += stride) {
    int64_t row = i / half_width;
    int64_t p = i - row * half_width;
    int64_t xi = row * half_width * 2 + 2 * p;
    int64_t ti = (row / rows_per_table_row) * half_width * 2 + 2 * p;
    float xe = to_f32(x[xi]), xo = to_f32(x[xi + 1]);
    float ce = to_f32(cos_tab[ti]), co = to_f32(cos_tab[ti + 1]);
    float se = to_f32(sin_tab[ti]), so = to_f32(sin_tab[ti + 1]);
    rope_pair<T>(xe, xo, ce, co, se, so, out[xi], out[xi + 1]);
  }
}

static unsigned elementwise_grid(int64_t work_items, int per_cta) {
  int64_t need = (work_items + per_cta - 1) / per_cta;
  int64_t cap = (int64_t)sm_count() * 8;  // 8 CTAs of 256 threads fill an SM
  if (need < 1) need = 1;
  return (unsigned)(need < cap ? need : cap);
}

template <typename T, int VB, int UNROLL>
static int launch_rope(const void* x, const void* c, const void* sn, void* out, int64_t rows, int64_t width,
                       int64_t rptr, cudaStream_t s) {
  const int64_t vpr = width * (int64_t)sizeof(T) / VB;
  const int64_t total_vec = rows * vpr;
  auto kernel = rope_kernel<T, VB, UNROLL>;
  unsigned grid = resident_grid(kernel, total_vec, kThreads * UNROLL);
  TL_CUDA(launch_overlapped(kernel, dim3(grid), dim3(kThreads), 0, s, (const T*)x, (const T*)c, (const T*)sn, (T*)out,
                            (uint32_t)total_vec, (uint32_t)vpr, (uint32_t)(vpr * rptr)));
  TL_LAUNCH_CHECK("rope_kernel");
  return TL_B200_OK;
}

template <typename T>
static int rope_dispatch(const void* x, const void* c, const void* sn, void* out, int64_t rows, int64_t width,
                         int64_t rptr, cudaStream_t s) {
  const int64_t row_bytes = width * (int64_t)sizeof(T);
  // the vector kernels index with 32 bits
  const bool small = rows * row_bytes / 16 < (1ll << 31) && row_bytes / 16 * rptr < (1ll << 31);
  if (small && row_bytes % 32 == 0 && aligned32(x) && aligned32(c) && aligned32(sn) && aligned32(out))
    return launch_rope<T, 32, 2>(x, c, sn, out, rows, width, rptr, s);
  if (small && row_bytes % 16 == 0 && aligned16(x) && aligned16(c) && aligned16(sn) && aligned16(out))
    return launch_rope<T, 16, 4>(x, c, sn, out, rows, width, rptr, s);
  int64_t total_pairs = rows * (width / 2);
  unsigned grid = elementwise_grid(total_pairs, kThreads);
  rope_generic_kernel<T><<<grid, kThreads, 0, s>>>((const T*)x, (const T*)c, (const T*)sn, (T*)out,
                                                   total_pairs, width / 2, rptr);
  TL_LAUNCH_CHECK("rope_generic_kernel");
  return TL_B200_OK;
}

// =================================================================================
// SwiGLU: out = up * gate / (1 + exp(-gate)).
// =================================================================================
template <typename T> __device__ __forceinline__ float silu_mul(float g, float u) {
  if constexpr (sizeof(T) == 4) {
    return u * (g / (1.0f + expf(-g)));
  } else {
    // 16-bit outputs keep 8-11 significant bits; the fast exponential and division
    // are far inside that.
    // silu(g) = g * sigmoid(g) = 0.5 g (1 + tanh(g / 2)): one XU operation (tanh.approx, relative error
    // 2^-11) instead of two (ex2 and rcp)
    // Below -17 the true value is under 1e-6 in magnitude and 1 + tanh would be all rounding error: zero.
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * g));
    return g < -17.0f ? 0.0f * u : u * (0.5f * g * (1.0f + t));
  }
}

template <typename T, int VB, int UNROLL>
__global__ void __launch_bounds__(kThreads)
swiglu_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out, int64_t nvec,
              int64_t n_elems) {
  dependency_wait();             // launched so that it may start under its predecessor's tail
  dependency_release();
  using V = VecT<T, VB>;
  constexpr int VN = V::N;
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  const int64_t tid = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  const char* gb = reinterpret_cast<const char*>(gate);
  const char* ub = reinterpret_cast<const char*>(up);
  char* ob = reinterpret_cast<char*>(out);
  for (int64_t base = tid; base < nvec; base += stride * UNROLL) {
    V g[UNROLL], u[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      int64_t i = base + k * stride;
      if (i < nvec) {
        g[k].load_stream(gb + i * VB);
        u[k].load_stream(ub + i * VB);
      }
    }
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
      int64_t i = base + k * stride;
      if (i < nvec) {
        V o;
#pragma unroll
        for (int j = 0; j < VN; ++j) o[j] = from_f32<T>(silu_mul<T>(to_f32(g[k][j]), to_f32(u[k][j])));
        o.store_stream(ob + i * VB);
      }
    }
  }
  // ragged tail (fewer than one vector)
  for (int64_t i = nvec * VN + tid; i < n_elems; i += stride)
    out[i] = from_f32<T>(silu_mul<T>(to_f32(gate[i]), to_f32(up[i])));
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_scalar_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride)
    out[i] = from_f32<T>(silu_mul<T>(to_f32(gate[i]), to_f32(up[i])));
}

template <typename T, int VB, int UNROLL>
static int launch_swiglu(const void* g, const void* u, void* o, int64_t n, cudaStream_t s) {
  int64_t nvec = n * (int64_t)sizeof(T) / VB;
  auto kernel = swiglu_kernel<T, VB, UNROLL>;
  unsigned grid = resident_grid(kernel, nvec, kThreads * UNROLL);
  TL_CUDA(launch_overlapped(kernel, dim3(grid), dim3(kThreads), 0, s, (const T*)g, (const T*)u, (T*)o, nvec, n));
  TL_LAUNCH_CHECK("swiglu_kernel");
  return TL_B200_OK;
}

template <typename T>
static int swiglu_dispatch(const void* g, const void* u, void* o, int64_t n, cudaStream_t s) {
  if (aligned32(g) && aligned32(u) && aligned32(o)) return launch_swiglu<T, 32, 2>(g, u, o, n, s);
  if (aligned16(g) && aligned16(u) && aligned16(o)) return launch_swiglu<T, 16, 4>(g, u, o, n, s);
  unsigned grid = elementwise_grid(n, kThreads);
  swiglu_scalar_kernel<T><<<grid, kThreads, 0, s>>>((const T*)g, (const T*)u, (T*)o, n);
  TL_LAUNCH_CHECK("swiglu_scalar_kernel");
  return TL_B200_OK;
}

// =================================================================================
// Row reductions: sum or max over the columns of each row, fp32 accumulation.
// TPR threads (a warp or the whole CTA) walk one row.
// =================================================================================
template <typename T, int TPR, bool IS_MAX, bool VEC>
__global__ void __launch_bounds__(kThreads)
reduce_rows_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int64_t cols) {
  constexpr int VN = Vec16<T>::N;
  constexpr int ROWS_PER_CTA = kThreads / TPR;
  __shared__ float partial[kThreads / 32];
  const int lane_in_row = threadIdx.x % TPR;
  const int row_in_cta = threadIdx.x / TPR;
  const int64_t row = (int64_t)blockIdx.x * ROWS_PER_CTA + row_in_cta;
  const bool live = row < rows;
  float acc = IS_MAX ? -INFINITY : 0.f;
  if (live) {
    const T* xr = x + row * cols;
    int64_t done = 0;
    if constexpr (VEC) {
      const int64_t nvec = cols / VN;
      const uint4* xv = reinterpret_cast<const uint4*>(xr);
      // four independent 16-byte loads in flight per thread, then their elements
      constexpr int U = 4;
      for (int64_t c = lane_in_row; c < nvec; c += (int64_t)TPR * U) {
        Vec16<T> v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (c + (int64_t)u * TPR < nvec) v[u].raw = ld_stream16(xv + c + (int64_t)u * TPR);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (c + (int64_t)u * TPR < nvec) {
#pragma unroll
            for (int j = 0; j < VN; ++j) {
              float f = to_f32(v[u].e[j]);
              acc = IS_MAX ? fmaxf(acc, f) : acc + f;
            }
          }
        }
      }
      done = nvec * VN;
    }
    for (int64_t c = done + lane_in_row; c < cols; c += TPR) {
      float f = to_f32(xr[c]);
      acc = IS_MAX ? fmaxf(acc, f) : acc + f;
    }
  }
  acc = IS_MAX ? warp_max(acc) : warp_sum(acc);
  if constexpr (TPR > 32) {
    constexpr int WPR = TPR / 32;
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x / 32] = acc;
    __syncthreads();
    acc = IS_MAX ? -INFINITY : 0.f;
#pragma unroll
    for (int k = 0; k < WPR; ++k) {
      float p = partial[row_in_cta * WPR + k];
      acc = IS_MAX ? fmaxf(acc, p) : acc + p;
    }
  }
  if (live && lane_in_row == 0) y[row] = from_f32<T>(acc);
}

template <typename T, bool IS_MAX>
static int reduce_dispatch(const void* x, void* y, int64_t rows, int64_t cols, cudaStream_t s) {
  constexpr int VN = Vec16<T>::N;
  const bool vec = aligned16(x) && cols % VN == 0;
  const bool wide = cols * (int64_t)sizeof(T) > 4096;  // beyond 4 KB a whole CTA walks the row
  const int rpc = wide ? 1 : kThreads / 32;
  int64_t grid = (rows + rpc - 1) / rpc;
  TL_REQUIRE(grid < (1ll << 31), "reduce_rows: too many rows (%lld)", (long long)rows);
#define TL_RED(TPR, V)                                                                        \
  reduce_rows_kernel<T, TPR, IS_MAX, V><<<(unsigned)grid, kThreads, 0, s>>>((const T*)x, (T*)y, rows, cols)
  if (wide) { if (vec) TL_RED(256, true); else TL_RED(256, false); }
  else      { if (vec) TL_RED(32, true);  else TL_RED(32, false); }
#undef TL_RED
  TL_LAUNCH_CHECK("reduce_rows_kernel");
  return TL_B200_OK;
}

// Integer row sums (ppl_reduce_sum accepts int32 / uint32 / int16 tiles, src/target/codegen_ppl.cc:1570-1592):
// a warp per row, sums modulo 2^32 (int16: the 32-bit sum cut to 16 bits), so signed and unsigned share the bits.
template <typename T>
__global__ void __launch_bounds__(kThreads)
reduce_sum_int_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int64_t cols) {
  const int lane = threadIdx.x % 32;
  const int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + threadIdx.x / 32;
  if (row >= rows) return;
  const T* xr = x + row * cols;
  uint32_t acc = 0;
  for (int64_t c = lane; c < cols; c += 32) acc += (uint32_t)(int32_t)xr[c];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) y[row] = (T)acc;
}

template <typename T>
static int reduce_sum_int(const void* x, void* y, int64_t rows, int64_t cols, cudaStream_t s) {
  const int64_t grid = (rows + kThreads / 32 - 1) / (kThreads / 32);
  TL_REQUIRE(grid < (1ll << 31), "reduce_rows: too many rows (%lld)", (long long)rows);
  reduce_sum_int_kernel<T><<<(unsigned)grid, kThreads, 0, s>>>((const T*)x, (T*)y, rows, cols);
  TL_LAUNCH_CHECK("reduce_sum_int_kernel");
  return TL_B200_OK;
}

// =================================================================================
// Elementwise tile ops (scalar indexing; these back the generic per-op path, not a
// bandwidth headline).
// =================================================================================
template <int OP> __device__ __forceinline__ float unary_op(float f) {
  // sigmoid: ex2-based exponential (error 2 + |1.16 x| ulp, inside the 1e-5 of the fp32 path up to the overflow of
  // exp) and an IEEE-rounded reciprocal, which unlike the fast division keeps the results below 2^-126
  if constexpr (OP == 0) return __frcp_rn(1.0f + __expf(-f));
  else if constexpr (OP == 1) return expf(f);
  else if constexpr (OP == 2) return 1.0f / sqrtf(f);
  else return f;
}

// fp32 -> fp32 on 16-byte aligned tensors: four elements per load and store, two vectors in flight per thread
template <int OP>
__global__ void __launch_bounds__(kThreads)
unary_vec_kernel(const float4* __restrict__ x, float4* __restrict__ y, int64_t n4) {
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  constexpr int U = 2;
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += stride * U) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = i + u * stride < n4 ? __ldg(x + i + u * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i + u * stride < n4)
        y[i + u * stride] = make_float4(unary_op<OP>(v[u].x), unary_op<OP>(v[u].y), unary_op<OP>(v[u].z), unary_op<OP>(v[u].w));
  }
}

template <typename TI, typename TO, int OP>
__global__ void __launch_bounds__(kThreads)
unary_kernel(const TI* __restrict__ x, TO* __restrict__ y, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  constexpr int U = 4;                          // four independent loads in flight per thread
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride * U) {
    float f[U];
#pragma unroll
    for (int u = 0; u < U; ++u) f[u] = i + u * stride < n ? to_f32(x[i + u * stride]) : 0.f;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const float r = unary_op<OP>(f[u]);
      if (i + u * stride < n) y[i + u * stride] = from_f32<TO>(r);
    }
  }
}

template <typename T, int OP, int BMODE>
__global__ void __launch_bounds__(kThreads)
binary_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t n, int64_t cols,
              float scalar) {
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
    float av = to_f32(a[i]);
    float bv;
    if constexpr (BMODE == 0) bv = to_f32(b[i]);
    else if constexpr (BMODE == 1) bv = to_f32(b[i / cols]);
    else if constexpr (BMODE == 3) bv = to_f32(b[i % cols]);
    else bv = to_f32(from_f32<T>(scalar));  // scalar is first cast to the tile dtype
    float r;
    if constexpr (OP == 0) r = av + bv;
    else if constexpr (OP == 1) r = av - bv;
    else if constexpr (OP == 2) r = av * bv;
    else if constexpr (OP == 3) r = av / bv;
    else r = fmaxf(av, bv);
    out[i] = from_f32<T>(r);
  }
}

// fp32 tensors of equal shape (or a scalar second operand) on 16-byte aligned memory: four elements per access
template <int OP, bool SCALAR>
__global__ void __launch_bounds__(kThreads)
binary_vec_kernel(const float4* __restrict__ a, const float4* __restrict__ b, float4* __restrict__ out, int64_t n4,
                  float scalar) {
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  auto op = [](float x, float y) {
    if constexpr (OP == 0) return x + y;
    else if constexpr (OP == 1) return x - y;
    else if constexpr (OP == 2) return x * y;
    else if constexpr (OP == 3) return x / y;
    else return fmaxf(x, y);
  };
  constexpr int U = 2;
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n4; i += stride * U) {
    float4 av[U], bv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t k = i + u * stride;
      av[u] = k < n4 ? __ldg(a + k) : make_float4(0.f, 0.f, 0.f, 0.f);
      if constexpr (SCALAR) bv[u] = make_float4(scalar, scalar, scalar, scalar);
      else bv[u] = k < n4 ? __ldg(b + k) : make_float4(1.f, 1.f, 1.f, 1.f);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t k = i + u * stride;
      if (k < n4) out[k] = make_float4(op(av[u].x, bv[u].x), op(av[u].y, bv[u].y), op(av[u].z, bv[u].z), op(av[u].w, bv[u].w));
    }
  }
}

// Strided 2-D copy with a cast (a tile <-> a window of a larger tensor), and a 2-D fill.
template <typename TI, typename TO>
__global__ void __launch_bounds__(kThreads)
copy2d_kernel(const TI* __restrict__ src, TO* __restrict__ dst, int64_t rows, int64_t cols, int64_t src_ld,
              int64_t dst_ld) {
  // grid.y walks the rows, grid.x the columns: no division per element
  for (int64_t r = blockIdx.y; r < rows; r += gridDim.y) {
    const TI* sr = src + r * src_ld;
    TO* dr = dst + r * dst_ld;
    for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < cols; c += (int64_t)gridDim.x * kThreads) {
      if constexpr (std::is_same<TI, TO>::value) dr[c] = sr[c];
      else dr[c] = from_f32<TO>(to_f32(sr[c]));
    }
  }
}

// Launch shape of the 2-D kernels: up to 64 CTAs across a row, as many row walkers as fill the machine.
static dim3 grid2d(int64_t rows, int64_t cols) {
  int64_t gx = (cols + kThreads - 1) / kThreads;
  if (gx > 64) gx = 64;
  int64_t gy = ((int64_t)sm_count() * 8 + gx - 1) / gx;
  if (gy > rows) gy = rows;
  if (gy > 65535) gy = 65535;
  if (gy < 1) gy = 1;
  return dim3((unsigned)gx, (unsigned)gy);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
fill2d_kernel(T* __restrict__ dst, int64_t rows, int64_t cols, int64_t ld, T value) {
  for (int64_t r = blockIdx.y; r < rows; r += gridDim.y)
    for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < cols; c += (int64_t)gridDim.x * kThreads)
      dst[r * ld + c] = value;
}

// out[:, 2i] = e1[:, 2i] + e2[:, 2i+1];  out[:, 2i+1] = o1[:, 2i+1] + o2[:, 2i]   (contiguous tiles)
template <typename T>
__global__ void __launch_bounds__(kThreads)
rope_add_kernel(T* __restrict__ out, const T* __restrict__ e1, const T* __restrict__ e2, const T* __restrict__ o1,
                const T* __restrict__ o2, int64_t pairs) {
  const int64_t stride = (int64_t)gridDim.x * kThreads;
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < pairs; i += stride) {
    const int64_t c = 2 * i;
    out[c] = from_f32<T>(__fadd_rn(to_f32(e1[c]), to_f32(e2[c + 1])));
    out[c + 1] = from_f32<T>(__fadd_rn(to_f32(o1[c + 1]), to_f32(o2[c])));
  }
}

template <typename T>
static int rope_add_launch(void* out, const void* e1, const void* e2, const void* o1, const void* o2, int64_t pairs,
                           cudaStream_t s) {
  rope_add_kernel<T><<<elementwise_grid(pairs, kThreads * 4), kThreads, 0, s>>>((T*)out, (const T*)e1, (const T*)e2,
                                                                               (const T*)o1, (const T*)o2, pairs);
  TL_LAUNCH_CHECK("rope_add_kernel");
  return TL_B200_OK;
}

template <typename TI>
static int copy2d_out(const void* src, void* dst, int64_t rows, int64_t cols, int64_t sld, int64_t dld, int out_dtype,
                      cudaStream_t s) {
  const dim3 grid = grid2d(rows, cols);
  switch (out_dtype) {
    case TL_F32: copy2d_kernel<TI, float><<<grid, kThreads, 0, s>>>((const TI*)src, (float*)dst, rows, cols, sld, dld); break;
    case TL_F16: copy2d_kernel<TI, __half><<<grid, kThreads, 0, s>>>((const TI*)src, (__half*)dst, rows, cols, sld, dld); break;
    case TL_BF16:
      copy2d_kernel<TI, __nv_bfloat16><<<grid, kThreads, 0, s>>>((const TI*)src, (__nv_bfloat16*)dst, rows, cols, sld, dld);
      break;
    default: return fail(TL_B200_EINVAL, "copy2d: unsupported output dtype %d", out_dtype);
  }
  TL_LAUNCH_CHECK("copy2d_kernel");
  return TL_B200_OK;
}

template <typename TI, typename TO>
static int unary_dispatch(const void* x, void* y, int64_t n, int op, cudaStream_t s) {
  if constexpr (std::is_same<TI, float>::value && std::is_same<TO, float>::value) {
    if (n % 4 == 0 && aligned16(x) && aligned16(y) && op >= 0 && op <= 3) {
      const int64_t n4 = n / 4;
      unsigned vgrid = elementwise_grid(n4, kThreads * 2);
      const float4* xv = (const float4*)x;
      float4* yv = (float4*)y;
      switch (op) {
        case 0: unary_vec_kernel<0><<<vgrid, kThreads, 0, s>>>(xv, yv, n4); break;
        case 1: unary_vec_kernel<1><<<vgrid, kThreads, 0, s>>>(xv, yv, n4); break;
        case 2: unary_vec_kernel<2><<<vgrid, kThreads, 0, s>>>(xv, yv, n4); break;
        default: unary_vec_kernel<3><<<vgrid, kThreads, 0, s>>>(xv, yv, n4); break;
      }
      TL_LAUNCH_CHECK("unary_vec_kernel");
      return TL_B200_OK;
    }
  }
  unsigned grid = elementwise_grid(n, kThreads * 4);
  switch (op) {
    case 0: unary_kernel<TI, TO, 0><<<grid, kThreads, 0, s>>>((const TI*)x, (TO*)y, n); break;
    case 1: unary_kernel<TI, TO, 1><<<grid, kThreads, 0, s>>>((const TI*)x, (TO*)y, n); break;
    case 2: unary_kernel<TI, TO, 2><<<grid, kThreads, 0, s>>>((const TI*)x, (TO*)y, n); break;
    case 3: unary_kernel<TI, TO, 3><<<grid, kThreads, 0, s>>>((const TI*)x, (TO*)y, n); break;
    default: return fail(TL_B200_EINVAL, "unary: unknown op %d", op);
  }
  TL_LAUNCH_CHECK("unary_kernel");
  return TL_B200_OK;
}

template <typename TI>
static int unary_out(const void* x, void* y, int64_t n, int op, int out_dtype, cudaStream_t s) {
  switch (out_dtype) {
    case TL_F32: return unary_dispatch<TI, float>(x, y, n, op, s);
    case TL_F16: return unary_dispatch<TI, __half>(x, y, n, op, s);
    case TL_BF16: return unary_dispatch<TI, __nv_bfloat16>(x, y, n, op, s);
    default: return fail(TL_B200_EINVAL, "unary: unsupported output dtype %d", out_dtype);
  }
}

template <typename T, int OP>
static int binary_mode(const void* a, const void* b, void* o, int64_t n, int64_t cols, int b_mode, float sc,
                       cudaStream_t s) {
  if constexpr (std::is_same<T, float>::value) {
    if ((b_mode == 0 || b_mode == 2) && n % 4 == 0 && aligned16(a) && aligned16(o) && (b_mode == 2 || aligned16(b))) {
      const int64_t n4 = n / 4;
      unsigned vgrid = elementwise_grid(n4, kThreads * 2);
      if (b_mode == 0)
        binary_vec_kernel<OP, false><<<vgrid, kThreads, 0, s>>>((const float4*)a, (const float4*)b, (float4*)o, n4, sc);
      else
        binary_vec_kernel<OP, true><<<vgrid, kThreads, 0, s>>>((const float4*)a, nullptr, (float4*)o, n4, sc);
      TL_LAUNCH_CHECK("binary_vec_kernel");
      return TL_B200_OK;
    }
  }
  unsigned grid = elementwise_grid(n, kThreads * 4);
  switch (b_mode) {
    case 0: binary_kernel<T, OP, 0><<<grid, kThreads, 0, s>>>((const T*)a, (const T*)b, (T*)o, n, cols, sc); break;
    case 1: binary_kernel<T, OP, 1><<<grid, kThreads, 0, s>>>((const T*)a, (const T*)b, (T*)o, n, cols, sc); break;
    case 2: binary_kernel<T, OP, 2><<<grid, kThreads, 0, s>>>((const T*)a, (const T*)b, (T*)o, n, cols, sc); break;
    case 3: binary_kernel<T, OP, 3><<<grid, kThreads, 0, s>>>((const T*)a, (const T*)b, (T*)o, n, cols, sc); break;
    default: return fail(TL_B200_EINVAL, "binary: unknown b_mode %d", b_mode);
  }
  TL_LAUNCH_CHECK("binary_kernel");
  return TL_B200_OK;
}

template <typename T>
static int binary_op(const void* a, const void* b, void* o, int64_t n, int64_t cols, int op, int b_mode,
                     float sc, cudaStream_t s) {
  switch (op) {
    case 0: return binary_mode<T, 0>(a, b, o, n, cols, b_mode, sc, s);
    case 1: return binary_mode<T, 1>(a, b, o, n, cols, b_mode, sc, s);
    case 2: return binary_mode<T, 2>(a, b, o, n, cols, b_mode, sc, s);
    case 3: return binary_mode<T, 3>(a, b, o, n, cols, b_mode, sc, s);
    case 4: return binary_mode<T, 4>(a, b, o, n, cols, b_mode, sc, s);
    default: return fail(TL_B200_EINVAL, "binary: unknown op %d", op);
  }
}

}  // namespace tl

using namespace tl;

#define TL_FLOAT_DISPATCH(dtype, CALL)                                         \
  switch (dtype) {                                                             \
    case TL_F32: { using T = float; return CALL; }                             \
    case TL_F16: { using T = __half; return CALL; }                            \
    case TL_BF16: { using T = __nv_bfloat16; return CALL; }                    \
    default: return fail(TL_B200_EINVAL, "%s: unsupported dtype %d", __func__, dtype); \
  }

extern "C" {

int tl_b200_rmsnorm(const void* x, const void* weight, void* y, int64_t rows, int64_t cols, float eps,
                    int dtype, void* stream) {
  TL_REQUIRE(rows >= 0 && cols >= 0, "rmsnorm: negative size");
  if (rows == 0 || cols == 0) return TL_B200_OK;
  TL_REQUIRE(x && y, "rmsnorm: null tensor pointer");
  cudaStream_t s = (cudaStream_t)stream;
  TL_FLOAT_DISPATCH(dtype, rmsnorm_dispatch<T>(x, weight, y, rows, cols, eps, s));
}

int tl_b200_rope(const void* x, const void* cos_tab, const void* sin_tab, void* out, int64_t rows,
                 int64_t width, int64_t rows_per_table_row, int dtype, void* stream) {
  TL_REQUIRE(rows >= 0 && width >= 0, "rope: negative size");
  TL_REQUIRE(width % 2 == 0, "rope: width %lld must be even", (long long)width);
  TL_REQUIRE(rows_per_table_row >= 1, "rope: rows_per_table_row must be >= 1");
  if (rows == 0 || width == 0) return TL_B200_OK;
  TL_REQUIRE(x && cos_tab && sin_tab && out, "rope: null tensor pointer");
  cudaStream_t s = (cudaStream_t)stream;
  TL_FLOAT_DISPATCH(dtype, rope_dispatch<T>(x, cos_tab, sin_tab, out, rows, width, rows_per_table_row, s));
}

int tl_b200_swiglu(const void* gate, const void* up, void* out, int64_t n_elems, int dtype, void* stream) {
  TL_REQUIRE(n_elems >= 0, "swiglu: negative size");
  if (n_elems == 0) return TL_B200_OK;
  TL_REQUIRE(gate && up && out, "swiglu: null tensor pointer");
  cudaStream_t s = (cudaStream_t)stream;
  TL_FLOAT_DISPATCH(dtype, swiglu_dispatch<T>(gate, up, out, n_elems, s));
}

int tl_b200_reduce_rows(const void* x, void* y, int64_t rows, int64_t cols, int op, int dtype, void* stream) {
  TL_REQUIRE(rows >= 0 && cols >= 0, "reduce_rows: negative size");
  TL_REQUIRE(op == 0 || op == 1, "reduce_rows: op must be 0 (sum) or 1 (max)");
  if (rows == 0) return TL_B200_OK;
  TL_REQUIRE(x && y, "reduce_rows: null tensor pointer");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TL_I32 || dtype == TL_U32 || dtype == TL_I16) {
    TL_REQUIRE(op == 0, "reduce_rows: integer tiles support the sum only (as ppl_reduce_sum does)");
    if (dtype == TL_I16) return reduce_sum_int<int16_t>(x, y, rows, cols, s);
    return reduce_sum_int<uint32_t>(x, y, rows, cols, s);
  }
  if (op == 0) { TL_FLOAT_DISPATCH(dtype, (reduce_dispatch<T, false>(x, y, rows, cols, s))); }
  TL_FLOAT_DISPATCH(dtype, (reduce_dispatch<T, true>(x, y, rows, cols, s)));
}

int tl_b200_unary(const void* x, void* y, int64_t n_elems, int op, int in_dtype, int out_dtype, void* stream) {
  TL_REQUIRE(n_elems >= 0, "unary: negative size");
  if (n_elems == 0) return TL_B200_OK;
  TL_REQUIRE(x && y, "unary: null tensor pointer");
  cudaStream_t s = (cudaStream_t)stream;
  TL_FLOAT_DISPATCH(in_dtype, unary_out<T>(x, y, n_elems, op, out_dtype, s));
}

int tl_b200_rope_add(void* out, const void* even1, const void* even2, const void* odd1, const void* odd2, int64_t rows,
                     int64_t cols, int dtype, void* stream) {
  TL_REQUIRE(rows >= 0 && cols >= 0, "rope_add: negative size");
  TL_REQUIRE(cols % 2 == 0, "rope_add: the row length %lld must be even", (long long)cols);
  if (rows == 0 || cols == 0) return TL_B200_OK;
  TL_REQUIRE(out && even1 && even2 && odd1 && odd2, "rope_add: null tensor pointer");
  cudaStream_t s = (cudaStream_t)stream;
  TL_FLOAT_DISPATCH(dtype, rope_add_launch<T>(out, even1, even2, odd1, odd2, rows * cols / 2, s));
}

int tl_b200_copy2d(const void* src, void* dst, int64_t rows, int64_t cols, int64_t src_ld, int64_t dst_ld, int src_dtype,
                   int dst_dtype, void* stream) {
  TL_REQUIRE(rows >= 0 && cols >= 0, "copy2d: negative size");
  if (rows == 0 || cols == 0) return TL_B200_OK;
  TL_REQUIRE(src && dst, "copy2d: null tensor pointer");
  TL_REQUIRE(src_ld >= cols && dst_ld >= cols, "copy2d: a leading dimension is smaller than the row length");
  cudaStream_t s = (cudaStream_t)stream;
  if ((src_dtype == TL_I32 || src_dtype == TL_U32) && (dst_dtype == TL_I32 || dst_dtype == TL_U32)) {   // index tiles: bits
    copy2d_kernel<uint32_t, uint32_t><<<grid2d(rows, cols), kThreads, 0, s>>>(
        (const uint32_t*)src, (uint32_t*)dst, rows, cols, src_ld, dst_ld);
    TL_LAUNCH_CHECK("copy2d_kernel");
    return TL_B200_OK;
  }
  TL_FLOAT_DISPATCH(src_dtype, copy2d_out<T>(src, dst, rows, cols, src_ld, dst_ld, dst_dtype, s));
}

int tl_b200_fill(void* dst, int64_t rows, int64_t cols, int64_t ld, float value, int dtype, void* stream) {
  TL_REQUIRE(rows >= 0 && cols >= 0, "fill: negative size");
  if (rows == 0 || cols == 0) return TL_B200_OK;
  TL_REQUIRE(dst, "fill: null tensor pointer");
  TL_REQUIRE(ld >= cols, "fill: the leading dimension is smaller than the row length");
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid = grid2d(rows, cols);
  switch (dtype) {
    case TL_F32: fill2d_kernel<float><<<grid, kThreads, 0, s>>>((float*)dst, rows, cols, ld, value); break;
    case TL_F16: fill2d_kernel<__half><<<grid, kThreads, 0, s>>>((__half*)dst, rows, cols, ld, __float2half_rn(value)); break;
    case TL_BF16:
      fill2d_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>((__nv_bfloat16*)dst, rows, cols, ld, __float2bfloat16_rn(value));
      break;
    default: return fail(TL_B200_EINVAL, "fill: unsupported dtype %d", dtype);
  }
  TL_LAUNCH_CHECK("fill2d_kernel");
  return TL_B200_OK;
}

int tl_b200_binary(const void* a, const void* b, void* out, int64_t rows, int64_t cols, int op, int b_mode,
                   float scalar, int dtype, void* stream) {
  TL_REQUIRE(rows >= 0 && cols >= 0, "binary: negative size");
  if (rows == 0 || cols == 0) return TL_B200_OK;
  TL_REQUIRE(a && out && (b || b_mode == 2), "binary: null tensor pointer");
  cudaStream_t s = (cudaStream_t)stream;
  TL_FLOAT_DISPATCH(dtype, binary_op<T>(a, b, out, rows * cols, cols, op, b_mode, scalar, s));
}

}  // extern "C"
