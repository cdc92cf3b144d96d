// The generic entry point: one symbol with the `void**` shape of the reference's generated
// `extern "C" int tilelang_tpu_run(void** args)` (src/tl_templates/tpu/main_template.cpp:39), so a
// reference-side binding can keep a single ctypes prototype.  The generated symbol has the sizes of
// its program baked in; this library is pre-built, so the sizes travel in `meta`.
#include "common.cuh"

namespace {
inline float meta_f32(int64_t v) {          // a float travels as its IEEE-754 bit pattern in the low 32 bits
  uint32_t bits = (uint32_t)(uint64_t)v;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
}  // namespace

#include <string.h>

extern "C" int tl_b200_run(int kernel_id, void** a, const int64_t* m, void* stream) {
  TL_REQUIRE(a != nullptr && m != nullptr, "tl_b200_run: null args / meta");
  switch (kernel_id) {
    case TL_B200_K_RMSNORM:
      return tl_b200_rmsnorm(a[0], a[1], a[2], m[0], m[1], meta_f32(m[2]), (int)m[3], stream);
    case TL_B200_K_ROPE:
      return tl_b200_rope(a[0], a[1], a[2], a[3], m[0], m[1], m[2], (int)m[3], stream);
    case TL_B200_K_SWIGLU:
      return tl_b200_swiglu(a[0], a[1], a[2], m[0], (int)m[1], stream);
    case TL_B200_K_REDUCE_ROWS:
      return tl_b200_reduce_rows(a[0], a[1], m[0], m[1], (int)m[2], (int)m[3], stream);
    case TL_B200_K_UNARY:
      return tl_b200_unary(a[0], a[1], m[0], (int)m[1], (int)m[2], (int)m[3], stream);
    case TL_B200_K_BINARY:
      return tl_b200_binary(a[0], a[1], a[2], m[0], m[1], (int)m[2], (int)m[3], meta_f32(m[4]), (int)m[5], stream);
    case TL_B200_K_ROPE_ADD:
      return tl_b200_rope_add(a[0], a[1], a[2], a[3], a[4], m[0], m[1], (int)m[2], stream);
    case TL_B200_K_COPY2D:
      return tl_b200_copy2d(a[0], a[1], m[0], m[1], m[2], m[3], (int)m[4], (int)m[5], stream);
    case TL_B200_K_FILL:
      return tl_b200_fill(a[0], m[0], m[1], m[2], meta_f32(m[3]), (int)m[4], stream);
    case TL_B200_K_GATHER_ROWS:
      return tl_b200_gather_rows(a[0], (const uint32_t*)a[1], a[2], m[0], m[1], m[2], stream);
    case TL_B200_K_TOPK:
      return tl_b200_topk(a[0], a[1], (int32_t*)a[2], m[0], m[1], (int)m[2], (int)m[3], m[4], (int)m[5], stream);
    case TL_B200_K_GEMM:
      return tl_b200_gemm(a[0], a[1], a[2], m[0], m[1], m[2], (int)m[3], (int)m[4], (int)m[5], stream);
    case TL_B200_K_MLP_GATE_UP:
      return tl_b200_mlp_gate_up(a[0], a[1], a[2], a[3], m[0], m[1], m[2], (int)m[3], stream);
    case TL_B200_K_GEMM_FP8_BLOCKSCALE:
      return tl_b200_gemm_fp8_blockscale(a[0], a[1], (const float*)a[2], (const float*)a[3], a[4], m[0], m[1], m[2],
                                         (int)m[3], stream);
    case TL_B200_K_FLASH_ATTN_FWD:
      return tl_b200_flash_attn_fwd(a[0], a[1], a[2], a[3], m[0], m[1], m[2], m[3], m[4], meta_f32(m[5]), (int)m[6],
                                    (int)m[7], (int)m[8], (int)m[9], stream);
    case TL_B200_K_MLA_DECODE_DENSE:
      return tl_b200_mla_decode_dense(a[0], a[1], a[2], a[3], a[4], m[0], m[1], m[2], m[3], m[4], meta_f32(m[5]),
                                      (int)m[6], stream);
    case TL_B200_K_MLA_DECODE_PAGED:
      return tl_b200_mla_decode_paged(a[0], a[1], (const float*)a[2], (const int32_t*)a[3], (const int32_t*)a[4], a[5],
                                      m[0], m[1], m[2], m[3], m[4], m[5], m[6], meta_f32(m[7]), (int)m[8], (int)m[9],
                                      a[6], m[10], stream);
    default:
      return ::tl::fail(TL_B200_EINVAL, "tl_b200_run: unknown kernel id %d", kernel_id);
  }
}
