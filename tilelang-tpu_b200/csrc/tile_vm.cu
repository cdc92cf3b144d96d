// Fused execution of row-local tile programs.
//
// A `ppl_*` program whose every op works row by row (loads, stores and casts, fill, add / sub / mul / div with a
// full, (M,1) or (1,N) second operand, mul_C / add_C, exp, sigmoid, rsqrt, row sum / max, rope_add) needs no
// tile ever to exist in memory: one row of every tile fits in the registers of the threads that own the row.
// The host side (tilelang/engine/fuser.py) turns such a program into a short list of instructions for a small
// accumulator machine, and this kernel runs the whole program - every block of the launch grid, every row of a
// block - in ONE launch: a group of TPR threads owns a row, holds NT tile registers of EPT elements per thread
// plus an accumulator, eight per-row scalars (the (M,1) tiles), and walks the instruction list.  Every global
// element is read once and written once, with 16-byte accesses where alignment allows.
//
// The reference runs such a program as one runtime call per tile op on one TPU core
// (src/target/codegen_ppl.cc:879-1906); arithmetic follows the same rules here: fp32 evaluation, results rounded
// to the destination tile's type (round-to-nearest-even), scalar operands first cast to the tile's type.
#include "common.cuh"

namespace tl {

constexpr int kVmMaxInstr = TL_B200_VM_MAX_INSTR;
constexpr int kVmMaxParams = TL_B200_VM_MAX_PARAMS;
constexpr int kVmScalars = 8;
constexpr int kVmThreads = 256;

struct VmProgram {
  tl_b200_vm_instr ins[kVmMaxInstr];
  void* params[kVmMaxParams];
  int n_instr;
  int grid_x, grid_y, grid_z;
  int rows_per_block;
  long long total_rows;
};

__device__ __forceinline__ float vm_round(float v, int dtype) {
  if (dtype == TL_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  if (dtype == TL_F16) return __half2float(__float2half_rn(v));
  return v;
}
__device__ __forceinline__ float vm_binary(float a, float b, int sub) {
  switch (sub) {
    case 0: return a + b;
    case 1: return a - b;
    case 2: return a * b;
    case 3: return __fdividef(a, b);        // 2 ulp; the reference's division is a table + polynomial routine
    default: return fmaxf(a, b);
  }
}
__device__ __forceinline__ float vm_unary(float a, int sub) {
  switch (sub) {
    // ex2-based exponential: error 2 + |1.16 a| ulp, inside the 1e-5 of the fp32 path up to the overflow of exp
    case 0: return __fdividef(1.0f, 1.0f + __expf(-a));
    case 1: return __expf(a);
    default: return rsqrtf(a);
  }
}
__device__ __forceinline__ float vm_load(const void* base, long long idx, int dtype) {
  switch (dtype) {
    case TL_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
    case TL_F16: return __half2float(reinterpret_cast<const __half*>(base)[idx]);
    default: return reinterpret_cast<const float*>(base)[idx];
  }
}
__device__ __forceinline__ void vm_store(void* base, long long idx, int dtype, float v) {
  switch (dtype) {
    case TL_BF16: reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v); break;
    case TL_F16: reinterpret_cast<__half*>(base)[idx] = __float2half_rn(v); break;
    default: reinterpret_cast<float*>(base)[idx] = v;
  }
}

// Column of element e of a thread: chunks of 8 consecutive columns, dealt round-robin to the TPR threads of a row.
template <int TPR> __device__ __forceinline__ int vm_col(int t, int e) { return ((e >> 3) * TPR + t) * 8 + (e & 7); }

template <int TPR, int EPT, int NT>
__global__ void __launch_bounds__(kVmThreads, (NT * EPT <= 64) ? 2 : 1)
tile_vm_kernel(const __grid_constant__ VmProgram prog) {
  constexpr int G = kVmThreads / TPR;              // rows in flight per CTA
  __shared__ float red[kVmThreads / 32];
  const int t = threadIdx.x % TPR, group = threadIdx.x / TPR;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float T[NT][EPT];
  float A[EPT];
  float S[kVmScalars];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int e = 0; e < EPT; ++e) T[i][e] = 0.f;
#pragma unroll
  for (int e = 0; e < EPT; ++e) A[e] = 0.f;
#pragma unroll
  for (int j = 0; j < kVmScalars; ++j) S[j] = 0.f;

// run BODY with Treg bound to tile register number `idx` (static indexing keeps the registers in registers)
#define VM_WITH_TILE(idx, BODY)                                  \
  switch (idx) {                                                 \
    case 0: { float(&Treg)[EPT] = T[0]; BODY } break;            \
    case 1: { float(&Treg)[EPT] = T[1 % NT]; BODY } break;       \
    case 2: { float(&Treg)[EPT] = T[2 % NT]; BODY } break;       \
    case 3: { float(&Treg)[EPT] = T[3 % NT]; BODY } break;       \
    case 4: { float(&Treg)[EPT] = T[4 % NT]; BODY } break;       \
    case 5: { float(&Treg)[EPT] = T[5 % NT]; BODY } break;       \
    case 6: { float(&Treg)[EPT] = T[6 % NT]; BODY } break;       \
    default: { float(&Treg)[EPT] = T[7 % NT]; BODY } break;      \
  }
#define VM_SCALAR(idx) S[(idx) & (kVmScalars - 1)]

  for (long long unit0 = (long long)blockIdx.x * G; unit0 < prog.total_rows; unit0 += (long long)gridDim.x * G) {
    const long long unit = unit0 + group;
    const bool live = unit < prog.total_rows;
    const long long blk = live ? unit / prog.rows_per_block : 0;
    const int r = live ? (int)(unit - blk * prog.rows_per_block) : 0;
    const int bx = (int)(blk % prog.grid_x), by = (int)((blk / prog.grid_x) % prog.grid_y);
    const int bz = (int)(blk / ((long long)prog.grid_x * prog.grid_y));
#pragma unroll 1
    for (int pc = 0; pc < prog.n_instr; ++pc) {
      const tl_b200_vm_instr& in = prog.ins[pc];
      const int op = in.op;
      if (op == TL_VM_LD_A || op == TL_VM_ST_A || op == TL_VM_LD_S || op == TL_VM_ST_S) {
        const long long off = in.base + in.coef[0] * bx + in.coef[1] * by + in.coef[2] * bz + (long long)r * in.row_stride;
        char* base = reinterpret_cast<char*>(prog.params[in.param]);
        if (op == TL_VM_LD_S) {
          VM_SCALAR(in.r0) = live ? vm_load(base, off, in.dtype) : 0.f;
        } else if (op == TL_VM_ST_S) {
          if (live && t == 0) vm_store(base, off, in.dtype, VM_SCALAR(in.r0));
        } else {
          const int esz = in.dtype == TL_F32 ? 4 : 2;
          // 16-byte (16-bit types) or 32-byte-as-two-16-byte (fp32) accesses when every chunk of 8 is aligned
          const bool vec = in.vec != 0;
#pragma unroll
          for (int c8 = 0; c8 < EPT / 8; ++c8) {
            const int col = (c8 * TPR + t) * 8;
            if (!live || col >= in.width) {
              if (op == TL_VM_LD_A) {
#pragma unroll
                for (int e = 0; e < 8; ++e) A[c8 * 8 + e] = 0.f;
              }
              continue;
            }
            char* p = base + (off + col) * esz;
            if (vec && col + 8 <= in.width) {
              if (op == TL_VM_LD_A) {
                if (esz == 2) {
                  const uint4 raw = *reinterpret_cast<const uint4*>(p);
                  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    if (in.dtype == TL_BF16) {
                      A[c8 * 8 + 2 * e] = __uint_as_float(w[e] << 16);
                      A[c8 * 8 + 2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
                    } else {
                      const __half2 h = *reinterpret_cast<const __half2*>(&w[e]);
                      A[c8 * 8 + 2 * e] = __low2float(h);
                      A[c8 * 8 + 2 * e + 1] = __high2float(h);
                    }
                  }
                } else {
                  const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 16);
                  A[c8 * 8] = lo.x; A[c8 * 8 + 1] = lo.y; A[c8 * 8 + 2] = lo.z; A[c8 * 8 + 3] = lo.w;
                  A[c8 * 8 + 4] = hi.x; A[c8 * 8 + 5] = hi.y; A[c8 * 8 + 6] = hi.z; A[c8 * 8 + 7] = hi.w;
                }
              } else {
                if (esz == 2) {
                  uint32_t w[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    if (in.dtype == TL_BF16) {
                      const __nv_bfloat162 h = __floats2bfloat162_rn(A[c8 * 8 + 2 * e], A[c8 * 8 + 2 * e + 1]);
                      w[e] = *reinterpret_cast<const uint32_t*>(&h);
                    } else {
                      const __half2 h = __floats2half2_rn(A[c8 * 8 + 2 * e], A[c8 * 8 + 2 * e + 1]);
                      w[e] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                  }
                  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
                } else {
                  *reinterpret_cast<float4*>(p) = make_float4(A[c8 * 8], A[c8 * 8 + 1], A[c8 * 8 + 2], A[c8 * 8 + 3]);
                  *reinterpret_cast<float4*>(p + 16) = make_float4(A[c8 * 8 + 4], A[c8 * 8 + 5], A[c8 * 8 + 6], A[c8 * 8 + 7]);
                }
              }
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const bool in_row = col + e < in.width;
                if (op == TL_VM_LD_A) A[c8 * 8 + e] = in_row ? vm_load(base, off + col + e, in.dtype) : 0.f;
                else if (in_row) vm_store(base, off + col + e, in.dtype, A[c8 * 8 + e]);
              }
            }
          }
        }
        continue;
      }
      switch (op) {
        case TL_VM_MOV_A_T:
          VM_WITH_TILE(in.r0, {
#pragma unroll
            for (int e = 0; e < EPT; ++e) A[e] = Treg[e];
          })
          break;
        case TL_VM_MOV_T_A:
          VM_WITH_TILE(in.r0, {
#pragma unroll
            for (int e = 0; e < EPT; ++e) Treg[e] = A[e] = vm_round(A[e], in.dtype);   // A keeps the stored (rounded) row
          })
          break;
        case TL_VM_BIN_A_T:
          VM_WITH_TILE(in.r0, {
#pragma unroll
            for (int e = 0; e < EPT; ++e) A[e] = vm_binary(A[e], Treg[e], in.sub);
          })
          break;
        case TL_VM_BIN_A_S: {
          const float s = VM_SCALAR(in.r0);
#pragma unroll
          for (int e = 0; e < EPT; ++e) A[e] = vm_binary(A[e], s, in.sub);
          break;
        }
        case TL_VM_BIN_A_I:
#pragma unroll
          for (int e = 0; e < EPT; ++e) A[e] = vm_binary(A[e], in.imm, in.sub);
          break;
        case TL_VM_UN_A:
#pragma unroll
          for (int e = 0; e < EPT; ++e) A[e] = vm_unary(A[e], in.sub);
          break;
        case TL_VM_FILL_A:
#pragma unroll
          for (int e = 0; e < EPT; ++e) A[e] = in.imm;
          break;
        case TL_VM_ROUND_A:
#pragma unroll
          for (int e = 0; e < EPT; ++e) A[e] = vm_round(A[e], in.dtype);
          break;
        case TL_VM_RED_S: {
          const bool is_max = in.sub == 1;
          float acc = is_max ? -INFINITY : 0.f;
#pragma unroll
          for (int e = 0; e < EPT; ++e) {
            if (vm_col<TPR>(t, e) < in.width) acc = is_max ? fmaxf(acc, A[e]) : acc + A[e];
          }
          acc = is_max ? warp_max(acc) : warp_sum(acc);
          if constexpr (TPR > 32) {
            __syncthreads();                      // the staging array may still be read from the reduction before
            if (lane == 0) red[warp] = acc;
            __syncthreads();
            acc = is_max ? -INFINITY : 0.f;
#pragma unroll
            for (int k = 0; k < TPR / 32; ++k) {
              const float v = red[group * (TPR / 32) + k];
              acc = is_max ? fmaxf(acc, v) : acc + v;
            }
          }
          VM_SCALAR(in.r0) = vm_round(acc, in.dtype);
          break;
        }
        case TL_VM_MOV_S_I:
          VM_SCALAR(in.r0) = in.imm;
          break;
        case TL_VM_MOV_S_S:
          VM_SCALAR(in.r0) = vm_round(VM_SCALAR(in.r1), in.dtype);
          break;
        case TL_VM_BIN_S_S:
          VM_SCALAR(in.r0) = vm_round(vm_binary(VM_SCALAR(in.r1), VM_SCALAR(in.r2), in.sub), in.dtype);
          break;
        case TL_VM_BIN_S_I:
          VM_SCALAR(in.r0) = vm_round(vm_binary(VM_SCALAR(in.r1), in.imm, in.sub), in.dtype);
          break;
        case TL_VM_UN_S:
          VM_SCALAR(in.r0) = vm_round(vm_unary(VM_SCALAR(in.r1), in.sub), in.dtype);
          break;
        case TL_VM_BCAST_A_S: {
          const float s = VM_SCALAR(in.r0);
#pragma unroll
          for (int e = 0; e < EPT; ++e) A[e] = s;
          break;
        }
        case TL_VM_ROPE_A: {
          // A[2i] = E1[2i] + E2[2i+1]; A[2i+1] = O1[2i+1] + O2[2i]; a thread's elements come in aligned pairs
          float e1[EPT], e2[EPT], o1[EPT], o2[EPT];
          VM_WITH_TILE(in.r0, {
#pragma unroll
            for (int e = 0; e < EPT; ++e) e1[e] = Treg[e];
          })
          VM_WITH_TILE(in.r1, {
#pragma unroll
            for (int e = 0; e < EPT; ++e) e2[e] = Treg[e];
          })
          VM_WITH_TILE(in.r2, {
#pragma unroll
            for (int e = 0; e < EPT; ++e) o1[e] = Treg[e];
          })
          VM_WITH_TILE(in.r3, {
#pragma unroll
            for (int e = 0; e < EPT; ++e) o2[e] = Treg[e];
          })
#pragma unroll
          for (int e = 0; e < EPT; e += 2) {
            A[e] = e1[e] + e2[e + 1];
            A[e + 1] = o1[e + 1] + o2[e];
          }
          break;
        }
        default:
          break;
      }
    }
  }
#undef VM_WITH_TILE
#undef VM_SCALAR
}

template <int TPR, int EPT, int NT>
static int launch_vm(const VmProgram& prog, cudaStream_t s) {
  constexpr int G = kVmThreads / TPR;
  long long ctas = (prog.total_rows + G - 1) / G;
  const long long cap = (long long)sm_count() * 8;
  if (ctas > cap) ctas = cap;
  tile_vm_kernel<TPR, EPT, NT><<<(unsigned)ctas, kVmThreads, 0, s>>>(prog);
  TL_LAUNCH_CHECK("tile_vm_kernel");
  return TL_B200_OK;
}

}  // namespace tl

using namespace tl;

extern "C" int tl_b200_tile_program_registers(int64_t max_width) {
  if (max_width <= 0 || max_width > 8192) return 0;
  return max_width > 4096 ? 4 : 8;
}

extern "C" int tl_b200_tile_program(const tl_b200_vm_instr* instrs, int n_instr, const void* const* params, int n_params,
                                    int grid_x, int grid_y, int grid_z, int rows_per_block, int64_t max_width,
                                    void* stream) {
  int highest_tile = -1;
  TL_REQUIRE(instrs && n_instr > 0 && n_instr <= kVmMaxInstr, "tile_program: 1..%d instructions", kVmMaxInstr);
  TL_REQUIRE(n_params >= 0 && n_params <= kVmMaxParams && (params || n_params == 0), "tile_program: at most %d parameters",
             kVmMaxParams);
  TL_REQUIRE(grid_x > 0 && grid_y > 0 && grid_z > 0 && rows_per_block > 0, "tile_program: empty grid");
  TL_REQUIRE(max_width > 0 && max_width <= 8192, "tile_program: tile width %lld outside 1..8192", (long long)max_width);
  const int nt = tl_b200_tile_program_registers(max_width);
  VmProgram prog;
  for (int i = 0; i < n_instr; ++i) {
    const tl_b200_vm_instr& in = instrs[i];
    TL_REQUIRE(in.op >= 0 && in.op < TL_VM_OPCODES, "tile_program: instruction %d has unknown opcode %d", i, in.op);
    const bool mem = in.op == TL_VM_LD_A || in.op == TL_VM_ST_A || in.op == TL_VM_LD_S || in.op == TL_VM_ST_S;
    if (mem) {
      TL_REQUIRE(in.param >= 0 && in.param < n_params && params[in.param], "tile_program: instruction %d names parameter %d", i, in.param);
      TL_REQUIRE(in.dtype == TL_F32 || in.dtype == TL_F16 || in.dtype == TL_BF16, "tile_program: instruction %d: float tensors only", i);
      TL_REQUIRE(in.width >= 0 && in.width <= max_width, "tile_program: instruction %d: width %d", i, in.width);
    }
    const bool tile_reg = in.op == TL_VM_MOV_A_T || in.op == TL_VM_MOV_T_A || in.op == TL_VM_BIN_A_T;
    if (tile_reg) TL_REQUIRE(in.r0 >= 0 && in.r0 < nt, "tile_program: instruction %d uses tile register %d of %d", i, in.r0, nt);
    if (tile_reg && in.r0 > highest_tile) highest_tile = in.r0;
    if (in.op == TL_VM_ROPE_A) {
      const int m4 = in.r0 > in.r1 ? in.r0 : in.r1, m5 = in.r2 > in.r3 ? in.r2 : in.r3;
      if ((m4 > m5 ? m4 : m5) > highest_tile) highest_tile = m4 > m5 ? m4 : m5;
    }
    if (in.op == TL_VM_ROPE_A)
      TL_REQUIRE(in.r0 >= 0 && in.r0 < nt && in.r1 >= 0 && in.r1 < nt && in.r2 >= 0 && in.r2 < nt && in.r3 >= 0 && in.r3 < nt,
                 "tile_program: instruction %d uses a tile register outside 0..%d", i, nt - 1);
    prog.ins[i] = in;
  }
  for (int i = 0; i < n_params; ++i) prog.params[i] = const_cast<void*>(params[i]);
  prog.n_instr = n_instr;
  prog.grid_x = grid_x; prog.grid_y = grid_y; prog.grid_z = grid_z;
  prog.rows_per_block = rows_per_block;
  prog.total_rows = (long long)grid_x * grid_y * grid_z * rows_per_block;
  cudaStream_t s = (cudaStream_t)stream;
  // a program that needs at most four tile registers runs the variant with half the registers (two CTAs per SM)
  const bool few = highest_tile < 4;
  if (max_width <= 256) return few ? launch_vm<32, 8, 4>(prog, s) : launch_vm<32, 8, 8>(prog, s);
  if (max_width <= 512) return few ? launch_vm<32, 16, 4>(prog, s) : launch_vm<32, 16, 8>(prog, s);
  if (max_width <= 2048) return few ? launch_vm<256, 8, 4>(prog, s) : launch_vm<256, 8, 8>(prog, s);
  if (max_width <= 4096) return few ? launch_vm<256, 16, 4>(prog, s) : launch_vm<256, 16, 8>(prog, s);
  return launch_vm<256, 32, 4>(prog, s);
}
