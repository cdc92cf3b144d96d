"""Generated kernels for row-local tile programs.

`fuser.py` lowers a row-local `ppl_*` program to the instruction list of the accumulator machine of
csrc/tile_vm.cu.  That kernel interprets the list (a switch per instruction, a loop over the register elements
behind it), which removes the launches and HBM round trips of the op-by-op executor but leaves it issue-bound.
Here the same list is printed as straight-line CUDA C with every constant of the program in place (opcodes,
operand registers, immediates, tile widths, types, the launch grid), compiled for sm_100a with NVRTC and launched
through the driver API: one generated kernel per program, as the reference generates one `kernel.c` per program
(src/target/codegen_ppl.cc:2180-2307) and builds it at compile time (tilelang/jit/adapter/libgen.py:345-415).

The arithmetic is the interpreter's, statement for statement (fp32 evaluation, every result rounded to its tile's
type, `--fmad=false` so that no two tile ops are contracted into one rounding): both paths give the same bits, and
the interpreter stays the path taken when NVRTC is not there.  Compiled code is cached on disk by the hash of its
source.
"""
from __future__ import annotations

import ctypes
import hashlib
import struct
from typing import Callable, Dict, List, Optional

from ..cache import cache_dir, is_cache_enabled
from . import fuser as F

_HEADER = r'''
typedef unsigned int u32;
typedef unsigned short u16;
typedef long long i64;
#define INFINITY __int_as_float(0x7f800000)
struct Params { void* p[16]; u32 vec; u32 pad; };

__device__ __forceinline__ float bf2f(u16 b) { return __uint_as_float(((u32)b) << 16); }
__device__ __forceinline__ u16 f2bf(float v) { u16 r; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(v)); return r; }
__device__ __forceinline__ float h2f(u16 b) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(b)); return f; }
__device__ __forceinline__ u16 f2h(float v) { u16 r; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(r) : "f"(v)); return r; }
// type codes: 0 float32, 1 float16, 2 bfloat16
template <int DT> __device__ __forceinline__ float rnd(float v) {
  if (DT == 2) return bf2f(f2bf(v));
  if (DT == 1) return h2f(f2h(v));
  return v;
}
template <int DT> __device__ __forceinline__ float ld1(const void* base, i64 i) {
  if (DT == 2) return bf2f(((const u16*)base)[i]);
  if (DT == 1) return h2f(((const u16*)base)[i]);
  return ((const float*)base)[i];
}
template <int DT> __device__ __forceinline__ void st1(void* base, i64 i, float v) {
  if (DT == 2) ((u16*)base)[i] = f2bf(v);
  else if (DT == 1) ((u16*)base)[i] = f2h(v);
  else ((float*)base)[i] = v;
}
template <int SUB> __device__ __forceinline__ float bin(float a, float b) {
  if (SUB == 0) return a + b;
  if (SUB == 1) return a - b;
  if (SUB == 2) return a * b;
  if (SUB == 3) return __fdividef(a, b);
  return fmaxf(a, b);
}
template <int SUB> __device__ __forceinline__ float un(float a) {
  if (SUB == 0) return __fdividef(1.0f, 1.0f + __expf(-a));
  if (SUB == 1) return __expf(a);
  return rsqrtf(a);
}
__device__ __forceinline__ float warp_sum(float v) {
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
  for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}
// Columns of a thread: chunks of 8 consecutive columns, dealt round-robin to the TPR threads of a row.
template <int TPR, int EPT, int DT>
__device__ __forceinline__ void ld_a(float (&A)[EPT], const char* base, i64 off, int width, bool vec, bool live, int t) {
  constexpr int ESZ = DT == 0 ? 4 : 2;
#pragma unroll
  for (int c8 = 0; c8 < EPT / 8; ++c8) {
    const int col = (c8 * TPR + t) * 8;
    if (!live || col >= width) {
#pragma unroll
      for (int e = 0; e < 8; ++e) A[c8 * 8 + e] = 0.f;
      continue;
    }
    const char* p = base + (off + col) * ESZ;
    if (vec && col + 8 <= width) {
      if (ESZ == 2) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const u32 w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (DT == 2) {
            A[c8 * 8 + 2 * e] = __uint_as_float(w[e] << 16);
            A[c8 * 8 + 2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
          } else {
            A[c8 * 8 + 2 * e] = h2f((u16)(w[e] & 0xffffu));
            A[c8 * 8 + 2 * e + 1] = h2f((u16)(w[e] >> 16));
          }
        }
      } else {
        const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 16);
        A[c8 * 8] = lo.x; A[c8 * 8 + 1] = lo.y; A[c8 * 8 + 2] = lo.z; A[c8 * 8 + 3] = lo.w;
        A[c8 * 8 + 4] = hi.x; A[c8 * 8 + 5] = hi.y; A[c8 * 8 + 6] = hi.z; A[c8 * 8 + 7] = hi.w;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) A[c8 * 8 + e] = col + e < width ? ld1<DT>(base, off + col + e) : 0.f;
    }
  }
}
template <int TPR, int EPT, int DT>
__device__ __forceinline__ void st_a(const float (&A)[EPT], char* base, i64 off, int width, bool vec, bool live, int t) {
  constexpr int ESZ = DT == 0 ? 4 : 2;
#pragma unroll
  for (int c8 = 0; c8 < EPT / 8; ++c8) {
    const int col = (c8 * TPR + t) * 8;
    if (!live || col >= width) continue;
    char* p = base + (off + col) * ESZ;
    if (vec && col + 8 <= width) {
      if (ESZ == 2) {
        u32 w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = A[c8 * 8 + 2 * e], hi = A[c8 * 8 + 2 * e + 1];
          if (DT == 2) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w[e]) : "f"(hi), "f"(lo));
          else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(w[e]) : "f"(hi), "f"(lo));
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
      } else {
        *reinterpret_cast<float4*>(p) = make_float4(A[c8 * 8], A[c8 * 8 + 1], A[c8 * 8 + 2], A[c8 * 8 + 3]);
        *reinterpret_cast<float4*>(p + 16) = make_float4(A[c8 * 8 + 4], A[c8 * 8 + 5], A[c8 * 8 + 6], A[c8 * 8 + 7]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (col + e < width) st1<DT>(base, off + col + e, A[c8 * 8 + e]);
    }
  }
}
// Row sum (IS_MAX = 0) or maximum over the first `width` columns; every thread of the row's group gets the result.
template <int TPR, int EPT, int IS_MAX>
__device__ __forceinline__ float red_row(const float (&A)[EPT], int width, int t, int lane, int warp, int group, float* red) {
  float acc = IS_MAX ? -INFINITY : 0.f;
#pragma unroll
  for (int e = 0; e < EPT; ++e) {
    const int col = ((e >> 3) * TPR + t) * 8 + (e & 7);
    if (col < width) acc = IS_MAX ? fmaxf(acc, A[e]) : acc + A[e];
  }
  acc = IS_MAX ? warp_max(acc) : warp_sum(acc);
  if (TPR > 32) {
    __syncthreads();                      // the staging array may still be read from the reduction before
    if (lane == 0) red[warp] = acc;
    __syncthreads();
    acc = IS_MAX ? -INFINITY : 0.f;
#pragma unroll
    for (int k = 0; k < TPR / 32; ++k) {
      const float v = red[group * (TPR / 32) + k];
      acc = IS_MAX ? fmaxf(acc, v) : acc + v;
    }
  }
  return acc;
}
'''

THREADS = 256


def _shape(max_width: int):
    """(threads per row, elements per thread): the split of tile_vm.cu."""
    if max_width <= 256:
        return 32, 8
    if max_width <= 512:
        return 32, 16
    if max_width <= 2048:
        return 256, 8
    if max_width <= 4096:
        return 256, 16
    return 256, 32


def _f(x: float) -> str:
    """A float immediate with its exact bits."""
    bits = struct.unpack("<I", struct.pack("<f", float(x)))[0]
    return f"__uint_as_float(0x{bits:08x}u)"


def generate(ins: List[F.Instr], grid, rows_per_block: int, max_width: int) -> str:
    """CUDA C of one program: the instruction list, instruction by instruction, inside the row loop of tile_vm.cu."""
    tpr, ept = _shape(max_width)
    tiles = set()
    for i in ins:
        if i.op in (F.MOV_A_T, F.MOV_T_A, F.BIN_A_T):
            tiles.add(i.r0)
        elif i.op == F.ROPE_A:
            tiles.update((i.r0, i.r1, i.r2, i.r3))
    nt = (max(tiles) + 1) if tiles else 0
    gx, gy, gz = (int(g) for g in grid)
    total = gx * gy * gz * int(rows_per_block)
    minb = 2 if nt * ept <= 64 else 1
    body: List[str] = []
    each = "_Pragma(\"unroll\") for (int e = 0; e < EPT; ++e)"

    def off(i):
        return (f"({i.base}ll + {i.coef[0]}ll * bx + {i.coef[1]}ll * by + {i.coef[2]}ll * bz + (i64)r * {i.row_stride})")

    for n, i in enumerate(ins):
        op, s0 = i.op, f"S{i.r0 & 7}"
        vec = f"(({i.vec} != 0) && ((prm.vec >> {i.param}) & 1u))"
        if op == F.LD_A:
            line = f"ld_a<TPR, EPT, {i.dtype}>(A, (const char*)prm.p[{i.param}], {off(i)}, {i.width}, {vec}, live, t);"
        elif op == F.ST_A:
            line = f"st_a<TPR, EPT, {i.dtype}>(A, (char*)prm.p[{i.param}], {off(i)}, {i.width}, {vec}, live, t);"
        elif op == F.LD_S:
            line = f"{s0} = live ? ld1<{i.dtype}>(prm.p[{i.param}], {off(i)}) : 0.f;"
        elif op == F.ST_S:
            line = f"if (live && t == 0) st1<{i.dtype}>(prm.p[{i.param}], {off(i)}, {s0});"
        elif op == F.MOV_A_T:
            line = f"{each} A[e] = T{i.r0}[e];"
        elif op == F.MOV_T_A:
            line = f"{each} T{i.r0}[e] = A[e] = rnd<{i.dtype}>(A[e]);"
        elif op == F.BIN_A_T:
            line = f"{each} A[e] = bin<{i.sub}>(A[e], T{i.r0}[e]);"
        elif op == F.BIN_A_S:
            line = f"{each} A[e] = bin<{i.sub}>(A[e], {s0});"
        elif op == F.BIN_A_I:
            line = f"{each} A[e] = bin<{i.sub}>(A[e], {_f(i.imm)});"
        elif op == F.UN_A:
            line = f"{each} A[e] = un<{i.sub}>(A[e]);"
        elif op == F.FILL_A:
            line = f"{each} A[e] = {_f(i.imm)};"
        elif op == F.ROUND_A:
            line = f"{each} A[e] = rnd<{i.dtype}>(A[e]);"
        elif op == F.BCAST_A_S:
            line = f"{each} A[e] = {s0};"
        elif op == F.RED_S:
            line = (f"{s0} = rnd<{i.dtype}>(red_row<TPR, EPT, {1 if i.sub == 1 else 0}>(A, {i.width}, t, lane, warp, group, red));")
        elif op == F.MOV_S_I:
            line = f"{s0} = {_f(i.imm)};"
        elif op == F.MOV_S_S:
            line = f"{s0} = rnd<{i.dtype}>(S{i.r1 & 7});"
        elif op == F.BIN_S_S:
            line = f"{s0} = rnd<{i.dtype}>(bin<{i.sub}>(S{i.r1 & 7}, S{i.r2 & 7}));"
        elif op == F.BIN_S_I:
            line = f"{s0} = rnd<{i.dtype}>(bin<{i.sub}>(S{i.r1 & 7}, {_f(i.imm)}));"
        elif op == F.UN_S:
            line = f"{s0} = rnd<{i.dtype}>(un<{i.sub}>(S{i.r1 & 7}));"
        elif op == F.ROPE_A:
            line = (f"_Pragma(\"unroll\") for (int e = 0; e < EPT; e += 2) {{ A[e] = T{i.r0}[e] + T{i.r1}[e + 1]; "
                    f"A[e + 1] = T{i.r2}[e + 1] + T{i.r3}[e]; }}")
        else:
            raise ValueError(f"instruction {n}: opcode {op}")
        body.append(f"    /* {n:2d} */ {line}")
    decl_t = "".join(f"  float T{k}[EPT];\n  _Pragma(\"unroll\") for (int e = 0; e < EPT; ++e) T{k}[e] = 0.f;\n" for k in range(nt))
    decl_s = "  float " + ", ".join(f"S{k} = 0.f" for k in range(F.SCALARS)) + ";\n"
    return (_HEADER + f"""
extern "C" __global__ void __launch_bounds__({THREADS}, {minb}) tile_program(const Params prm) {{
  constexpr int TPR = {tpr}, EPT = {ept}, G = {THREADS} / TPR;
  __shared__ float red[{THREADS} / 32];
  const int t = threadIdx.x % TPR, group = threadIdx.x / TPR, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  (void)lane; (void)warp; (void)red;
  float A[EPT];
  _Pragma("unroll") for (int e = 0; e < EPT; ++e) A[e] = 0.f;
{decl_t}{decl_s}
  for (i64 unit0 = (i64)blockIdx.x * G; unit0 < {total}ll; unit0 += (i64)gridDim.x * G) {{
    const i64 unit = unit0 + group;
    const bool live = unit < {total}ll;
    const i64 blk = live ? unit / {int(rows_per_block)} : 0;
    const int r = live ? (int)(unit - blk * {int(rows_per_block)}) : 0;
    const int bx = (int)(blk % {gx}), by = (int)((blk / {gx}) % {gy}), bz = (int)(blk / {gx * gy}ll);
    (void)bx; (void)by; (void)bz; (void)r;
""" + "\n".join(body) + """
  }
}
""")


# ------------------------------------------------------------------------------- NVRTC + driver
class Unavailable(RuntimeError):
    """NVRTC or the driver bindings cannot be used here; the caller keeps the interpreter."""


def _bindings():
    try:
        from cuda.bindings import driver, nvrtc
    except Exception as exc:                                   # pragma: no cover - depends on the installation
        raise Unavailable(f"cuda.bindings is not importable: {exc}") from exc
    return driver, nvrtc


def compile_cubin(source: str) -> bytes:
    """sm_100a code of `source` (cached on disk by the hash of the source and the NVRTC version)."""
    driver, nvrtc = _bindings()
    err, major, minor = nvrtc.nvrtcVersion()
    if int(err) != 0:
        raise Unavailable(f"nvrtcVersion failed: {err}")
    key = hashlib.sha256((f"nvrtc {major}.{minor}\n" + source).encode()).hexdigest()[:32]
    path = cache_dir() / f"gen_{key}.cubin"
    if is_cache_enabled() and path.exists():
        try:
            cached = path.read_bytes()
        except OSError:
            cached = b""
        if cached[:4] == b"\x7fELF":                          # anything else (a torn write) is compiled again
            return cached
    err, prog = nvrtc.nvrtcCreateProgram(source.encode(), b"tile_program.cu", 0, [], [])
    if int(err) != 0:
        raise Unavailable(f"nvrtcCreateProgram failed: {err}")
    opts = [b"--gpu-architecture=sm_100a", b"--fmad=false", b"-std=c++17", b"-lineinfo"]
    err, = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
    if int(err) != 0:
        _, n = nvrtc.nvrtcGetProgramLogSize(prog)
        log = b" " * n
        nvrtc.nvrtcGetProgramLog(prog, log)
        nvrtc.nvrtcDestroyProgram(prog)
        raise RuntimeError("generated tile program does not compile:\n" + log.decode(errors="replace"))
    _, n = nvrtc.nvrtcGetCUBINSize(prog)
    cubin = b" " * n
    nvrtc.nvrtcGetCUBIN(prog, cubin)
    nvrtc.nvrtcDestroyProgram(prog)
    if is_cache_enabled():
        try:
            path.parent.mkdir(parents=True, exist_ok=True)
            tmp = path.with_suffix(".tmp")
            tmp.write_bytes(cubin)
            tmp.replace(path)
        except OSError:
            pass
    return cubin


class _ParamBlock(ctypes.Structure):
    _fields_ = [("p", ctypes.c_void_p * 16), ("vec", ctypes.c_uint32), ("pad", ctypes.c_uint32)]


_functions: Dict[tuple, object] = {}          # (device index, source hash) -> CUfunction (its module is kept alive beside it)
_modules: List[object] = []


def _function(cubin: bytes, device: int):
    driver, _ = _bindings()
    key = (device, hashlib.sha256(cubin).hexdigest())
    fn = _functions.get(key)
    if fn is None:
        err, module = driver.cuModuleLoadData(cubin)
        if int(err) != 0:
            raise RuntimeError(f"cuModuleLoadData failed for a generated tile program: {err}")
        err, fn = driver.cuModuleGetFunction(module, b"tile_program")
        if int(err) != 0:
            raise RuntimeError(f"cuModuleGetFunction failed: {err}")
        _modules.append(module)
        _functions[key] = fn
    return fn


def build(ins: List[F.Instr], mem_instrs, n_params: int, grid, rows_per_block: int, max_width: int) -> Callable[..., int]:
    """run(*device_tensors) -> 0 launching the program's generated kernel; raises Unavailable without NVRTC."""
    import torch
    from .. import ops as K
    driver, _ = _bindings()
    source = generate(ins, grid, rows_per_block, max_width)
    cubin = compile_cubin(source)
    tpr, _ = _shape(max_width)
    rows_in_flight = THREADS // tpr
    total = int(grid[0]) * int(grid[1]) * int(grid[2]) * int(rows_per_block)

    def run(*tensors):
        stream = K._prepare(*tensors)
        dev = tensors[0].device.index if tensors else torch.cuda.current_device()
        fn = _function(cubin, dev)
        block = _ParamBlock()
        vec = 0
        for k, t in enumerate(tensors):
            block.p[k] = t.data_ptr()
            if t.data_ptr() % 16 == 0:
                vec |= 1 << k
        block.vec = vec
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        ctas = max(1, min((total + rows_in_flight - 1) // rows_in_flight, sms * 8))
        args = (ctypes.c_void_p * 1)(ctypes.addressof(block))
        err, = driver.cuLaunchKernel(fn, ctas, 1, 1, THREADS, 1, 1, 0, stream, ctypes.addressof(args), 0)
        if int(err) != 0:
            raise RuntimeError(f"launch of a generated tile program failed: {err}")
        K.generated_launches += 1
        return 0

    run.source = source
    return run
