"""Tile-op executor: runs a traced `ppl.*` program op by op on the GPU.

The matcher (matcher.py) binds the programs it knows to fused kernels.  Any other program built
from the tile intrinsics is executed here the way the reference's generated C executes it on one
TPU core (src/target/codegen_ppl.cc: the launch grid becomes serial loops, every `ppl.*` call
becomes one runtime call on tiles in local memory): the grid is walked block by block, tiles are
device buffers, and every op is one launch of a kernel of this library - never a CPU or torch
computation.  It is correct rather than fast (one small launch per tile op); programs that matter
get a matcher.

Semantics follow tilelang/language/customize.py and the code generator:
  ppl.copy      window of a tensor <-> tile, tile <-> tile, casting when dtypes differ      (:136-207)
  ppl.fill      constant into a tile                                                        (:210-231)
  ppl.gemm      transpose_B=False: C (fp32) += A B;  transpose_B=True: C = A B^T            (codegen_ppl.cc:1244-1279)
  ppl.add/sub/mul/div   out = in1 (op) in2, in2 shaped like in1 or (M, 1)                   (:234-310, 423-472; codegen :868-913)
  ppl.mul_C/add_C       out = in (op) constant, the constant first cast to the tile dtype   (:263-284, 400-420; codegen :917-957)
  ppl.exp       natural exponential in place;  ppl.sigmoid, ppl.rsqrt: out = f(in)          (:313-397)
  ppl.reduce_sum  out (M,1) = row sums;  ppl.reduce_max  out = max(out, row maxima)         (:476-560)
  ppl.rope_add  out[2i] = e1[2i] + e2[2i+1], out[2i+1] = o1[2i+1] + o2[2i]                  (:563-603; codegen :1809-1848)
  ppl.gather / ppl.topk  on whole tensors                                                   (:353-362)
"""
from __future__ import annotations

from typing import Callable

import torch

from ..language.ir import Buffer, PrimFunc, Region, const_value

_BINARY_OPS = {"ppl.add": "add", "ppl.sub": "sub", "ppl.mul": "mul", "ppl.div": "div"}
_CONST_OPS = {"ppl.mul_C": "mul", "ppl.add_C": "add"}
_SUPPORTED = set(_BINARY_OPS) | set(_CONST_OPS) | {
    "ppl.copy", "ppl.fill", "ppl.gemm", "ppl.exp", "ppl.sigmoid", "ppl.rsqrt", "ppl.reduce_sum", "ppl.reduce_max",
    "ppl.rope_add", "ppl.gather", "ppl.topk", "loop.begin", "loop.end"}
_FLOATS = ("float32", "float16", "bfloat16")


class InterpreterError(NotImplementedError):
    pass


def _need(cond, msg):
    if not cond:
        raise InterpreterError(msg)


def _buf(x) -> Buffer:
    return x.buffer if isinstance(x, Region) else x


def validate(func: PrimFunc) -> None:
    """Static checks, so that an unsupported program is rejected when it is compiled, not when it runs."""
    depth = 0
    for op in func.ops:
        _need(op.name in _SUPPORTED, f"tile op {op.name} is not available in the generic executor")
        if op.name == "loop.begin":
            depth += 1
            _need(const_value(op.args[1]) is not None, "loop extents must be compile-time constants")
        elif op.name == "loop.end":
            depth -= 1
        for a in op.args:
            if isinstance(a, (Buffer, Region)):
                b = _buf(a)
                if b.scope == "global" and op.name == "ppl.copy":
                    continue                       # a window of a tensor of any rank; checked against the tile when it is addressed
                _need(1 <= len(b.shape) <= 2, f"{op.name}: {b.name} has rank {len(b.shape)}; tiles of rank 1 or 2 only")
        if op.name == "ppl.gemm":
            a, b, c = op.args
            _need(not op.attrs["transpose_A"], "ppl.gemm: transpose_A is not supported (the reference's code generator ignores it)")
            _need(a.dtype == b.dtype and a.dtype in _FLOATS + ("float8_e4m3", "e4m3_float8"),
                  "ppl.gemm: A and B must share a float dtype (fp32, fp16, bf16 or e4m3)")
            if op.attrs["transpose_B"]:
                _need(c.dtype in (a.dtype, "float32") and c.dtype in _FLOATS, "ppl.gemm: C must have the input dtype or float32")
            else:
                _need(c.dtype == "float32", "ppl.gemm without transpose_B accumulates: C must be float32")
        if op.name in _BINARY_OPS:
            out, x, y = op.args
            _need(out.shape == x.shape and out.dtype == x.dtype == y.dtype, f"{op.name}: out and in1 must agree in shape and dtype")
            _need(y.shape == x.shape or (len(x.shape) == 2 and tuple(y.shape) in ((x.shape[0], 1), (1, x.shape[1]))),
                  f"{op.name}: in2 must be shaped like in1, (M, 1) or (1, N)")
        if op.name == "ppl.rope_add":
            _need(all(len(t.shape) == 2 and t.shape == op.args[0].shape and t.dtype == op.args[0].dtype for t in op.args)
                  and op.args[0].shape[1] % 2 == 0, "ppl.rope_add: five 2-D tiles of one shape and dtype, even width")
        if op.name in ("ppl.reduce_sum", "ppl.reduce_max"):
            x, y = op.args[0], op.args[1]
            _need(len(x.shape) == 2 and y.dtype == x.dtype and y.shape[0] == x.shape[0] and
                  (len(y.shape) == 1 or y.shape[1] == 1), f"{op.name}: (M, N) -> (M, 1) of one dtype")
    _need(depth == 0, "unbalanced loops")
    _need(all(const_value(g) is not None for g in func.grid), "the launch grid must be static")


def build(func: PrimFunc) -> Callable[..., int]:
    """run(*device_tensors) -> int for a validated program."""
    validate(func)
    from .. import ops as K

    grid = [int(const_value(g)) for g in func.grid]
    loops = {}                                     # index of loop.begin -> index of its loop.end
    stack = []
    for i, op in enumerate(func.ops):
        if op.name == "loop.begin":
            stack.append(i)
        elif op.name == "loop.end":
            loops[stack.pop()] = i

    def run(*tensors):
        dev = tensors[0].device
        tiles: dict = {}

        def tensor_of(b: Buffer) -> torch.Tensor:
            if b.scope == "global":
                return tensors[b.param_index]
            t = tiles.get(b)
            if t is None:
                t = tiles[b] = torch.empty(tuple(b.shape), dtype=b.torch_dtype, device=dev)
            return t

        def view(x, env) -> torch.Tensor:
            """2-D strided view (rows, cols) of a buffer or of a region of it."""
            if isinstance(x, Buffer):
                t = tensor_of(x)
                return t if t.dim() == 2 else t.view(1, -1)
            t = tensor_of(x.buffer)
            idx = []
            for s, e in zip(x.starts, x.extents):
                lo = int(s.evaluate(env)) if hasattr(s, "evaluate") else int(s)
                idx.append(slice(lo, lo + int(e)))
            v = t[tuple(idx)]
            return v if v.dim() == 2 else v.reshape(1, -1) if v.is_contiguous() else v.unsqueeze(0)

        def copy_views(src, dst, env):
            """2-D views of the two sides of a ppl.copy.  A window of a tensor of rank 3 or 4 (or any window that is
            not a plain 2-D slice) is addressed like the fused path does: evenly strided rows, contiguous columns."""
            def plain(x):
                return isinstance(x, Buffer) or len(x.buffer.shape) <= 2
            if plain(src) and plain(dst):
                return view(src, env), view(dst, env)
            from .fuser import NotFusable, _window
            out = []
            for x, other in ((src, dst), (dst, src)):
                if plain(x):
                    out.append(view(x, env))
                    continue
                ob = _buf(other)
                shape = tuple(ob.shape) if len(ob.shape) == 2 else (1, int(ob.shape[0]))
                if ob.scope == "global":            # tensor to tensor: rows x last extent of this window
                    ext = [1 if e is None else int(e) for e in x.extents]
                    width = ext[-1]
                    rows = 1
                    for e in ext[:-1]:
                        rows *= e
                    shape = (rows, width)
                vars_ = [v for v in env]
                try:
                    base, coef, row_stride = _window(x, shape[0], shape[1], {}, vars_)
                except NotFusable as why:
                    raise InterpreterError(f"ppl.copy: {why}") from None
                off = base + sum(c * int(env[v]) for c, v in zip(coef, vars_))
                t = tensor_of(x.buffer)
                out.append(t.as_strided(shape, (row_stride if shape[0] > 1 else max(shape[1], 1), 1), t.storage_offset() + off))
            return out[0], out[1]

        def execute(lo: int, hi: int, env: dict) -> int:
            i = lo
            while i < hi:
                op = func.ops[i]
                if op.name == "loop.begin":
                    var, extent = op.args[0], int(const_value(op.args[1]))
                    end = loops[i]
                    for it in range(extent):
                        env[var] = it
                        rc = execute(i + 1, end, env)
                        if rc:
                            return rc
                    i = end + 1
                    continue
                rc = one(op, env)
                if rc:
                    return rc
                i += 1
            return 0

        def one(op, env) -> int:
            n, a = op.name, op.args
            if n == "ppl.copy":
                src, dst = copy_views(a[0], a[1], env)
                if src.numel() != dst.numel():
                    raise ValueError(f"ppl.copy: {a[0]!r} and {a[1]!r} differ in size")
                if src.shape != dst.shape:             # e.g. a (M, 1) column into a rank-1 tensor
                    _need(dst.is_contiguous() or src.is_contiguous(), "ppl.copy: reshaping copy between strided windows")
                    if dst.is_contiguous():
                        dst = dst.view(src.shape)
                    else:
                        src = src.view(dst.shape)
                return K.copy2d(src, dst)
            if n == "ppl.fill":
                return K.fill(view(a[0], env), float(a[1]))
            if n == "ppl.gemm":
                A, B, C = (tensor_of(x) for x in a)
                if op.attrs["transpose_B"]:
                    return K.gemm(A, B, C, transpose_b=True)
                tmp = torch.empty_like(C)
                return K.gemm(A, B, tmp) or K.binary(C, tmp, C, "add")
            if n in _BINARY_OPS:
                out, x, y = (view(t, env) for t in a)
                return K.binary(x, y, out, _BINARY_OPS[n])
            if n in _CONST_OPS:
                return K.binary(view(a[1], env), float(a[2]), view(a[0], env), _CONST_OPS[n])
            if n == "ppl.exp":
                t = tensor_of(a[0])
                return K.unary(t, t, "exp")
            if n == "ppl.sigmoid":
                return K.unary(tensor_of(a[1]), tensor_of(a[0]), "sigmoid")
            if n == "ppl.rsqrt":
                return K.unary(tensor_of(a[1]), tensor_of(a[0]), "rsqrt")
            if n == "ppl.reduce_sum":
                return K.reduce_rows(tensor_of(a[0]), tensor_of(a[1]), "sum")
            if n == "ppl.reduce_max":                  # the running maximum: `clear=True` filled -inf just before
                x, y = tensor_of(a[0]), tensor_of(a[1])
                tmp = torch.empty_like(y)
                y2, t2 = y.view(-1, 1), tmp.view(-1, 1)
                return K.reduce_rows(x, tmp, "max") or K.binary(y2, t2, y2, "max")
            if n == "ppl.rope_add":
                return K.rope_add(*(tensor_of(t) for t in a))
            if n == "ppl.gather":
                out, param, index = (tensor_of(_buf(t)) for t in a[:3])
                return K.gather_rows(param.view(a[3], -1), index.view(-1), out.view(index.numel(), -1))
            if n == "ppl.topk":
                vals, idx, src = (tensor_of(_buf(t)) for t in a[:3])
                return K.topk(src.view(-1)[:a[5]], vals.view(-1), idx.view(-1), a[3], bool(a[4]))
            raise InterpreterError(n)

        def walk(dim: int, env: dict) -> int:
            if dim == len(grid):
                return execute(0, len(func.ops), env)
            for b in range(grid[dim]):
                env[func.block_vars[dim]] = b
                rc = walk(dim + 1, env)
                if rc:
                    return rc
            return 0

        return walk(0, {})

    return run
