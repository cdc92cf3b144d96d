"""`import tilelang.language as T` — the tile DSL surface of the reference's TPU path.

Names, argument order and argument meaning follow tilelang/language/customize.py:101-603 (the
19 `ppl_*` intrinsics), tilelang/language/kernel.py (`T.Kernel`), allocate.py (`T.alloc_shared`),
pipeline.py (`T.Pipelined`) and the script-parser helpers the demos use (`T.prim_func`,
`T.macro`, `T.Tensor`, `T.ceildiv`, `T.min`, `T.float32`, `T.infinity` ...).  Instead of TVM TIR
the calls are recorded into the tracing IR of `ir.py`.
"""
from __future__ import annotations

import functools
import inspect
import math

from . import ir
from .ir import Buffer, Expr, PrimFunc, Region, Tracer, as_region, const_value

# ------------------------------------------------------------------------------- types & scalars
int32 = lambda v=None: "int32" if v is None else ir.Const(int(v), "int32")      # noqa: E731
int64 = lambda v=None: "int64" if v is None else ir.Const(int(v), "int64")      # noqa: E731


def _scalar(dtype):
    def make(value=None):
        if value is None:
            return dtype
        v = const_value(value)
        if v is None:
            raise ValueError(f"T.{dtype}(...) needs a compile-time constant")
        return ir.Const(float(v), dtype)
    make.__name__ = dtype
    return make


float32 = _scalar("float32")
float16 = _scalar("float16")
bfloat16 = _scalar("bfloat16")


def infinity(dtype="float32"):
    return ir.Const(math.inf, "float32" if dtype == "float" else dtype)


def ceildiv(a, b):
    return ir.ceildiv(a, b)


def min(*args):          # noqa: A001  (name fixed by the reference API)
    return ir.emin(*args)


def max(*args):          # noqa: A001
    return ir.emax(*args)


def Tensor(shape, dtype="float32"):
    """Parameter annotation: `A: T.Tensor((M, K), "float16")`."""
    return ir.TensorAnnotation(tuple(shape), str(dtype))


Buffer_ = Tensor       # some upstream programs spell it T.Buffer


def symbolic(name, dtype="int32"):
    raise NotImplementedError("T.symbolic (dynamic shapes) is not supported: kernels are bound to the "
                              "static shapes of the program, as on the reference's TPU path")


# ------------------------------------------------------------------------------- program structure
def prim_func(fn):
    """Trace `fn` once with symbolic tensors and return the recorded program."""
    sig = inspect.signature(fn)
    params = []
    for i, (pname, p) in enumerate(sig.parameters.items()):
        ann = p.annotation
        if isinstance(ann, str):      # `from __future__ import annotations` in the caller's module: evaluate it there
            scope = dict(fn.__globals__)
            scope.update(inspect.getclosurevars(fn).nonlocals)
            ann = eval(ann, scope)    # noqa: S307 - the annotation text of the user's own function
        if not isinstance(ann, ir.TensorAnnotation):
            raise TypeError(f"{fn.__name__}: parameter {pname} needs a T.Tensor(shape, dtype) annotation")
        for d in ann.shape:
            if const_value(d) is None:
                raise ValueError(f"{fn.__name__}: parameter {pname} has a non-constant dimension {d!r}")
        shape = tuple(int(const_value(d)) for d in ann.shape)
        params.append(Buffer(pname, shape, ann.dtype, "global", param_index=i))
    tracer = Tracer()
    previous, Tracer.current = Tracer.current, tracer
    try:
        fn(*params)
    finally:
        Tracer.current = previous
    return PrimFunc(fn.__name__, params, tracer)


def macro(fn):
    """Macros are inlined at trace time: calling one simply runs its body."""
    @functools.wraps(fn)
    def call(*args, **kwargs):
        return fn(*args, **kwargs)
    return call


class Kernel:
    """`with T.Kernel(gx, gy, gz, is_cpu=True) as (bx, by, bz):` — the launch grid.

    On the TPU the grid becomes serial loops on one core (src/ir.cc:164-173); here the block
    indices stay symbolic and the bound CUDA kernel chooses its own decomposition.
    """

    def __init__(self, *extents, threads=None, is_cpu=False, prelude=None):
        self.extents = tuple(extents)
        self.attrs = {"threads": threads, "is_cpu": is_cpu}

    def __enter__(self):
        t = Tracer.get()
        if t.grid:
            raise RuntimeError("only one T.Kernel scope per prim_func is supported")
        names = ["bx", "by", "bz"]
        vs = tuple(ir.Var(names[i] if i < 3 else f"b{i}") for i in range(len(self.extents)))
        t.grid, t.block_vars, t.kernel_attrs = self.extents, vs, self.attrs
        return vs[0] if len(vs) == 1 else vs

    def __exit__(self, *exc):
        return False


class _Loop:
    def __init__(self, kind, extent, **attrs):
        self.kind, self.extent, self.attrs = kind, extent, attrs

    def __iter__(self):
        t = Tracer.get()
        v = ir.Var(t.fresh("k"))
        t.emit("loop.begin", v, self.extent, kind=self.kind, **self.attrs)
        yield v                    # the body is traced once with a symbolic induction variable
        t.emit("loop.end", v)


def Pipelined(start, stop=None, num_stages=0, order=None, stage=None, sync=None, group=None):
    """Software-pipelined loop.  On the TPU `num_stages` only brackets the body with
    tpu_parallel_start/end (inject_pipeline.cc:844-853) and has no numerical effect."""
    if stop is not None:
        raise NotImplementedError("T.Pipelined(start, stop): only the single-extent form is used on this path")
    return _Loop("pipelined", start, num_stages=num_stages)


def serial(start, stop=None):
    if stop is not None:
        raise NotImplementedError("T.serial(start, stop)")
    return _Loop("serial", start)


def Parallel(*extents):
    raise NotImplementedError("T.Parallel element loops are not part of the ppl_* tile path")


def alloc_shared(shape, dtype, scope="shared.dyn"):
    """A tile in on-chip memory (allocate.py:22-33)."""
    t = Tracer.get()
    dims = []
    for d in shape:
        v = const_value(d)
        if v is None:
            raise ValueError(f"T.alloc_shared: non-constant tile dimension {d!r}")
        dims.append(int(v))
    buf = Buffer(t.fresh("tile"), tuple(dims), "float32" if str(dtype) == "float" else str(dtype), scope)
    t.tiles.append(buf)
    return buf


alloc_fragment = alloc_shared
alloc_local = alloc_shared


# ------------------------------------------------------------------------------- ppl_* intrinsics
def _emit(name, *args, **attrs):
    Tracer.get().emit(name, *args, **attrs)


def _scalar_value(value, what):
    v = const_value(value)
    if v is None:
        raise ValueError(f"{what}: the scalar operand must be a compile-time constant")
    return float(v)


def ppl_gemm(A, B, C, transpose_A=False, transpose_B=False):
    """C (+)= A x B on tiles; `C` is the accumulation tile (customize.py:101-133)."""
    K = A.shape[0] if transpose_A else A.shape[1]
    K_B = B.shape[1] if transpose_B else B.shape[0]
    assert K == K_B, "gemm K shape check failed"
    _emit("ppl.gemm", A, B, C, transpose_A=bool(transpose_A), transpose_B=bool(transpose_B),
          M=C.shape[0], N=C.shape[1], K=K)


def ppl_copy(src, dst):
    """Copy a tile/region between global and tile memory, casting when dtypes differ
    (customize.py:136-207).  A point-indexed operand (`A[bx*bm, 0]`) takes its extents from
    the other operand, right-aligned, as the reference's extent merging does."""
    s, d = as_region(src), as_region(dst)

    def fill(r: Region, other: Region) -> Region:
        if all(e is not None for e in r.extents):
            return r
        if any(e is not None for e in r.extents):
            # a region with slices: point indices select one element along their axis
            return Region(r.buffer, r.starts, tuple(1 if e is None else e for e in r.extents))
        oe = [1 if e is None else e for e in other.extents]
        rank = len(r.extents)
        oe = ([1] * (rank - len(oe)) + oe)[-rank:]
        return Region(r.buffer, r.starts, tuple(oe))

    s2, d2 = fill(s, d), fill(d, s)
    _emit("ppl.copy", s2, d2)


def ppl_fill(buffer, value):
    _emit("ppl.fill", buffer, _scalar_value(value, "ppl_fill"))


def ppl_clear(buffer):
    return ppl_fill(buffer, float32(0))


def ppl_subtract(out, inp1, inp2): _emit("ppl.sub", out, inp1, inp2)
def ppl_mul(out, inp1, inp2): _emit("ppl.mul", out, inp1, inp2)
def ppl_add(out, inp1, inp2): _emit("ppl.add", out, inp1, inp2)
def ppl_div(out, inp1, inp2): _emit("ppl.div", out, inp1, inp2)


def ppl_mul_C(out, inp1, value): _emit("ppl.mul_C", out, inp1, _scalar_value(value, "ppl_mul_C"))
def ppl_add_C(out, inp1, value): _emit("ppl.add_C", out, inp1, _scalar_value(value, "ppl_add_C"))


def ppl_exp2(out, work0, work1, coeff, table):
    """In-place NATURAL exponential of an fp32 tile (the name is historical,
    customize.py:313-339); the scratch operands are accepted and unused."""
    _emit("ppl.exp", out, work0, work1, coeff, table)


def ppl_sigmoid(out, inp, work0, work1, coeff, table):
    _emit("ppl.sigmoid", out, inp, work0, work1, coeff, table)


def ppl_rsqrt(out, inp): _emit("ppl.rsqrt", out, inp)


def ppl_gather(output, param, index, param_h): _emit("ppl.gather", output, param, index, int(const_value(param_h)))


def ppl_topk(dst_data, dst_idx, src, K, descended, length):
    _emit("ppl.topk", dst_data, dst_idx, src, int(const_value(K)), int(const_value(descended)),
          int(const_value(length)))


def ppl_reduce_sum(inp, out, dim):
    assert dim == 1, "Only dim=1 is supported for reduction"
    _emit("ppl.reduce_sum", inp, out)


def ppl_reduce_max(inp, out, dim, clear=True):
    assert dim == 1, "Only dim=1 is supported"
    if clear:
        _emit("ppl.fill", out, -math.inf)
    _emit("ppl.reduce_max", inp, out)


def ppl_rope_add(out, even_inp1, even_inp2, odd_inp1, odd_inp2):
    _emit("ppl.rope_add", out, even_inp1, even_inp2, odd_inp1, odd_inp2)


copy = ppl_copy          # the demos alias it themselves (`T.copy = T.ppl_copy`)

__all__ = [n for n in dir() if not n.startswith("_")]
