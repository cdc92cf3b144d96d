"""A small tracing IR for `T.prim_func` programs built from `T.ppl_*` tile intrinsics.

The reference parses the Python body into TVM TIR and every intrinsic becomes a
`T.call_extern("handle", "ppl.<op>", ...)` statement (tilelang/language/customize.py:101-603).
Here the body is executed once with symbolic values and the same stream of `ppl.<op>` records is
kept as plain Python objects: global tensors, tile buffers, regions with symbolic offsets, loop
brackets.  The recorded stream is what the program matcher (engine/matcher.py) reads.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Any, Optional

import torch

_DTYPE_NAMES = {
    "float32": torch.float32, "float": torch.float32, "float16": torch.float16, "half": torch.float16,
    "bfloat16": torch.bfloat16, "int32": torch.int32, "uint32": torch.uint32, "int16": torch.int16,
    "int8": torch.int8, "uint8": torch.uint8, "int64": torch.int64, "bool": torch.bool,
    "e4m3_float8": torch.float8_e4m3fn, "float8_e4m3": torch.float8_e4m3fn, "e5m2_float8": torch.float8_e5m2,
}


def map_torch_type(dtype) -> torch.dtype:
    """String dtype -> torch dtype (role of tilelang/utils/tensor.py `map_torch_type`)."""
    if isinstance(dtype, torch.dtype):
        return dtype
    try:
        return _DTYPE_NAMES[str(dtype)]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype!r}") from None


# --------------------------------------------------------------------------- expressions
class Expr:
    """Symbolic integer/float expression with just enough algebra for tile offsets."""

    def _bin(self, op, other, swap=False):
        a, b = (other, self) if swap else (self, other)
        return BinOp(op, wrap(a), wrap(b)).fold()

    def __add__(self, o): return self._bin("+", o)
    def __radd__(self, o): return self._bin("+", o, True)
    def __sub__(self, o): return self._bin("-", o)
    def __rsub__(self, o): return self._bin("-", o, True)
    def __mul__(self, o): return self._bin("*", o)
    def __rmul__(self, o): return self._bin("*", o, True)
    def __floordiv__(self, o): return self._bin("//", o)
    def __rfloordiv__(self, o): return self._bin("//", o, True)
    def __mod__(self, o): return self._bin("%", o)
    def __neg__(self): return BinOp("-", Const(0), self).fold()
    def __lt__(self, o): return self._bin("<", o)
    def __le__(self, o): return self._bin("<=", o)
    def __gt__(self, o): return self._bin(">", o)
    def __ge__(self, o): return self._bin(">=", o)

    def __bool__(self):
        raise TypeError("a symbolic value has no truth value at trace time; use T.min/T.max or "
                        "Python-level constants for control flow")

    def evaluate(self, env: dict) -> Any:
        raise NotImplementedError

    def affine(self) -> Optional[tuple[dict, Any]]:
        """({var: coeff}, const) if the expression is affine in its variables, else None."""
        return None


@dataclass(frozen=True, eq=False)
class Const(Expr):
    value: Any
    dtype: Optional[str] = None

    def evaluate(self, env): return self.value
    def affine(self): return ({}, self.value)
    def __repr__(self): return repr(self.value)
    def __float__(self): return float(self.value)
    def __int__(self): return int(self.value)
    def __index__(self): return int(self.value)
    def __bool__(self): return bool(self.value)
    def __neg__(self): return Const(-self.value, self.dtype)


@dataclass(frozen=True, eq=False)
class Var(Expr):
    name: str

    def evaluate(self, env): return env[self]
    def affine(self): return ({self: 1}, 0)
    def __repr__(self): return self.name
    def __hash__(self): return id(self)

    def __iter__(self):           # `with T.Kernel(n) as (bx,):` unpacks a single block index
        yield self


@dataclass(frozen=True, eq=False)
class BinOp(Expr):
    op: str
    a: Expr
    b: Expr

    def fold(self) -> Expr:
        if isinstance(self.a, Const) and isinstance(self.b, Const):
            return Const(_apply(self.op, self.a.value, self.b.value))
        if self.op in "+-*":
            aff = self.affine()
            if aff is not None and not aff[0]:
                return Const(aff[1])
        return self

    def evaluate(self, env):
        return _apply(self.op, self.a.evaluate(env), self.b.evaluate(env))

    def affine(self):
        fa, fb = self.a.affine(), self.b.affine()
        if fa is None or fb is None:
            return None
        (va, ca), (vb, cb) = fa, fb
        if self.op in "+-":
            sign = 1 if self.op == "+" else -1
            out = dict(va)
            for v, c in vb.items():
                out[v] = out.get(v, 0) + sign * c
            return ({v: c for v, c in out.items() if c != 0}, ca + sign * cb)
        if self.op == "*":
            if not va:
                return ({v: c * ca for v, c in vb.items() if c * ca != 0}, ca * cb)
            if not vb:
                return ({v: c * cb for v, c in va.items() if c * cb != 0}, ca * cb)
        return None

    def __repr__(self): return f"({self.a!r} {self.op} {self.b!r})"


@dataclass(frozen=True, eq=False)
class Call(Expr):
    fn: str
    args: tuple

    def evaluate(self, env):
        vals = [a.evaluate(env) for a in self.args]
        if self.fn == "min": return min(vals)
        if self.fn == "max": return max(vals)
        if self.fn == "ceildiv": return -(-vals[0] // vals[1])
        raise ValueError(self.fn)

    def __repr__(self): return f"{self.fn}({', '.join(map(repr, self.args))})"


def _apply(op, x, y):
    return {"+": lambda: x + y, "-": lambda: x - y, "*": lambda: x * y, "//": lambda: x // y,
            "%": lambda: x % y, "<": lambda: x < y, "<=": lambda: x <= y, ">": lambda: x > y,
            ">=": lambda: x >= y}[op]()


def wrap(v) -> Expr:
    return v if isinstance(v, Expr) else Const(v)


def const_value(v):
    """Python number behind a constant expression, or None if it is symbolic."""
    if isinstance(v, (int, float)):
        return v
    if isinstance(v, Const):
        return v.value
    if isinstance(v, Expr):
        aff = v.affine()
        if aff is not None and not aff[0]:
            return aff[1]
    return None


def ceildiv(a, b):
    ca, cb = const_value(a), const_value(b)
    if ca is not None and cb is not None:
        return -(-ca // cb)
    return Call("ceildiv", (wrap(a), wrap(b)))


def emin(*args):
    vals = [const_value(a) for a in args]
    if all(v is not None for v in vals):
        return min(vals)
    return Call("min", tuple(wrap(a) for a in args))


def emax(*args):
    vals = [const_value(a) for a in args]
    if all(v is not None for v in vals):
        return max(vals)
    return Call("max", tuple(wrap(a) for a in args))


# --------------------------------------------------------------------------- buffers and regions
@dataclass(eq=False)
class Buffer:
    name: str
    shape: tuple
    dtype: str
    scope: str                     # "global" (kernel parameter) or "shared.dyn" (tile)
    param_index: int = -1

    @property
    def torch_dtype(self) -> torch.dtype:
        return map_torch_type(self.dtype)

    def __getitem__(self, idx) -> "Region":
        if not isinstance(idx, tuple):
            idx = (idx,)
        if len(idx) != len(self.shape):
            raise IndexError(f"{self.name}: {len(idx)} indices for a rank-{len(self.shape)} buffer")
        starts, extents = [], []
        for i, dim in zip(idx, self.shape):
            if isinstance(i, slice):
                lo = 0 if i.start is None else i.start
                hi = dim if i.stop is None else i.stop
                ext = const_value(wrap(hi) - wrap(lo))
                if ext is None:
                    raise ValueError(f"{self.name}: slice extent {hi!r} - {lo!r} is not a constant")
                starts.append(lo)
                extents.append(ext)
            else:
                starts.append(i)
                extents.append(None)       # a point index: extent comes from the other operand
        return Region(self, tuple(starts), tuple(extents))

    def whole(self) -> "Region":
        return Region(self, tuple(0 for _ in self.shape), tuple(self.shape))

    def __repr__(self): return f"{self.name}<{self.scope} {list(self.shape)} {self.dtype}>"


@dataclass(eq=False)
class Region:
    buffer: Buffer
    starts: tuple
    extents: tuple                 # None where the source was a point index (`A[bx*bm, 0]`)

    def __repr__(self):
        parts = []
        for s, e in zip(self.starts, self.extents):
            parts.append(f"{s!r}" if e is None else f"{s!r}:+{e}")
        return f"{self.buffer.name}[{', '.join(parts)}]"


def as_region(x) -> Region:
    if isinstance(x, Region):
        return x
    if isinstance(x, Buffer):
        return x.whole()
    raise TypeError(f"expected a buffer or a buffer region, got {type(x).__name__}")


# --------------------------------------------------------------------------- the op stream
@dataclass(eq=False)
class Op:
    name: str                      # "ppl.copy", "ppl.gemm", ..., "loop.begin", "loop.end"
    args: tuple
    attrs: dict = field(default_factory=dict)

    def __repr__(self):
        a = ", ".join(repr(x) for x in self.args)
        extra = f" {self.attrs}" if self.attrs else ""
        return f"{self.name}({a}){extra}"


class Tracer:
    """Collects the op stream of one prim_func body."""
    current: Optional["Tracer"] = None

    def __init__(self):
        self.ops: list[Op] = []
        self.grid: tuple = ()
        self.block_vars: tuple = ()
        self.tiles: list[Buffer] = []
        self._names = itertools.count()
        self.kernel_attrs: dict = {}

    def emit(self, name, *args, **attrs):
        self.ops.append(Op(name, tuple(args), attrs))

    def fresh(self, prefix):
        return f"{prefix}_{next(self._names)}"

    @classmethod
    def get(cls) -> "Tracer":
        if cls.current is None:
            raise RuntimeError("T.* tile intrinsics can only be used inside a @T.prim_func body")
        return cls.current


@dataclass
class TensorAnnotation:
    """What `T.Tensor(shape, dtype)` evaluates to in a parameter annotation."""
    shape: tuple
    dtype: str


class PrimFunc:
    """A traced program: parameters, launch grid and the `ppl.*` op stream."""

    def __init__(self, name, params, tracer: Tracer):
        self.name = name
        self.params: list[Buffer] = params
        self.grid = tracer.grid
        self.block_vars = tracer.block_vars
        self.ops = tracer.ops
        self.tiles = tracer.tiles
        self.kernel_attrs = tracer.kernel_attrs
        self.attrs = {"global_symbol": name}

    def script(self) -> str:
        """Readable listing of the recorded program (what `get_kernel_source` shows)."""
        lines = [f"prim_func {self.name}(" + ", ".join(
            f"{p.name}: Tensor({list(p.shape)}, {p.dtype})" for p in self.params) + ")",
            f"  grid {list(self.grid)} as {list(self.block_vars)}"]
        depth = 1
        for op in self.ops:
            if op.name == "loop.end":
                depth -= 1
            lines.append("  " * depth + repr(op))
            if op.name == "loop.begin":
                depth += 1
        return "\n".join(lines)

    def __repr__(self): return self.script()
