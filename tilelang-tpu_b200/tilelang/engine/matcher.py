"""Program matcher: binds a traced `ppl.*` program to a hand-written CUDA program.

The reference lowers every program through TVM passes and prints C for the SOPHGO runtime
(tilelang/engine/lower.py:195-250, src/target/codegen_ppl.cc).  Here the kernels are pre-built,
so "lowering" is recognition: the op stream of a prim_func is compared with the canonical form
of each supported program (the programs of tpu_demo/), the facts that matter (shapes, scalars,
operand order, layouts) are extracted and checked, and the program is bound to one C-ABI entry
point.  A program that matches nothing is rejected loudly; nothing ever falls back to the CPU.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Optional

import torch

from ..language.ir import Buffer, Call, Op, PrimFunc, Region, const_value


class UnsupportedProgram(NotImplementedError):
    pass


@dataclass
class BoundKernel:
    """A recognised program: `run(*device_tensors) -> int` launches the CUDA kernels."""
    program: str                   # e.g. "rmsnorm"
    entry_point: str               # C-ABI symbol(s) it calls
    run: Callable[..., int]
    facts: dict
    full_outputs: bool = True      # every element of every output is written (the adapter need not upload outputs)

    def describe(self) -> str:
        return f"{self.program} -> {self.entry_point} {self.facts}"


# ------------------------------------------------------------------------------- helpers
def _names(ops):
    return [o.name for o in ops]


def _is_param(x, func: PrimFunc, index: Optional[int] = None) -> bool:
    buf = x.buffer if isinstance(x, Region) else x
    if not isinstance(buf, Buffer) or buf.scope != "global":
        return False
    return index is None or buf.param_index == index


def _buf(x) -> Buffer:
    return x.buffer if isinstance(x, Region) else x


def _close(a: float, b: float, rel=1e-6) -> bool:
    return abs(a - b) <= rel * max(abs(a), abs(b), 1e-30)


def _same_expr(a, b) -> bool:
    """Two index expressions denote the same value (compared as affine forms over the block and loop variables)."""
    ca, cb = const_value(a), const_value(b)
    if ca is not None or cb is not None:
        return ca is not None and cb is not None and ca == cb
    fa, fb = a.affine(), b.affine()
    if fa is None or fb is None:
        return a is b
    return fa[1] == fb[1] and {id(v): c for v, c in fa[0].items()} == {id(v): c for v, c in fb[0].items()}


def _extents(r: Region):
    return tuple(1 if e is None else int(e) for e in r.extents)


def _require(cond, msg):
    if not cond:
        raise UnsupportedProgram(msg)


def _check_tiling(func: PrimFunc, what: str, pairs):
    """The reference checks tile bounds statically and has no tail masking
    (src/target/codegen_ppl.cc:967-1002): tiles must divide the tensor."""
    for full, tile in pairs:
        _require(full % tile == 0, f"{what}: tile {tile} does not divide dimension {full} "
                                   f"(the tile path has no tail masking)")


def _grid(func: PrimFunc):
    g = [const_value(e) for e in func.grid]
    _require(all(v is not None for v in g), "launch grid must be static")
    return [int(v) for v in g]


# ------------------------------------------------------------------------------- programs
def _match_matmul(func: PrimFunc):
    n = _names(func.ops)
    if n[:6] != ["ppl.fill", "loop.begin", "ppl.copy", "ppl.copy", "ppl.gemm", "loop.end"]:
        return None
    tail = n[6:]
    if tail not in (["ppl.copy"], ["ppl.copy", "ppl.copy"]) or len(func.params) != 3:
        return None
    ops = func.ops
    fill, _, cp_a, cp_b, gemm, _ = ops[:6]
    a_tile, b_tile, c_tile = gemm.args
    if fill.args[0] is not c_tile or fill.args[1] != 0.0:
        return None
    if _buf(cp_a.args[1]) is not a_tile or _buf(cp_b.args[1]) is not b_tile:
        return None
    a_src, b_src, store = cp_a.args[0], cp_b.args[0], ops[-1].args[1]
    if not (_is_param(a_src, func) and _is_param(b_src, func) and _is_param(store, func)):
        return None
    _require(not gemm.attrs["transpose_A"], "matmul: transpose_A is not supported (the reference's code "
                                            "generator ignores it)")
    trans_b = gemm.attrs["transpose_B"]
    A, B, C = _buf(a_src), _buf(b_src), _buf(store)
    _require(len(A.shape) == 2 and len(B.shape) == 2 and len(C.shape) == 2, "matmul: tensors must be 2-D")
    M, K = A.shape
    N = B.shape[0] if trans_b else B.shape[1]
    _require((B.shape[1] if trans_b else B.shape[0]) == K and tuple(C.shape) == (M, N),
             "matmul: inconsistent A/B/C shapes")
    bm, bk = a_tile.shape
    bn = b_tile.shape[0] if trans_b else b_tile.shape[1]
    _check_tiling(func, "matmul", [(M, bm), (N, bn), (K, bk)])
    _require(const_value(ops[1].args[1]) == K // bk, "matmul: the K loop must cover K")
    if trans_b and K // bk > 1:
        # `C = A B^T` carries no accumulate flag in the reference's generated code
        # (src/target/codegen_ppl.cc:1276-1279): every K iteration overwrites C, so the program
        # does not compute the full product.  The tile-op executor reproduces that; the fused GEMM
        # (which sums over all of K) is bound only where the two agree.
        return None
    _require(sorted(_grid(func)) == sorted([N // bn, M // bm]), "matmul: the grid must cover C")
    # addressing: A[row block, k tile], B[k tile, column block] (or B[column block, k tile]), C[row block, column block]
    kvar = ops[1].args[0]
    ar, br, cr = cp_a.args[0], cp_b.args[0], ops[-1].args[1]

    def steps(e, var, size):
        f = e.affine() if hasattr(e, "affine") else None
        return f is not None and f[1] == 0 and {id(v): c for v, c in f[0].items()} == {id(var): size}

    b_k, b_n = (br.starts[1], br.starts[0]) if trans_b else (br.starts[0], br.starts[1])
    if not (steps(ar.starts[1], kvar, bk) and steps(b_k, kvar, bk) and _same_expr(ar.starts[0], cr.starts[0])
            and _same_expr(b_n, cr.starts[1]) and const_value(ar.starts[0]) is None and const_value(b_n) is None):
        return None                     # same op order, other addressing: the tile-op executor runs it as written
    fa, fn_ = ar.starts[0].affine(), b_n.affine()
    if fa is None or fn_ is None or list(fa[0].values()) != [bm] or list(fn_[0].values()) != [bn] or fa[1] or fn_[1] \
            or next(iter(fa[0])) is next(iter(fn_[0])):
        return None
    ia, ib, ic = A.param_index, B.param_index, C.param_index
    from .. import ops as native

    def run(*t):
        return native.gemm(t[ia], t[ib], t[ic], transpose_b=trans_b)

    return BoundKernel("matmul", "tl_b200_gemm", run,
                       dict(M=M, N=N, K=K, transpose_B=trans_b, in_dtype=A.dtype, out_dtype=C.dtype))


_RMS_BODY = ["ppl.copy", "ppl.copy", "ppl.mul", "ppl.reduce_sum", "ppl.mul_C", "ppl.add_C", "ppl.rsqrt", "ppl.mul",
             "ppl.copy", "ppl.copy"]
_RMS_SPLITK = ["ppl.fill", "loop.begin", "ppl.copy", "ppl.copy", "ppl.mul", "ppl.reduce_sum", "ppl.add", "loop.end",
               "ppl.mul_C", "ppl.add_C", "ppl.rsqrt", "loop.begin", "ppl.copy", "ppl.copy", "ppl.mul", "ppl.copy",
               "ppl.copy", "loop.end"]


# the float32 programs are the same without the casting copies
_RMS_BODY_F32 = ["ppl.copy", "ppl.mul", "ppl.reduce_sum", "ppl.mul_C", "ppl.add_C", "ppl.rsqrt", "ppl.mul", "ppl.copy"]
_RMS_SPLITK_F32 = ["ppl.fill", "loop.begin", "ppl.copy", "ppl.mul", "ppl.reduce_sum", "ppl.add", "loop.end", "ppl.mul_C",
                   "ppl.add_C", "ppl.rsqrt", "loop.begin", "ppl.copy", "ppl.mul", "ppl.copy", "loop.end"]


def _strip_weight(func: PrimFunc):
    """Splits off the per-column weight of the Llama form of RMSNorm, if the program has one:
    a third parameter of shape (1, N) that is loaded into a (1, N) tile (cast to fp32 for 16-bit
    tensors) and multiplied into the normalised tile with a row-broadcast `ppl_mul`.  The reference's
    `ppl_mul` only broadcasts an (M, 1) column (src/target/codegen_ppl.cc:868-889); the (1, N) row is
    an extension of this library for the benchmark's weighted RMSNorm.  Returns (ops without the
    weight ops, weight buffer or None, the weight mul or None)."""
    if len(func.params) != 3:
        return list(func.ops), None, None
    ops = list(func.ops)
    w_tiles, drop, W = set(), set(), None
    for i, o in enumerate(ops):
        if o.name != "ppl.copy":
            continue
        src, dst = _buf(o.args[0]), _buf(o.args[1])
        if _is_param(src, func) and len(src.shape) == 2 and src.shape[0] == 1 and dst.scope != "global" \
                and tuple(dst.shape) == tuple(src.shape):
            if W is not None and src is not W:
                return list(func.ops), None, None
            W = src
            w_tiles.add(id(dst))
            drop.add(i)
        elif id(src) in w_tiles and dst.scope != "global" and tuple(dst.shape) == tuple(src.shape):
            w_tiles.add(id(dst))                      # the cast copy of the weight tile
            drop.add(i)
    if W is None:
        return list(func.ops), None, None
    muls = [i for i, o in enumerate(ops) if o.name == "ppl.mul" and id(o.args[2]) in w_tiles]
    if len(muls) != 1:
        return list(func.ops), None, None
    wmul = ops[muls[0]]
    drop.add(muls[0])
    return [o for i, o in enumerate(ops) if i not in drop], W, wmul


def _match_rmsnorm(func: PrimFunc):
    ops, W, wmul = _strip_weight(func)
    n = _names(ops)
    if n not in (_RMS_BODY, _RMS_SPLITK, _RMS_BODY_F32, _RMS_SPLITK_F32) or len(func.params) != (3 if W is not None else 2):
        return None
    split = n in (_RMS_SPLITK, _RMS_SPLITK_F32)
    if split and W is not None:
        return None
    copies = [o for o in ops if o.name == "ppl.copy"]
    load = next((o for o in copies if _is_param(o.args[0], func)), None)          # first load of the input
    store = next((o for o in reversed(copies) if _is_param(o.args[1], func)), None)
    if load is None or store is None:
        return None
    muls = [o for o in ops if o.name == "ppl.mul"]
    red = next(o for o in ops if o.name == "ppl.reduce_sum")
    mul_c = next(o for o in ops if o.name == "ppl.mul_C")
    add_c = next(o for o in ops if o.name == "ppl.add_C")
    rsq = next(o for o in ops if o.name == "ppl.rsqrt")
    sq, norm = muls[0], muls[-1]
    # dataflow: x * x -> row sum -> * 1/N -> + eps -> rsqrt -> x * r (a program with the same op order
    # but other operands is not RMSNorm and goes to the tile-op executor)
    acc = rsq.args[0]
    flow = (sq.args[1] is sq.args[2] and red.args[0] is sq.args[0]
            and mul_c.args[0] is mul_c.args[1] and add_c.args[0] is add_c.args[1] and add_c.args[1] is mul_c.args[0]
            and rsq.args[1] is add_c.args[0] and norm.args[2] is acc and tuple(acc.shape) == (sq.args[1].shape[0], 1))
    if not split:
        flow = flow and mul_c.args[1] is red.args[1] and norm.args[1] is sq.args[1] and norm.args[0] is sq.args[1]
    if not flow:
        return None
    if wmul is not None and not (wmul.args[0] is norm.args[0] and wmul.args[1] is norm.args[0]
                                 and func.ops.index(wmul) > func.ops.index(norm)):
        return None
    X, Y = _buf(load.args[0]), _buf(store.args[1])
    _require(len(X.shape) == 2 and X.shape == Y.shape and X.dtype == Y.dtype, "rmsnorm: A and B must be equal 2-D")
    M, N = X.shape
    _require(_close(mul_c.args[2], 1.0 / N), f"rmsnorm: the mean scale {mul_c.args[2]} is not 1/N")
    tile = _buf(load.args[1])
    _check_tiling(func, "rmsnorm", [(M, tile.shape[0]), (N, tile.shape[1])])
    _require(split or tile.shape[1] == N, "rmsnorm: the row tile must span N")
    if W is not None:
        _require(tuple(W.shape) == (1, N) and W.dtype == X.dtype, "rmsnorm: the weight must be a (1, N) row of the input dtype")
    eps = float(add_c.args[2])
    ix, iy = X.param_index, Y.param_index
    iw = W.param_index if W is not None else None
    from .. import ops as native

    def run(*t):
        return native.rmsnorm(t[ix], t[iy], None if iw is None else t[iw].view(-1), eps)

    return BoundKernel("rmsnorm_splitk" if split else "rmsnorm", "tl_b200_rmsnorm", run,
                       dict(rows=M, cols=N, eps=eps, dtype=X.dtype, weight=W is not None))


_ROPE = ["ppl.copy", "ppl.copy", "ppl.copy", "ppl.mul", "ppl.mul", "ppl.mul_C", "ppl.mul", "ppl.rope_add", "ppl.copy"]


def _match_rope(func: PrimFunc):
    if _names(func.ops) != _ROPE or len(func.params) != 4:
        return None
    ops = func.ops
    ld_x, ld_c, ld_s, mul_xc, mul_xs, neg, mul_ns, radd, store = ops
    x_t, c_t, s_t = _buf(ld_x.args[1]), _buf(ld_c.args[1]), _buf(ld_s.args[1])
    ok = (mul_xc.args[1] is x_t and mul_xc.args[2] is c_t and mul_xs.args[1] is x_t and mul_xs.args[2] is s_t
          and neg.args[1] is x_t and neg.args[2] == -1.0 and mul_ns.args[1] is neg.args[0]
          and mul_ns.args[2] is s_t)
    x_cos, x_sin, x_neg_sin = mul_xc.args[0], mul_xs.args[0], mul_ns.args[0]
    out_t, e1, e2, o1, o2 = radd.args
    ok = ok and e1 is x_cos and e2 is x_neg_sin and o1 is x_cos and o2 is x_sin and _buf(store.args[0]) is out_t
    if not ok:
        return None
    X, Cs, Sn, Out = _buf(ld_x.args[0]), _buf(ld_c.args[0]), _buf(ld_s.args[0]), _buf(store.args[1])
    _require(X.dtype == Cs.dtype == Sn.dtype == Out.dtype, "rope: one dtype for x/cos/sin/out")
    _require(x_t.shape[1] % 2 == 0, "rope: tile width must be even")
    if len(X.shape) == 3:
        # x and out are (tokens, heads, W); cos/sin are (tokens, W) tables shared by the heads of a
        # token: a block loads rows [t0, t0 + bt) of ONE head and the same rows of the tables
        T_, H_, W_ = X.shape
        _require(Out.shape == X.shape and tuple(Cs.shape) == (T_, W_) and Sn.shape == Cs.shape,
                 "rope: x/out (tokens, heads, W) need cos/sin tables of shape (tokens, W)")
        xr, cr, sr, orr = ld_x.args[0], ld_c.args[0], ld_s.args[0], store.args[1]
        bt = x_t.shape[0]
        _require(_extents(xr) == (bt, 1, W_) and _extents(orr) == (bt, 1, W_) and _extents(cr) == (bt, W_)
                 and _extents(sr) == (bt, W_) and tuple(x_t.shape) == (bt, W_),
                 "rope: a block must cover bt tokens of one head and the full width")
        _require(_same_expr(xr.starts[0], cr.starts[0]) and _same_expr(xr.starts[0], sr.starts[0])
                 and _same_expr(xr.starts[0], orr.starts[0]) and _same_expr(xr.starts[1], orr.starts[1]),
                 "rope: x, cos, sin and out must be addressed by the same token block (and x, out by the same head)")
        _check_tiling(func, "rope", [(T_, bt)])
        _require(sorted(_grid(func)) == sorted([T_ // bt, H_]), "rope: the grid must cover tokens x heads")
    else:
        _require(X.shape == Cs.shape == Sn.shape == Out.shape and len(X.shape) == 2, "rope: x/cos/sin/out must be "
                 "equal 2-D tensors")
        _check_tiling(func, "rope", [(X.shape[0], x_t.shape[0]), (X.shape[1], x_t.shape[1])])
    idx = [b.param_index for b in (X, Cs, Sn, Out)]
    from .. import ops as native

    def run(*t):
        return native.rope(t[idx[0]], t[idx[1]], t[idx[2]], t[idx[3]])

    return BoundKernel("rope", "tl_b200_rope", run, dict(shape=list(X.shape), table=list(Cs.shape), dtype=X.dtype))


_SWIGLU = ["ppl.fill", "ppl.copy", "ppl.copy", "ppl.copy", "ppl.copy", "ppl.mul_C", "ppl.exp", "ppl.add", "ppl.div",
           "ppl.mul", "ppl.copy", "ppl.copy"]


_SWIGLU_F32 = ["ppl.fill", "ppl.copy", "ppl.copy", "ppl.mul_C", "ppl.exp", "ppl.add", "ppl.div", "ppl.mul", "ppl.copy"]


def _match_swiglu(func: PrimFunc):
    names = _names(func.ops)
    if names not in (_SWIGLU, _SWIGLU_F32) or len(func.params) != 3:
        return None
    if names == _SWIGLU:
        fill, ld_g, ld_u, cv_g, cv_u, neg, ex, add1, div, mul, cv_o, store = func.ops
        g32, u32 = _buf(cv_g.args[1]), _buf(cv_u.args[1])
        casts = (_buf(cv_g.args[0]) is _buf(ld_g.args[1]) and _buf(cv_u.args[0]) is _buf(ld_u.args[1])
                 and _buf(cv_o.args[0]) is mul.args[0] and _buf(store.args[0]) is _buf(cv_o.args[1]))
    else:                                                   # float32: loads and the store touch the fp32 tiles directly
        fill, ld_g, ld_u, neg, ex, add1, div, mul, store = func.ops
        g32, u32 = _buf(ld_g.args[1]), _buf(ld_u.args[1])
        casts = _buf(store.args[0]) is mul.args[0]
    ones = fill.args[0]
    ok = (casts and fill.args[1] == 1.0
          and neg.args[1] is g32 and neg.args[2] == -1.0 and ex.args[0] is neg.args[0]
          and add1.args[1] is neg.args[0] and add1.args[2] is ones
          and div.args[1] is g32 and div.args[2] is add1.args[0]
          and {id(mul.args[1]), id(mul.args[2])} == {id(u32), id(div.args[0])})
    if not ok:
        return None
    G, U, Out = _buf(ld_g.args[0]), _buf(ld_u.args[0]), _buf(store.args[1])
    _require(G.shape == U.shape == Out.shape and G.dtype == U.dtype == Out.dtype, "swiglu: equal shapes and dtypes")
    t = _buf(ld_g.args[1])
    _check_tiling(func, "swiglu", [(G.shape[0], t.shape[0]), (G.shape[1], t.shape[1])])
    idx = [b.param_index for b in (G, U, Out)]
    from .. import ops as native

    def run(*ts):
        return native.swiglu(ts[idx[0]], ts[idx[1]], ts[idx[2]])

    return BoundKernel("swiglu", "tl_b200_swiglu", run, dict(shape=list(G.shape), dtype=G.dtype))


_MLP = ["ppl.fill", "ppl.copy", "ppl.copy", "ppl.copy", "ppl.copy", "ppl.gemm", "ppl.copy", "ppl.mul_C", "ppl.exp",
        "ppl.add", "ppl.div", "ppl.gemm", "ppl.copy", "ppl.mul", "ppl.copy", "ppl.gemm", "ppl.copy"]


def _match_mlp(func: PrimFunc):
    """The gated MLP tile program (tpu_demo/ppl/mlp/mlp_bf16.py:56-137): gate GEMM -> SiLU, up GEMM,
    product, down GEMM.  Bound to the fused gate/up kernel plus one GEMM."""
    if _names(func.ops) != _MLP or len(func.params) != 5:
        return None
    (fill, ld_x, ld_g, ld_u, ld_d, gemm_g, cv_g, neg, ex, add1, div, gemm_u, cv_u, mul, cv_a, gemm_d, store) = func.ops
    ones = fill.args[0]
    x_t, g_t, u_t, d_t = (_buf(o.args[1]) for o in (ld_x, ld_g, ld_u, ld_d))
    g32, u32 = _buf(cv_g.args[1]), _buf(cv_u.args[1])
    silu = div.args[0]
    ok = (fill.args[1] == 1.0
          and gemm_g.args[0] is x_t and gemm_g.args[1] is g_t and _buf(cv_g.args[0]) is gemm_g.args[2]
          and neg.args[1] is g32 and neg.args[2] == -1.0 and ex.args[0] is neg.args[0]
          and add1.args[1] is neg.args[0] and add1.args[2] is ones
          and div.args[1] is g32 and div.args[2] is add1.args[0]
          and gemm_u.args[0] is x_t and gemm_u.args[1] is u_t and _buf(cv_u.args[0]) is gemm_u.args[2]
          and {id(mul.args[1]), id(mul.args[2])} == {id(silu), id(u32)}
          and _buf(cv_a.args[0]) is mul.args[0] and gemm_d.args[0] is _buf(cv_a.args[1]) and gemm_d.args[1] is d_t
          and _buf(store.args[0]) is gemm_d.args[2])
    if not ok:
        return None
    srcs = [ld_x.args[0], ld_g.args[0], ld_u.args[0], ld_d.args[0], store.args[1]]
    if not all(_is_param(r, func) for r in srcs):
        return None
    for g in (gemm_g, gemm_u, gemm_d):
        _require(g.attrs["transpose_B"] and not g.attrs["transpose_A"],
                 "mlp: the weights are (out_features, in_features) tiles used with transpose_B=True")
    X, Wg, Wu, Wd, Out = (_buf(r) for r in srcs)
    _require(all(len(b.shape) == 2 for b in (X, Wg, Wu, Wd, Out)), "mlp: tensors must be 2-D")
    M, H = X.shape
    I = Wg.shape[0]
    _require(tuple(Wg.shape) == (I, H) and tuple(Wu.shape) == (I, H) and tuple(Wd.shape) == (H, I)
             and tuple(Out.shape) == (M, H), "mlp: inconsistent x / weight / output shapes")
    _require(len({b.dtype for b in (X, Wg, Wu, Wd, Out)}) == 1, "mlp: one 16-bit dtype for all tensors")
    bs, bh = x_t.shape
    bi = g_t.shape[0]
    _check_tiling(func, "mlp", [(M, bs)])
    # The program keeps no accumulator across tiles of the hidden or intermediate dimension (every
    # (by, bz) tile overwrites the same output block), so only its single-tile form is the MLP.
    if bh != H or bi != I:
        return None                     # the generic executor runs that form tile by tile, as the reference would
    _require(sorted(_grid(func)) == sorted([M // bs, 1, 1]), "mlp: the grid must cover the rows")
    ix, ig, iu, idn, io = (b.param_index for b in (X, Wg, Wu, Wd, Out))
    from .. import ops as native

    def run(*t):
        act = torch.empty((M, I), dtype=t[ix].dtype, device=t[ix].device)     # silu(gate) * up, never a kernel output
        rc = native.mlp_gate_up(t[ix], t[ig], t[iu], act)
        return rc or native.gemm(act, t[idn], t[io], transpose_b=True)

    return BoundKernel("mlp", "tl_b200_mlp_gate_up + tl_b200_gemm", run,
                       dict(M=M, hidden=H, intermediate=I, dtype=X.dtype))


def _match_reduce(func: PrimFunc):
    n = [x for x in _names(func.ops) if x != "ppl.fill"]
    if len(n) != 3 or n[0] != "ppl.copy" or n[2] != "ppl.copy" or n[1] not in ("ppl.reduce_sum", "ppl.reduce_max"):
        return None
    ops = [o for o in func.ops if o.name != "ppl.fill"]
    X, Y = _buf(ops[0].args[0]), _buf(ops[2].args[1])
    if not (_is_param(X, func) and _is_param(Y, func)):
        return None
    tile = _buf(ops[0].args[1])
    _require(len(X.shape) == 2 and tile.shape[1] == X.shape[1], "row reduce: the tile must span the whole row")
    _require(Y.shape[0] == X.shape[0] and X.dtype == Y.dtype, "row reduce: Y must be (M, 1) of X's dtype")
    _check_tiling(func, "row reduce", [(X.shape[0], tile.shape[0])])
    op = "sum" if n[1] == "ppl.reduce_sum" else "max"
    ix, iy = X.param_index, Y.param_index
    from .. import ops as native

    def run(*t):
        return native.reduce_rows(t[ix], t[iy], op)

    return BoundKernel(f"reduce_{op}", "tl_b200_reduce_rows", run, dict(rows=X.shape[0], cols=X.shape[1], dtype=X.dtype))


def _match_topk(func: PrimFunc):
    if _names(func.ops) != ["ppl.topk"]:
        return None
    dst, idx, src, k, desc, length = func.ops[0].args
    _require(all(_is_param(b, func) for b in (dst, idx, src)), "topk operates on kernel parameters")
    _require(src.shape[-1] == length, "topk: length must equal the source length")
    i_d, i_i, i_s = dst.param_index, idx.param_index, src.param_index
    from .. import ops as native

    def run(*t):
        return native.topk(t[i_s], t[i_d], t[i_i], k, bool(desc))

    return BoundKernel("topk", "tl_b200_topk", run, dict(length=length, K=k, descended=bool(desc), dtype=src.dtype),
                       full_outputs=False)       # only the first K entries of the two outputs are written


def _match_gather(func: PrimFunc):
    if _names(func.ops) != ["ppl.gather"]:
        return None
    out, param, index, rows = func.ops[0].args
    _require(all(_is_param(b, func) for b in (out, param, index)), "gather operates on kernel parameters")
    _require(rows == param.shape[0], "gather: param_h must equal the number of rows of Param")
    i_o, i_p, i_i = out.param_index, param.param_index, index.param_index
    from .. import ops as native

    def run(*t):
        return native.gather_rows(t[i_p], t[i_i], t[i_o])

    return BoundKernel("gather", "tl_b200_gather_rows", run,
                       dict(rows=rows, hidden=param.shape[1], n=out.shape[0], dtype=param.dtype))


def _match_elementwise(func: PrimFunc):
    n = _names(func.ops)
    from .. import ops as native
    if n == ["ppl.copy", "ppl.sigmoid", "ppl.copy"]:
        ld, sg, st = func.ops
        if not (sg.args[1] is _buf(ld.args[1]) and _buf(st.args[0]) is sg.args[0]):
            return None
        X, Y = _buf(ld.args[0]), _buf(st.args[1])
        _require(X.shape == Y.shape, "sigmoid: equal shapes")
        ix, iy = X.param_index, Y.param_index
        return BoundKernel("sigmoid", "tl_b200_unary", lambda *t: native.unary(t[ix], t[iy], "sigmoid"),
                           dict(shape=list(X.shape), dtype=X.dtype))
    binary = {"ppl.add": "add", "ppl.sub": "sub", "ppl.mul": "mul", "ppl.div": "div"}
    if len(n) == 4 and n[0] == n[1] == n[3] == "ppl.copy" and n[2] in binary:
        la, lb, op, st = func.ops
        if not (op.args[1] is _buf(la.args[1]) and op.args[2] is _buf(lb.args[1]) and _buf(st.args[0]) is op.args[0]):
            return None
        A, B, C = _buf(la.args[0]), _buf(lb.args[0]), _buf(st.args[1])
        if not (A.shape == B.shape == C.shape and A.dtype == B.dtype == C.dtype and len(A.shape) == 2):
            return None                 # e.g. an (N, 1) operand: the generic executor broadcasts it
        name = binary[n[2]]
        ia, ib, ic = A.param_index, B.param_index, C.param_index
        return BoundKernel(f"elementwise_{name}", "tl_b200_binary", lambda *t: native.binary(t[ia], t[ib], t[ic], name),
                           dict(shape=list(A.shape), dtype=A.dtype))
    return None


_FA_PROLOGUE = ["ppl.copy", "ppl.fill", "ppl.fill", "ppl.fill"]
_FA_LOOP = ["ppl.copy", "ppl.fill", "ppl.gemm",                                   # S = Q K^T
            "ppl.copy", "ppl.fill", "ppl.reduce_max", "ppl.sub", "ppl.mul_C", "ppl.exp",
            "ppl.sub", "ppl.mul_C", "ppl.exp", "ppl.reduce_sum", "ppl.mul", "ppl.add", "ppl.copy",
            "ppl.mul",                                                           # rescale O
            "ppl.copy", "ppl.gemm"]                                              # O += P V
_FA_EPILOGUE = ["ppl.div", "ppl.copy", "ppl.copy"]


def _match_flash_attention(func: PrimFunc):
    n = _names(func.ops)
    want = _FA_PROLOGUE + ["loop.begin"] + _FA_LOOP + ["loop.end"] + _FA_EPILOGUE
    if n != want or len(func.params) != 4:
        return None
    ops = func.ops
    ld_q = ops[0]
    loop = ops[4]
    body = ops[5:5 + len(_FA_LOOP)]
    ld_k, _, qk = body[0], body[1], body[2]
    mul_scale = body[7]
    ld_v, pv = body[17], body[18]
    store = ops[-1]
    Q, K, V, O = _buf(ld_q.args[0]), _buf(ld_k.args[0]), _buf(ld_v.args[0]), _buf(store.args[1])
    if not all(_is_param(b, func) for b in (Q, K, V, O)):
        return None
    _require(qk.attrs["transpose_B"] and not pv.attrs["transpose_B"], "flash attention: S = Q K^T, O += P V")
    _require(len(Q.shape) == 4 and Q.shape == O.shape and K.shape == V.shape, "flash attention: bshd tensors")
    batch, seq_q, heads, dim = Q.shape
    seq_k = K.shape[1]
    bm = _buf(ld_q.args[1]).shape[0]
    bn = _buf(ld_k.args[1]).shape[0]
    _check_tiling(func, "flash attention", [(seq_q, bm), (seq_k, bn)])
    # dataflow of the loop body (a program with these op names but other operands is not attention and goes
    # to the tile-op executor): S = Q K^T; m = rowmax(S); alpha = exp((m_prev - m) c); P = exp((S - m) c);
    # l = l alpha + rowsum(P); O = O alpha + P V; after the loop O / l
    q_t, k_t, s_t = qk.args
    (cp_prev, fill_m, rmax, sub_a, mul_a, exp_a, sub_s, mul_s, exp_s, rsum, mul_l, add_l, cast_p) = body[3:16]
    resc = body[16]
    v_t, o_acc = pv.args[1], pv.args[2]
    m_prev, m_cur = _buf(cp_prev.args[1]), _buf(cp_prev.args[0])
    alpha, l_sum = sub_a.args[0], mul_l.args[0]
    div, cast_o = ops[-3], ops[-2]
    flow = (q_t is _buf(ld_q.args[1]) and k_t is _buf(ld_k.args[1]) and body[1].args[0] is s_t and body[1].args[1] == 0.0
            and fill_m.args[0] is m_cur and fill_m.args[1] == -math.inf and rmax.args[0] is s_t and rmax.args[1] is m_cur
            and sub_a.args[1] is m_prev and sub_a.args[2] is m_cur and mul_a.args[0] is alpha and mul_a.args[1] is alpha
            and exp_a.args[0] is alpha
            and sub_s.args[0] is s_t and sub_s.args[1] is s_t and sub_s.args[2] is m_cur
            and mul_s.args[0] is s_t and mul_s.args[1] is s_t and exp_s.args[0] is s_t
            and rsum.args[0] is s_t and mul_l.args[1] is l_sum and mul_l.args[2] is alpha
            and add_l.args[0] is l_sum and add_l.args[1] is l_sum and add_l.args[2] is rsum.args[1]
            and _buf(cast_p.args[0]) is s_t and pv.args[0] is _buf(cast_p.args[1])
            and resc.args[0] is o_acc and resc.args[1] is o_acc and resc.args[2] is alpha
            and v_t is _buf(ld_v.args[1])
            and div.args[0] is o_acc and div.args[1] is o_acc and div.args[2] is l_sum
            and _buf(cast_o.args[0]) is o_acc and _buf(store.args[0]) is _buf(cast_o.args[1]))
    if not flow:
        return None
    _require(_close(float(mul_a.args[2]), float(mul_s.args[2])), "flash attention: one softmax scale for the row maxima and the scores")
    scale = float(mul_s.args[2])
    # tensor addressing: Q[bz, bx*bm : +bm, by, :], K/V[bz, k*bn : +bn, by, :], Output like Q
    qr, kr, vr, orr = ld_q.args[0], ld_k.args[0], ld_v.args[0], store.args[1]
    kvar = loop.args[0]
    bx = qr.starts[1].affine()
    _require(bx is not None and len(bx[0]) == 1 and bx[1] == 0 and list(bx[0].values()) == [bm],
             "flash attention: the query block must start at bx * block_M")
    bxv = next(iter(bx[0]))
    ka = kr.starts[1].affine()
    _require(ka is not None and ka[1] == 0 and {id(v): c for v, c in ka[0].items()} == {id(kvar): bn}
             and _same_expr(kr.starts[1], vr.starts[1]), "flash attention: K and V tiles must start at k * block_N")
    _require(all(_same_expr(qr.starts[i], r.starts[i]) for r in (kr, vr, orr) for i in (0, 2))
             and _same_expr(qr.starts[1], orr.starts[1]), "flash attention: Q, K, V and Output must address the same batch entry and head")
    extent = loop.args[1]
    full = -(-seq_k // bn)
    if const_value(extent) is not None:
        _require(const_value(extent) == full, "flash attention: the KV loop must cover the sequence")
        mode, diag = "none", 0
    else:
        # min(ceil(S/bn), ceil((bx+1)*bm / bn)): the reference's shortened causal loop; it does
        # NOT mask inside the last tile, so a query sees every key of that tile.
        _require(isinstance(extent, Call) and extent.fn == "min" and len(extent.args) == 2,
                 "flash attention: unrecognised KV loop extent")
        consts = [a for a in extent.args if const_value(a) is not None]
        calls = [a for a in extent.args if isinstance(a, Call) and a.fn == "ceildiv"]
        _require(len(consts) == 1 and const_value(consts[0]) == full and len(calls) == 1,
                 "flash attention: the causal KV loop must be min(ceil(S / block_N), ceil((bx + 1) * block_M / block_N))")
        num, den = calls[0].args
        na = num.affine()
        _require(const_value(den) == bn and na is not None and na[1] == bm
                 and {id(v): c for v, c in na[0].items()} == {id(bxv): bm},
                 "flash attention: the causal KV loop must be min(ceil(S / block_N), ceil((bx + 1) * block_M / block_N))")
        mode, diag = "block", 0
    idx = [b.param_index for b in (Q, K, V, O)]
    from .. import ops as native

    def run(*t):
        return native.flash_attn_fwd(t[idx[0]], t[idx[1]], t[idx[2]], t[idx[3]], scale=scale, causal=mode,
                                     block_m=bm, block_n=bn)

    return BoundKernel("flash_attention_fwd", "tl_b200_flash_attn_fwd", run,
                       dict(batch=batch, heads=heads, seq_q=seq_q, seq_kv=seq_k, dim=dim, scale=scale, causal=mode,
                            block_M=bm, block_N=bn, dtype=Q.dtype))


def _match_mla_decode(func: PrimFunc):
    n = _names(func.ops)
    if len(func.params) != 5 or n.count("ppl.gemm") != 3 or n.count("loop.begin") != 1:
        return None
    if n[:5] != ["ppl.copy", "ppl.copy", "ppl.fill", "ppl.fill", "ppl.fill"] or n[-3:] != ["ppl.div", "ppl.copy", "ppl.copy"]:
        return None
    ops = func.ops
    gemms = [o for o in ops if o.name == "ppl.gemm"]
    if not (gemms[0].attrs["transpose_B"] and gemms[1].attrs["transpose_B"] and not gemms[2].attrs["transpose_B"]):
        return None
    loop_i = n.index("loop.begin")
    ld_kv, ld_kpe = ops[loop_i + 1], ops[loop_i + 2]
    Q, Qpe = _buf(ops[0].args[0]), _buf(ops[1].args[0])
    KV, Kpe, Out = _buf(ld_kv.args[0]), _buf(ld_kpe.args[0]), _buf(ops[-1].args[1])
    if not all(_is_param(b, func) for b in (Q, Qpe, KV, Kpe, Out)):
        return None
    _require(gemms[2].args[1] is gemms[0].args[1], "mla decode: V must be the latent KV tile")
    # dataflow: S = Q KV^T + Q_pe K_pe^T (two products summed), P = exp(S c - m c) cast into the A operand of
    # O += P KV, O rescaled by exp(m_prev c - m c), O / l at the end; everything else goes to the executor
    body = ops[loop_i + 1:n.index("loop.end")]
    bn_ = _names(body)
    q_t, kv_t, s_t = gemms[0].args
    qpe_t, kpe_t, s_pe = gemms[1].args
    p_t, _, o_acc = gemms[2].args
    adds = [o for o in body if o.name == "ppl.add"]
    exps = [o for o in body if o.name == "ppl.exp"]
    rmax = next((o for o in body if o.name == "ppl.reduce_max"), None)
    rsum = next((o for o in body if o.name == "ppl.reduce_sum"), None)
    casts = [o for o in body if o.name == "ppl.copy" and _buf(o.args[1]) is p_t]
    div = ops[-3]
    flow = (bn_.count("ppl.exp") == 2 and rmax is not None and rsum is not None and len(adds) == 2 and len(casts) == 1
            and q_t is _buf(ops[0].args[1]) and qpe_t is _buf(ops[1].args[1])
            and kv_t is _buf(ld_kv.args[1]) and kpe_t is _buf(ld_kpe.args[1])
            and adds[0].args[0] is s_t and {id(adds[0].args[1]), id(adds[0].args[2])} == {id(s_t), id(s_pe)}
            and rmax.args[0] is s_t and exps[1].args[0] is s_t and rsum.args[0] is s_t and _buf(casts[0].args[0]) is s_t
            and adds[1].args[2] is rsum.args[1]
            and div.args[0] is o_acc and div.args[1] is o_acc and div.args[2] is adds[1].args[0]
            and any(o.name == "ppl.mul" and o.args[0] is o_acc and o.args[1] is o_acc and o.args[2] is exps[0].args[0] for o in body))
    if not flow:
        return None
    b, h, one, dim = Q.shape
    pe = Qpe.shape[-1]
    s = KV.shape[1]
    _require(one == 1 and KV.shape[2] == 1, "mla decode: one query token, one latent kv head")
    scales = {float(o.args[2]) for o in ops if o.name == "ppl.mul_C"}
    _require(len(scales) == 1, "mla decode: a single softmax scale is expected")
    scale = scales.pop()
    idx = [x.param_index for x in (Q, Qpe, KV, Kpe, Out)]
    from .. import ops as native

    def run(*t):
        return native.mla_decode_dense(t[idx[0]], t[idx[1]], t[idx[2]], t[idx[3]], t[idx[4]], scale=scale)

    return BoundKernel("mla_decode", "tl_b200_mla_decode_dense", run,
                       dict(batch=b, heads=h, seqlen_kv=s, dim=dim, pe_dim=pe, scale=scale, dtype=Q.dtype))


def _match_library_program(func: PrimFunc):
    """Programs of `tilelang.programs` that name the library kernel implementing them."""
    kernel = func.attrs.get("library_kernel")
    if kernel is None:
        return None
    facts = dict(func.attrs.get("facts", {}))
    from .. import ops as native
    if kernel == "gemm_fp8_blockscale":
        return BoundKernel("gemm_fp8_blockscale", "tl_b200_gemm_fp8_blockscale",
                           lambda a8, b8, sa, sb, c: native.gemm_fp8_blockscale(a8, b8, sa, sb, c), facts)
    if kernel == "mla_decode_paged":
        scale, dv = facts["softmax_scale"], facts["dv"]
        if facts["scaled"]:
            def run(q, kv, kvs, table, lens, out):
                return native.mla_decode_paged(q, kv, kvs, table, lens, out, dv=dv, softmax_scale=scale)
        else:
            def run(q, kv, table, lens, out):
                return native.mla_decode_paged(q, kv, None, table, lens, out, dv=dv, softmax_scale=scale)
        return BoundKernel("mla_decode_paged", "tl_b200_mla_decode_paged", run, facts)
    if kernel == "mlp":
        return BoundKernel("mlp", "tl_b200_mlp_gate_up + tl_b200_gemm",
                           lambda out, x, wg, wu, wd: native.mlp(x, wg, wu, wd, out), facts)
    raise UnsupportedProgram(f"unknown library kernel {kernel!r}")


_MATCHERS = [_match_library_program, _match_matmul, _match_rmsnorm, _match_rope, _match_swiglu, _match_mlp, _match_reduce, _match_topk, _match_gather,
             _match_elementwise, _match_flash_attention, _match_mla_decode]


def bind(func: PrimFunc) -> BoundKernel:
    """Recognise `func` and bind it to its CUDA program; raises UnsupportedProgram otherwise."""
    for m in _MATCHERS:
        bound = m(func)
        if bound is not None:
            return bound
    # not one of the hand-fused programs.  A row-local program runs as ONE launch of the tile-program kernel
    # (engine/fuser.py); anything else is run tile op by tile op on the GPU (engine/interpreter.py)
    from . import fuser, interpreter
    fused = fuser.build(func)
    if fused is not None:
        entry = ("kernel generated for the program (NVRTC, one launch)" if getattr(fused, "generated", False)
                 else "tl_b200_tile_program (one launch)")
        return BoundKernel("generic", entry, fused,
                           dict(ops=len(func.ops), instructions=fused.instructions, grid=[int(const_value(g)) for g in func.grid],
                                fused=True, generated=bool(getattr(fused, "generated", False))), full_outputs=False)
    try:
        run = interpreter.build(func)
    except interpreter.InterpreterError as why:
        reason = str(why)
    else:
        return BoundKernel("generic", "tile-op executor (one tl_b200_* launch per op)", run,
                           dict(ops=len(func.ops), grid=[int(const_value(g)) for g in func.grid], fused=False,
                                why_not_fused=fuser.build.last_reason), full_outputs=False)
    raise UnsupportedProgram(
        f"the generic tile-op executor cannot run it either ({reason}); "
        "this ppl_* program does not match any kernel of the b200 library (matmul, rmsnorm, "
        "rmsnorm split-K, rope, swiglu, gated MLP, row reduce, top-k, gather, sigmoid, elementwise, flash "
        "attention forward, MLA decode); there is no CPU fallback.  Recorded program:\n" + func.script())
