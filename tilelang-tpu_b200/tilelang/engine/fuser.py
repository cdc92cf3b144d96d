"""Fusion of row-local tile programs into ONE kernel launch.

A `ppl_*` program whose every op works row by row (loads / stores / casts, fill, add / sub / mul / div with a
full, (M,1) or (1,N) second operand, mul_C / add_C, exp, sigmoid, rsqrt, row sum / max, rope_add) is lowered
here to the instruction list of the accumulator machine in csrc/tile_vm.cu (`tl_b200_tile_program`): tiles
become tile registers (one row per thread group), (M,1) tiles become per-row scalars, the launch grid and the
rows of a block are walked inside the kernel, loops with constant extents are unrolled, and windows of tensors
of any rank become `base + coef . block + row * row_stride` addressing (rank-1 -> {1,1,1,W}, rank-2 -> {1,C,1,W},
rank-3 -> {N,C,1,W} in the reference's code generator, src/target/codegen_ppl.cc:802-829; here any window whose
rows are evenly strided and whose columns are contiguous is taken).

The reference executes the same program as one runtime call per op (codegen_ppl.cc:879-1906); arithmetic rules
are kept: fp32 evaluation, every result rounded to its tile's type, scalars cast to the tile's type first.
A program with an op that is not row-local (gemm, gather, top-k) is left to the op-by-op executor.
"""
from __future__ import annotations

import ctypes
import os
from typing import Callable, Dict, List, Optional

import torch

from ..language.ir import Buffer, Expr, PrimFunc, Region, const_value

(LD_A, ST_A, LD_S, ST_S, MOV_A_T, MOV_T_A, BIN_A_T, BIN_A_S, BIN_A_I, UN_A, FILL_A, ROUND_A, BCAST_A_S, RED_S, MOV_S_I,
 MOV_S_S, BIN_S_S, BIN_S_I, UN_S, ROPE_A) = range(20)
MAX_INSTR, MAX_PARAMS, SCALARS, MAX_WIDTH = 96, 16, 8, 8192
_BIN = {"ppl.add": 0, "ppl.sub": 1, "ppl.mul": 2, "ppl.div": 3}
_CONST = {"ppl.add_C": 0, "ppl.mul_C": 2}
_DT = {"float32": 0, "float": 0, "float16": 1, "half": 1, "bfloat16": 2}
_TORCH = {"float32": torch.float32, "float": torch.float32, "float16": torch.float16, "half": torch.float16,
          "bfloat16": torch.bfloat16}


class Instr(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int32), ("sub", ctypes.c_int32), ("r0", ctypes.c_int32), ("r1", ctypes.c_int32),
                ("r2", ctypes.c_int32), ("r3", ctypes.c_int32), ("dtype", ctypes.c_int32), ("width", ctypes.c_int32),
                ("param", ctypes.c_int32), ("row_stride", ctypes.c_int32), ("vec", ctypes.c_int32), ("imm", ctypes.c_float),
                ("base", ctypes.c_int64), ("coef", ctypes.c_int64 * 3)]


class NotFusable(Exception):
    pass


def _need(cond, why):
    if not cond:
        raise NotFusable(why)


def _round_imm(value: float, dtype: str) -> float:
    """A scalar operand is cast to the tile's type before it is used (codegen_ppl.cc:917-957)."""
    return float(torch.tensor(float(value), dtype=torch.float32).to(_TORCH[dtype]).float())


def _unroll(func: PrimFunc):
    """Flat list of (op, env) with constant-extent loops unrolled; env maps loop variables to integers."""
    out: list = []

    def walk(lo, hi, env):
        i = lo
        while i < hi:
            op = func.ops[i]
            if op.name == "loop.begin":
                extent = const_value(op.args[1])
                _need(extent is not None, "loop extent is not a constant")
                depth, j = 1, i + 1
                while depth:
                    depth += {"loop.begin": 1, "loop.end": -1}.get(func.ops[j].name, 0)
                    j += 1
                for it in range(int(extent)):
                    walk(i + 1, j - 1, {**env, op.args[0]: it})
                    _need(len(out) <= 4 * MAX_INSTR, "program too long to unroll")
                i = j
                continue
            out.append((op, env))
            i += 1

    walk(0, len(func.ops), {})
    return out


def _affine(e, env, block_vars):
    """(constant, [coefficient per block variable]) of an index expression; loop variables are in env."""
    if not isinstance(e, Expr):
        return int(e), [0] * len(block_vars)
    f = e.affine()
    _need(f is not None, f"index {e!r} is not affine")
    const, coefs = int(f[1]), [0] * len(block_vars)
    for v, c in f[0].items():
        if v in env:
            const += int(c) * int(env[v])
            continue
        hit = [i for i, b in enumerate(block_vars) if b is v]
        _need(bool(hit), f"index {e!r} uses a variable that is neither a block index nor a loop variable")
        coefs[hit[0]] += int(c)
    return const, coefs


def _window(region: Region, rows: int, width: int, env, block_vars):
    """Addressing of a (rows, width) tile against a window of a global tensor: element (r, c) lies at
    base + coef . block + r * row_stride + c (in elements)."""
    buf = region.buffer
    strides, acc = [], 1
    for s in reversed(buf.shape):
        strides.append(acc)
        acc *= int(s)
    strides.reverse()
    base, coef = 0, [0] * len(block_vars)
    dims = []                                    # non-unit dims of the window: (extent, stride, full extent of the tensor dim)
    for d, (st, ex) in enumerate(zip(region.starts, region.extents)):
        c0, cs = _affine(st, env, block_vars)
        base += c0 * strides[d]
        coef = [a + b * strides[d] for a, b in zip(coef, cs)]
        ex = 1 if ex is None else int(ex)
        if ex != 1:
            dims.append((ex, strides[d], int(buf.shape[d])))
    total = 1
    for ex, _, _ in dims:
        total *= ex
    _need(total == rows * width, f"window of {buf.name} holds {total} elements, the tile {rows} x {width}")
    # innermost dims make up the columns: they must be contiguous in memory
    cols, k = 1, len(dims)
    while cols < width:
        _need(k > 0, "window cannot be split into rows and columns")
        k -= 1
        ex, st, _ = dims[k]
        _need(st == cols, f"columns of the window of {buf.name} are not contiguous")
        cols *= ex
    _need(cols == width, f"window of {buf.name} does not split into rows of {width}")
    row_dims = dims[:k]
    if not row_dims:
        row_stride = 0
    else:
        row_stride = row_dims[-1][1]
        run = row_dims[-1][0] * row_stride
        for ex, st, _ in reversed(row_dims[:-1]):
            _need(st == run, f"rows of the window of {buf.name} are not evenly strided")
            run = ex * st
    _need(abs(row_stride) < 2 ** 31, "row stride too large")
    return base, coef, row_stride


class _Compiler:
    def __init__(self, func: PrimFunc):
        self.func = func
        self.flat = _unroll(func)
        self.block_vars = list(func.block_vars)
        _need(len(self.block_vars) <= 3, "more than three grid dimensions")
        self.ins: List[Instr] = []
        self.kind: Dict[int, str] = {}           # id(tile) -> "full" | "col"
        self.tiles: Dict[int, Buffer] = {}
        self.bm = self._classify()
        from .. import _native
        self.max_width = max([self._shape2(t)[1] for t in self.tiles.values() if self.kind[id(t)] == "full"] or [1])
        _need(self.max_width <= MAX_WIDTH, f"tile width {self.max_width} above {MAX_WIDTH}")
        self.nt = int(_native.load().tl_b200_tile_program_registers(self.max_width))
        self.treg: Dict[int, int] = {}
        self.sreg: Dict[int, int] = {}
        self.free_t = list(range(self.nt))
        self.free_s = list(range(SCALARS))
        self.last_use = self._liveness()
        self.pos = 0
        self.mem_instrs: List[int] = []
        self.a_holds = None                      # id of the tile whose row the accumulator currently equals

    # ---------------------------------------------------------------- tiles
    @staticmethod
    def _shape2(t: Buffer):
        s = tuple(int(x) for x in t.shape)
        if len(s) == 1:
            return (1, s[0])
        _need(len(s) == 2, f"tile {t.name} has rank {len(s)}")
        return s

    def _operands(self, op):
        """The tiles an op really reads or writes (the scratch operands of exp / sigmoid are unused)."""
        n, a = op.name, op.args
        if n == "ppl.exp":
            return [a[0]]
        if n == "ppl.sigmoid":
            return [a[0], a[1]]
        return [x for x in a if isinstance(x, (Buffer, Region))]

    def _classify(self) -> int:
        rows = set()
        for op, _ in self.flat:
            _need(op.name in _BIN or op.name in _CONST or op.name in ("ppl.copy", "ppl.fill", "ppl.exp", "ppl.sigmoid", "ppl.rsqrt",
                                                                       "ppl.reduce_sum", "ppl.reduce_max", "ppl.rope_add"),
                  f"{op.name} is not a row-local op")
            for x in self._operands(op):
                b = x.buffer if isinstance(x, Region) else x
                if b.scope == "global":
                    _need(b.dtype in _DT, f"{b.name}: dtype {b.dtype}")
                    continue
                _need(b.dtype in _DT, f"tile {b.name}: dtype {b.dtype}")
                if isinstance(x, Region):
                    _need(all(const_value(s) == 0 for s in x.starts) and
                          all(e is None or int(e) == int(d) for e, d in zip(x.extents, b.shape)), "windows of tiles are not supported")
                self.tiles[id(b)] = b
                rows.add(self._shape2(b)[0])
        _need(bool(self.tiles), "no tiles")
        bm = max(rows)
        _need(rows <= {bm, 1}, f"tiles with different row counts {sorted(rows)}")
        for t in self.tiles.values():
            r, c = self._shape2(t)
            self.kind[id(t)] = "col" if (c == 1 and r == bm) else "full"
        return bm

    def _liveness(self):
        last = {}
        for i, (op, _) in enumerate(self.flat):
            for x in self._operands(op):
                b = x.buffer if isinstance(x, Region) else x
                if b.scope != "global":
                    last[id(b)] = i
        return last

    def _t(self, tile: Buffer, define: bool = False) -> int:
        k = id(tile)
        if k not in self.treg:
            _need(bool(self.free_t), f"more than {self.nt} tiles of width {self.max_width} live at once")
            self.free_t.sort()                   # lowest free register: programs with few live tiles fit the small variant
            self.treg[k] = self.free_t.pop(0)
        return self.treg[k]

    def _s(self, tile: Buffer) -> int:
        k = id(tile)
        if k not in self.sreg:
            _need(bool(self.free_s), f"more than {SCALARS} (M,1) tiles live at once")
            self.sreg[k] = self.free_s.pop(0)
        return self.sreg[k]

    def _release(self):
        for k, last in self.last_use.items():
            if last == self.pos:
                if k in self.treg:
                    self.free_t.append(self.treg.pop(k))
                if k in self.sreg:
                    self.free_s.append(self.sreg.pop(k))

    # ---------------------------------------------------------------- emission
    def emit(self, op, **f):
        ins = Instr()
        ins.op = op
        for k, v in f.items():
            if k == "coef":
                for i in range(3):
                    ins.coef[i] = v[i] if i < len(v) else 0
            else:
                setattr(ins, k, v)
        self.ins.append(ins)
        if op in (LD_A, BIN_A_T, BIN_A_S, BIN_A_I, UN_A, FILL_A, ROUND_A, BCAST_A_S, ROPE_A):
            self.a_holds = None
        return len(self.ins) - 1

    def is_col(self, t: Buffer) -> bool:
        return self.kind[id(t)] == "col"

    def width(self, t: Buffer) -> int:
        return self._shape2(t)[1]

    def load_a(self, t: Buffer):
        if self.is_col(t):
            self.emit(BCAST_A_S, r0=self._s(t))
            self.a_holds = None
        elif self.a_holds != id(t):              # MOV_T_A leaves the stored row in the accumulator
            self.emit(MOV_A_T, r0=self._t(t))
            self.a_holds = id(t)

    def store_a(self, t: Buffer):
        self.emit(MOV_T_A, r0=self._t(t, True), dtype=_DT[t.dtype])
        self.a_holds = id(t)

    def mem(self, op, region: Region, tile_rows, tile_width, env, reg=0):
        buf = region.buffer
        base, coef, row_stride = _window(region, tile_rows, tile_width, env, self.block_vars)
        _need(tile_rows in (1, self.bm), "window rows do not match the block")
        if tile_rows == 1 and self.bm > 1:
            _need(op in (LD_A, LD_S), "a single-row tile cannot be stored from a block of several rows")
            row_stride = 0
        esz_unit = 8 if _DT[buf.dtype] != 0 else 4
        vec = int(base % esz_unit == 0 and all(c % esz_unit == 0 for c in coef) and row_stride % esz_unit == 0)
        i = self.emit(op, r0=reg, dtype=_DT[buf.dtype], width=tile_width, param=buf.param_index, row_stride=row_stride,
                      vec=vec, base=base, coef=coef)
        self.mem_instrs.append(i)

    def compile(self):
        for self.pos, (op, env) in enumerate(self.flat):
            self.one(op, env)
            self._release()
        self._drop_dead_stores()
        _need(len(self.ins) <= MAX_INSTR, f"program needs more than {MAX_INSTR} instructions")
        return self

    def _drop_dead_stores(self):
        """A MOV_T_A whose tile register is overwritten (or never read) before its next use only rounds the
        accumulator: it becomes ROUND_A, or disappears when the tile is fp32."""
        live = set()
        keep = [True] * len(self.ins)
        for i in range(len(self.ins) - 1, -1, -1):
            ins = self.ins[i]
            if ins.op == MOV_T_A:
                if ins.r0 in live:
                    live.discard(ins.r0)
                elif ins.dtype == 0:
                    keep[i] = False
                else:
                    ins.op = ROUND_A
            elif ins.op in (MOV_A_T, BIN_A_T):
                live.add(ins.r0)
            elif ins.op == ROPE_A:
                live.update((ins.r0, ins.r1, ins.r2, ins.r3))
        remap, out = {}, []
        for i, ins in enumerate(self.ins):
            if keep[i]:
                remap[i] = len(out)
                out.append(ins)
        self.mem_instrs = [remap[i] for i in self.mem_instrs]
        self.ins = out

    def one(self, op, env):
        n, a = op.name, op.args
        if n == "ppl.copy":
            src, dst = a
            sb, db = src.buffer, dst.buffer
            if sb.scope == "global" and db.scope != "global":
                r, w = self._shape2(db)
                if self.is_col(db):
                    self.mem(LD_S, src, r, 1, env, reg=self._s(db))
                    if _DT[db.dtype] != _DT[sb.dtype]:
                        self.emit(MOV_S_S, r0=self._s(db), r1=self._s(db), dtype=_DT[db.dtype])
                else:
                    self.mem(LD_A, src, r, w, env)
                    self.store_a(db)
            elif sb.scope != "global" and db.scope == "global":
                r, w = self._shape2(sb)
                if self.is_col(sb):
                    self.mem(ST_S, dst, r, 1, env, reg=self._s(sb))
                else:
                    self.load_a(sb)
                    self.mem(ST_A, dst, r, w, env)
            elif sb.scope != "global":
                _need(self._shape2(sb) == self._shape2(db) or (self.is_col(sb) and self.is_col(db)), "tile copy between different shapes")
                if self.is_col(sb) and self.is_col(db):
                    self.emit(MOV_S_S, r0=self._s(db), r1=self._s(sb), dtype=_DT[db.dtype])
                else:
                    _need(not self.is_col(sb) and not self.is_col(db), "copy between a column tile and a full tile")
                    self.load_a(sb)
                    self.store_a(db)
            else:
                raise NotFusable("copy between two global tensors")
        elif n == "ppl.fill":
            t, v = a
            imm = _round_imm(v, t.dtype)
            if self.is_col(t):
                self.emit(MOV_S_I, r0=self._s(t), imm=imm)
            else:
                self.emit(FILL_A, imm=imm)
                self.store_a(t)
        elif n in _BIN:
            out, x, y = a
            _need(out.dtype == x.dtype == y.dtype, f"{n}: operands of different types")
            if self.is_col(out):
                _need(self.is_col(x) and self.is_col(y), f"{n}: (M,1) result from wider operands")
                self.emit(BIN_S_S, sub=_BIN[n], r0=self._s(out), r1=self._s(x), r2=self._s(y), dtype=_DT[out.dtype])
                return
            _need(not self.is_col(x) and self._shape2(out) == self._shape2(x), f"{n}: out and in1 must have one shape")
            self.load_a(x)
            if self.is_col(y):
                self.emit(BIN_A_S, sub=_BIN[n], r0=self._s(y))
            else:
                ys = self._shape2(y)
                _need(ys == self._shape2(x) or ys == (1, self.width(x)), f"{n}: in2 must be shaped like in1, (M,1) or (1,N)")
                self.emit(BIN_A_T, sub=_BIN[n], r0=self._t(y))
            self.store_a(out)
        elif n in _CONST:
            out, x, c = a
            imm = _round_imm(c, x.dtype)
            if self.is_col(out):
                _need(self.is_col(x), f"{n}: (M,1) result from a wider operand")
                self.emit(BIN_S_I, sub=_CONST[n], r0=self._s(out), r1=self._s(x), imm=imm, dtype=_DT[out.dtype])
                return
            self.load_a(x)
            self.emit(BIN_A_I, sub=_CONST[n], imm=imm)
            self.store_a(out)
        elif n in ("ppl.exp", "ppl.sigmoid", "ppl.rsqrt"):
            sub = {"ppl.sigmoid": 0, "ppl.exp": 1, "ppl.rsqrt": 2}[n]
            out, x = (a[0], a[0]) if n == "ppl.exp" else (a[0], a[1])
            if self.is_col(out):
                _need(self.is_col(x), f"{n}: (M,1) result from a wider operand")
                self.emit(UN_S, sub=sub, r0=self._s(out), r1=self._s(x), dtype=_DT[out.dtype])
                return
            self.load_a(x)
            self.emit(UN_A, sub=sub)
            self.store_a(out)
        elif n in ("ppl.reduce_sum", "ppl.reduce_max"):
            x, y = a[0], a[1]
            _need(not self.is_col(x) and self.is_col(y), f"{n}: (M,N) -> (M,1)")
            self.load_a(x)
            if n == "ppl.reduce_sum":
                self.emit(RED_S, sub=0, r0=self._s(y), width=self.width(x), dtype=_DT[y.dtype])
            else:                                   # the running maximum: out = max(out, row maxima)
                _need(bool(self.free_s), "no scalar register left for the row maximum")
                tmp = self.free_s[0]
                self.emit(RED_S, sub=1, r0=tmp, width=self.width(x), dtype=_DT[y.dtype])
                self.emit(BIN_S_S, sub=4, r0=self._s(y), r1=self._s(y), r2=tmp, dtype=_DT[y.dtype])
        elif n == "ppl.rope_add":
            out, e1, e2, o1, o2 = a
            _need(all(not self.is_col(t) and self._shape2(t) == self._shape2(out) and t.dtype == out.dtype for t in a)
                  and self.width(out) % 2 == 0, "rope_add: five tiles of one shape and type, even width")
            self.emit(ROPE_A, r0=self._t(e1), r1=self._t(e2), r2=self._t(o1), r3=self._t(o2))
            self.store_a(out)
        else:
            raise NotFusable(n)


def build(func: PrimFunc) -> Optional[Callable[..., int]]:
    """run(*device_tensors) -> int launching the whole program as one kernel, or None if it is not row-local."""
    try:
        grid = [const_value(g) for g in func.grid]
        _need(all(g is not None for g in grid) and 1 <= len(grid) <= 3, "the launch grid must be static, 1 to 3 dimensions")
        _need(len(func.params) <= MAX_PARAMS, "too many parameters")
        c = _Compiler(func).compile()
    except NotFusable as why:
        build.last_reason = str(why)
        return None
    grid = [int(g) for g in grid] + [1] * (3 - len(grid))
    n = len(c.ins)
    table = (Instr * n)(*c.ins)
    static_vec = [c.ins[i].vec for i in c.mem_instrs]
    n_params = len(func.params)
    from .. import _native as N
    from .. import ops as K

    def run(*tensors):
        stream = K._prepare(*tensors)
        ptrs = (ctypes.c_void_p * n_params)(*[t.data_ptr() for t in tensors])
        aligned = [t.data_ptr() % 16 == 0 for t in tensors]
        for i, v in zip(c.mem_instrs, static_vec):
            table[i].vec = int(v and aligned[table[i].param])
        return N.check(N.load().tl_b200_tile_program(table, n, ptrs, n_params, grid[0], grid[1], grid[2], c.bm,
                                                    c.max_width, stream), "tl_b200_tile_program")

    run.instructions = n
    run.rows_per_block = c.bm
    run.max_width = c.max_width
    run.generated = False
    # The same instruction list as a kernel generated for this program (engine/codegen.py); the interpreter above stays
    # the path when NVRTC cannot be used, or when TILELANG_B200_TILE_PROGRAM=interpreter asks for it.
    if os.environ.get("TILELANG_B200_TILE_PROGRAM", "generated") != "interpreter":
        from . import codegen
        try:
            gen = codegen.build(c.ins, c.mem_instrs, n_params, grid, c.bm, c.max_width)
        except codegen.Unavailable as why:
            build.last_reason = f"generated kernel unavailable ({why}); interpreted"
        else:
            gen.instructions, gen.rows_per_block, gen.max_width, gen.generated = n, c.bm, c.max_width, True
            gen.interpreted = run
            return gen
    return run


build.last_reason = ""
