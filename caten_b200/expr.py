"""Generic schedule items on the B200: build an expression over the reference's aIR ops
(source/aasm/attrs.lisp:42-216), compile it to the postfix program ``caten_b200_eval_expr``
interprets, and run it over strided views (source/aasm/attrs.lisp:265-283).

This is the host-side counterpart of what the reference does per fused Schedule-Item: render the
:EXPR nodes to C (source/codegen/renderer.lisp:331-410), compile and call
(source/byoc/clang.lisp:163-205).  Operators follow the reference's composition rules: ``a - b``
is ``a + (-b)`` and ``a / b`` is ``a * recip(b)`` (source/api/function.lisp:525-547), ``<`` and
``!=`` give booleans, ``where`` selects.

    x, y = View.of(bx), View.of(by)
    run(rt, maximum(load(x) * const(2.0) + load(y), const(0.0)), View.of(out))      # relu(2x + y)
    run(rt, load(x), View.of(rowsum, strides=(1, 0)), shape=(R, C), n_reduce=1, reduce_op="sum")
"""
from __future__ import annotations

import ctypes as C
import struct
from typing import List, Optional, Sequence

import numpy as np

from . import _lib as L

F32, I32, BOOL = 0, 1, 2
DT_OF = {np.dtype(np.float32): (0, F32), np.dtype(np.int32): (1, I32), np.dtype(np.int64): (2, I32),
         np.dtype(np.uint8): (3, BOOL), np.dtype(np.bool_): (3, BOOL)}
OP = {"LOAD": 1, "CONST": 2, "INDEX": 3, "NEG": 10, "RECIP": 11, "SIN": 12, "EXP2": 13, "LOG2": 14, "SQRT": 15, "NOT": 16,
      "CAST": 17, "ADD": 30, "MUL": 31, "MOD": 32, "IDIV": 33, "AND": 34, "OR": 35, "XOR": 36, "MAX": 37, "NE": 38, "LT": 39,
      "WHERE": 50}
UNARY = ("NEG", "RECIP", "SIN", "EXP2", "LOG2", "SQRT", "NOT", "CAST")
BINARY = ("ADD", "MUL", "MOD", "IDIV", "AND", "OR", "XOR", "MAX", "NE", "LT")
RED = {None: 0, "sum": 1, "max": 2}


class View:
    """A buffer seen through element strides per loop (0 = broadcast) and an element offset."""

    def __init__(self, buf, strides: Optional[Sequence[int]] = None, offset: int = 0):
        self.buf, self.offset = buf, int(offset)
        if strides is None:  # contiguous over the buffer's own shape
            strides, acc = [], 1
            for n in reversed(buf.shape):
                strides.append(acc)
                acc *= n
            strides = list(reversed(strides))
        self.strides = tuple(int(s) for s in strides)

    @staticmethod
    def of(buf, strides=None, offset=0) -> "View":
        return View(buf, strides, offset)


class Node:
    def __init__(self, op: str, args=(), cls: int = F32, value=None):
        self.op, self.args, self.cls, self.value = op, tuple(args), cls, value

    # the reference's composition rules
    def __add__(self, o): return add(self, _lift(o, self.cls))
    def __radd__(self, o): return add(_lift(o, self.cls), self)
    def __mul__(self, o): return mul(self, _lift(o, self.cls))
    def __rmul__(self, o): return mul(_lift(o, self.cls), self)
    def __neg__(self): return neg(self)
    def __sub__(self, o): return add(self, neg(_lift(o, self.cls)))
    def __rsub__(self, o): return add(_lift(o, self.cls), neg(self))
    def __truediv__(self, o): return mul(self, recip(_lift(o, self.cls)))
    def __lt__(self, o): return lt(self, _lift(o, self.cls))
    def __gt__(self, o): return lt(_lift(o, self.cls), self)


def _lift(x, cls) -> Node:
    return x if isinstance(x, Node) else const(x, cls)


def load(view: View) -> Node:
    return Node("LOAD", cls=DT_OF[np.dtype(view.buf.dtype)][1], value=view)


def const(v, cls: Optional[int] = None) -> Node:
    if cls is None:
        cls = BOOL if isinstance(v, (bool, np.bool_)) else I32 if isinstance(v, (int, np.integer)) else F32
    return Node("CONST", cls=cls, value=v)


def index(axis: int) -> Node:
    return Node("INDEX", cls=I32, value=int(axis))


def _same(a: Node, b: Node, what: str):
    if a.cls != b.cls:
        raise TypeError(f"{what}: operand classes differ ({a.cls} vs {b.cls}); insert cast() as the reference's graph does")


def _unary(name, float_only=False):
    def f(a: Node) -> Node:
        if float_only and a.cls != F32:
            raise TypeError(f"{name} takes a float operand")
        return Node(name, (a,), BOOL if name == "NOT" else a.cls)
    return f


def _binary(name, int_only=False, boolean=False):
    def f(a: Node, b: Node) -> Node:
        _same(a, b, name)
        if int_only and a.cls == F32:
            raise TypeError(f"{name} takes integer operands")
        return Node(name, (a, b), BOOL if boolean else a.cls)
    return f


neg, recip, not_ = _unary("NEG"), _unary("RECIP"), _unary("NOT")
sin, exp2, log2, sqrt = _unary("SIN", True), _unary("EXP2", True), _unary("LOG2", True), _unary("SQRT", True)
add, mul, maximum = _binary("ADD"), _binary("MUL"), _binary("MAX")
mod, idiv, and_, or_, xor = (_binary(n, int_only=True) for n in ("MOD", "IDIV", "AND", "OR", "XOR"))
ne, lt = _binary("NE", boolean=True), _binary("LT", boolean=True)


def cast(a: Node, cls: int) -> Node:
    return a if a.cls == cls else Node("CAST", (a,), cls)


def where(cond: Node, a: Node, b: Node) -> Node:
    _same(a, b, "WHERE")
    return Node("WHERE", (cast(cond, BOOL) if cond.cls != BOOL else cond, a, b), a.cls)


class Program:
    """Postfix program + constant pool + operand list of one expression."""

    def __init__(self, root: Node):
        self.code: List[int] = []
        self.consts: List[int] = []
        self.operands: List[View] = []
        self.result_cls = root.cls
        self._emit(root)
        if len(self.code) > L.EXPR_MAX_CODE:
            raise ValueError(f"expression compiles to {len(self.code)} words (limit {L.EXPR_MAX_CODE}); split the item")

    def _const(self, v, cls) -> int:
        bits = struct.unpack("<I", struct.pack("<f", float(v)))[0] if cls == F32 else int(v) & 0xFFFFFFFF
        if bits not in self.consts:
            if len(self.consts) >= L.EXPR_MAX_CONSTS:
                raise ValueError("too many distinct constants in one item")
            self.consts.append(bits)
        return self.consts.index(bits)

    def _operand(self, view: View) -> int:
        for i, v in enumerate(self.operands):
            if v is view:
                return i
        if len(self.operands) >= L.EXPR_MAX_OPERANDS:
            raise ValueError("too many operands in one item")
        self.operands.append(view)
        return len(self.operands) - 1

    def _emit(self, n: Node):
        word = lambda op, arg, cls: OP[op] | (arg << 8) | (cls << 16)
        if n.op == "LOAD":
            self.code.append(word("LOAD", self._operand(n.value), n.cls))
        elif n.op == "CONST":
            self.code.append(word("CONST", self._const(n.value, n.cls), n.cls))
        elif n.op == "INDEX":
            self.code.append(word("INDEX", n.value, I32))
        else:
            for a in n.args:
                self._emit(a)
            if n.op == "CAST":
                self.code.append(word("CAST", n.args[0].cls, n.cls))
            elif n.op in ("NE", "LT", "NOT"):
                self.code.append(word(n.op, 0, n.args[0].cls))   # class field = class of the operands
            else:
                self.code.append(word(n.op, 0, n.cls))


def describe(prog: Program, out: View, shape: Sequence[int], n_reduce: int = 0, reduce_op: Optional[str] = None,
             accumulate: bool = False) -> L.ExprDesc:
    """Fills the C struct.  ``shape`` is the loop nest (outermost first); every view must give one
    stride per loop."""
    shape = tuple(int(s) for s in shape)
    if not 1 <= len(shape) <= L.EXPR_MAX_DIMS:
        raise ValueError(f"{len(shape)} loops (1..{L.EXPR_MAX_DIMS}); merge contiguous axes first")
    d = L.ExprDesc()
    d.ndim, d.n_reduce, d.reduce_op, d.accumulate = len(shape), int(n_reduce), RED[reduce_op], int(bool(accumulate))
    for i, s in enumerate(shape):
        d.shape[i] = s
    d.n_operands = len(prog.operands)
    for i, v in enumerate(prog.operands):
        if len(v.strides) != len(shape):
            raise ValueError(f"operand {i}: {len(v.strides)} strides for {len(shape)} loops")
        d.operand[i] = v.buf.ptr
        d.operand_dtype[i] = DT_OF[np.dtype(v.buf.dtype)][0]
        d.operand_offset[i] = v.offset
        for k, s in enumerate(v.strides):
            d.operand_stride[i][k] = s
    if len(out.strides) != len(shape):
        raise ValueError(f"output: {len(out.strides)} strides for {len(shape)} loops")
    d.out, d.out_dtype, d.out_offset = out.buf.ptr, DT_OF[np.dtype(out.buf.dtype)][0], out.offset
    for k, s in enumerate(out.strides):
        d.out_stride[k] = s
    d.n_code = len(prog.code)
    for i, w in enumerate(prog.code):
        d.code[i] = w
    for i, c in enumerate(prog.consts):
        d.consts[i] = c
    return d


def run(rt, root: Node, out: View, shape: Optional[Sequence[int]] = None, n_reduce: int = 0, reduce_op: Optional[str] = None,
        accumulate: bool = False) -> None:
    """Runs one item on the runtime's stream (asynchronous, like every kernel call)."""
    prog = root if isinstance(root, Program) else Program(root)
    d = describe(prog, out, shape if shape is not None else out.buf.shape, n_reduce, reduce_op, accumulate)
    L.check(rt.ctx, rt.lib.caten_b200_eval_expr(rt.ctx, C.byref(d)))
