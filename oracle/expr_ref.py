"""TEST INFRASTRUCTURE ONLY (imported by tests/): numpy restatement of one generic schedule item.

Interprets the same postfix program as ``caten_b200_eval_expr`` the way the C function the
reference renders for a Schedule-Item computes it (source/codegen/renderer.lisp:331-410,
source/byoc/clang.lisp:163-205): fp32 arithmetic element by element, SIN / EXP2 / LOG2 / SQRT in
double then rounded to float (C's double libm applied to a float), integer ops with C truncation,
and a reduction that walks the reduced loops in loop order (so a float sum has the reference's
order of additions).  Parity unpinned by reference vectors: the reference holds no golden values
for single schedule items; its tests compare against numpy/torch functions, as tests/ do here.
"""
import struct

import numpy as np

F32, I32, BOOL = 0, 1, 2
DT = {0: np.float32, 1: np.int32, 2: np.int64, 3: np.uint8}


def _cast(v, frm, to):
    if frm == to:
        return v
    if to == F32:
        return v.astype(np.float32)
    if frm == F32:
        return (v != 0).astype(np.int32) if to == BOOL else np.trunc(v).astype(np.int64).astype(np.int32)
    return (v != 0).astype(np.int32) if to == BOOL else v


def _gather(arr, offset, strides, idx):
    at = offset
    for s, i in zip(strides, idx):
        at = at + s * i
    return arr.reshape(-1)[at]


def run_program(code, consts, operands, idx):
    """operands: list of (flat array, dtype id, offset, strides); idx: list of broadcastable index grids."""
    st = []
    with np.errstate(all="ignore"):
        for w in code:
            op, arg, cls = w & 255, (w >> 8) & 255, (w >> 16) & 255
            if op == 1:
                arr, dt, off, strides = operands[arg]
                v = _gather(arr, off, strides, idx)
                v = v.astype(np.float32) if dt == 0 else (v != 0).astype(np.int32) if dt == 3 else v.astype(np.int32)
                st.append(v)
            elif op == 2:
                bits = consts[arg]
                st.append(np.float32(struct.unpack("<f", struct.pack("<I", bits))[0]) if cls == F32
                          else np.int32(struct.unpack("<i", struct.pack("<I", bits))[0]))
            elif op == 3:
                st.append(np.asarray(idx[arg]).astype(np.int32))
            elif op < 30:
                a = st.pop()
                f = cls == F32
                if op == 10: r = -a
                elif op == 11: r = (np.float32(1.0) / a).astype(np.float32) if f else np.where(a == 0, 0, np.trunc(1.0 / np.where(a == 0, 1, a))).astype(np.int32)
                elif op == 12: r = np.sin(a.astype(np.float64)).astype(np.float32)
                elif op == 13: r = np.exp2(a.astype(np.float64)).astype(np.float32)
                elif op == 14: r = np.log2(a.astype(np.float64)).astype(np.float32)
                elif op == 15: r = np.sqrt(a.astype(np.float64)).astype(np.float32)
                elif op == 16: r = (a == 0).astype(np.int32)
                else: r = _cast(a, arg, cls)
                st.append(r)
            elif op < 50:
                b, a = st.pop(), st.pop()
                f = cls == F32
                if op == 30: r = (a + b).astype(np.float32) if f else (a.astype(np.int64) + b).astype(np.int32)
                elif op == 31: r = (a * b).astype(np.float32) if f else (a.astype(np.int64) * b).astype(np.int32)
                elif op == 32: r = np.where(b == 0, 0, np.fmod(a, np.where(b == 0, 1, b))).astype(np.int32)
                elif op == 33: r = np.where(b == 0, 0, np.trunc(a / np.where(b == 0, 1, b).astype(np.float64))).astype(np.int32)
                elif op == 34: r = a & b
                elif op == 35: r = a | b
                elif op == 36: r = a ^ b
                elif op == 37: r = np.where(a > b, a, b)
                elif op == 38: r = (a != b).astype(np.int32)
                else: r = (a < b).astype(np.int32)
                st.append(r)
            else:
                b, a, c = st.pop(), st.pop(), st.pop()
                st.append(np.where(c != 0, a, b))
    assert len(st) == 1
    return st[0]


def eval_item(code, consts, operands, out, out_dtype, out_offset, out_strides, shape, n_reduce=0, reduce_op=0,
              accumulate=False, result_cls=F32):
    """Runs the item on host arrays; `out` (flat array) is updated in place and returned."""
    shape = tuple(shape)
    nd_out = len(shape) - n_reduce
    oshape, rshape = shape[:nd_out], shape[nd_out:]
    grids = np.meshgrid(*[np.arange(n) for n in oshape], indexing="ij") if nd_out else []
    oidx = [g.reshape(-1) for g in grids]
    n_out = int(np.prod(oshape, dtype=np.int64)) if nd_out else 1
    out_at = np.full(n_out, out_offset, dtype=np.int64)
    for s, i in zip(out_strides[:nd_out], oidx):
        out_at = out_at + s * i
    flat = out.reshape(-1)
    f = result_cls == F32

    def to_out(v):
        v = np.broadcast_to(v, (n_out,))
        if out_dtype == 0:
            return v.astype(np.float32)
        if out_dtype == 3:
            return (v != 0).astype(np.uint8)
        return (np.trunc(v) if f else v).astype(DT[out_dtype])

    if n_reduce == 0:
        flat[out_at] = to_out(run_program(code, consts, operands, oidx))
        return out
    n_red = int(np.prod(rshape, dtype=np.int64))
    acc, have = None, False
    if accumulate:
        old = flat[out_at]
        acc = old.astype(np.float32) if f else (np.trunc(old) if out_dtype == 0 else old).astype(np.int32)
        have = True
    elif reduce_op == 1:
        acc = np.zeros(n_out, np.float32 if f else np.int32)
    for r in range(n_red):
        ridx = np.unravel_index(r, rshape)
        idx = oidx + [np.int64(i) for i in ridx]
        v = np.broadcast_to(run_program(code, consts, operands, idx), (n_out,))
        if reduce_op == 1:
            acc = (acc + v).astype(np.float32) if f else (acc.astype(np.int64) + v).astype(np.int32)
        else:
            acc = np.where(acc > v, acc, v) if (have or r > 0) else v.copy()
    flat[out_at] = to_out(acc)
    return out
