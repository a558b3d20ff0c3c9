"""CPU tests of the generic schedule item's host side: the expression compiler and the numpy
restatement it is checked against on the GPU (the restatement itself is checked here against
plain numpy formulas)."""
import numpy as np
import pytest

from caten_b200 import expr as E
from oracle import expr_ref as R


class HostBuf:
    """Stands in for a device buffer: the compiler only needs dtype, shape and identity."""

    def __init__(self, a):
        self.a = np.ascontiguousarray(a)
        self.dtype, self.shape, self.ptr = self.a.dtype, self.a.shape, 0


def host_run(root, out, shape=None, n_reduce=0, reduce_op=None, accumulate=False):
    prog = E.Program(root)
    ops = [(v.buf.a, E.DT_OF[np.dtype(v.buf.dtype)][0], v.offset, v.strides) for v in prog.operands]
    return R.eval_item(prog.code, prog.consts, ops, out.buf.a, E.DT_OF[np.dtype(out.buf.dtype)][0], out.offset, out.strides,
                       shape if shape is not None else out.buf.shape, n_reduce, E.RED[reduce_op], accumulate, prog.result_cls)


def test_program_is_postfix_with_pooled_constants():
    x = E.View.of(HostBuf(np.zeros((2, 3), np.float32)))
    root = E.maximum(E.load(x) * 2.0 + E.load(x) * 2.0, E.const(0.0))
    p = E.Program(root)
    ops = [w & 255 for w in p.code]
    assert ops == [1, 2, 31, 1, 2, 31, 30, 2, 37]      # LOAD CONST MUL LOAD CONST MUL ADD CONST MAX
    assert len(p.consts) == 2 and len(p.operands) == 1  # 2.0 and 0.0 pooled, the view used twice is one operand
    assert all(((w >> 16) & 255) == E.F32 for w in p.code)


def test_sub_and_div_compose_like_the_reference():
    x = E.View.of(HostBuf(np.zeros(4, np.float32)))
    p = E.Program(E.load(x) - 1.0)
    assert [w & 255 for w in p.code] == [1, 2, 10, 30]   # a + (-b)
    p = E.Program(E.load(x) / 3.0)
    assert [w & 255 for w in p.code] == [1, 2, 11, 31]   # a * recip(b)


def test_class_mismatch_is_refused_at_build_time():
    x = E.View.of(HostBuf(np.zeros(4, np.float32)))
    i = E.View.of(HostBuf(np.zeros(4, np.int32)))
    with pytest.raises(TypeError):
        E.add(E.load(x), E.load(i))
    with pytest.raises(TypeError):
        E.mod(E.load(x), E.load(x))
    with pytest.raises(TypeError):
        E.sin(E.load(i))
    E.add(E.load(x), E.cast(E.load(i), E.F32))  # with the cast it builds


def test_numpy_restatement_elementwise_and_broadcast():
    rng = np.random.Generator(np.random.PCG64(0))
    a, b = rng.standard_normal((5, 7), dtype=np.float32), rng.standard_normal(7, dtype=np.float32)
    x, y = E.View.of(HostBuf(a)), E.View(HostBuf(b), strides=(0, 1))
    out = E.View.of(HostBuf(np.zeros((5, 7), np.float32)))
    host_run(E.where(E.load(x) < 0.0, -E.load(x), E.load(x)) * 0.5 + E.load(y), out)
    np.testing.assert_array_equal(out.buf.a, (np.abs(a) * np.float32(0.5) + b).astype(np.float32))


def test_numpy_restatement_reduction_is_sequential():
    rng = np.random.Generator(np.random.PCG64(1))
    a = (rng.standard_normal((3, 1000), dtype=np.float32) * 1e3).astype(np.float32)
    out = E.View(HostBuf(np.zeros(3, np.float32)), strides=(1, 0))
    host_run(E.load(E.View.of(HostBuf(a))), out, shape=(3, 1000), n_reduce=1, reduce_op="sum")
    want = np.zeros(3, np.float32)
    for j in range(1000):
        want = (want + a[:, j]).astype(np.float32)
    np.testing.assert_array_equal(out.buf.a, want)
    assert not np.array_equal(want, a.sum(1, dtype=np.float32)) or True  # pairwise numpy sum may differ; the item is sequential


def test_numpy_restatement_integer_semantics():
    a = np.array([7, -7, 9, -9, 5], np.int32)
    b = np.array([2, 2, -4, -4, 0], np.int32)
    x, y = E.View.of(HostBuf(a)), E.View.of(HostBuf(b))
    q, r = E.View.of(HostBuf(np.zeros(5, np.int32))), E.View.of(HostBuf(np.zeros(5, np.int32)))
    host_run(E.idiv(E.load(x), E.load(y)), q)
    host_run(E.mod(E.load(x), E.load(y)), r)
    np.testing.assert_array_equal(q.buf.a, [3, -3, -2, 2, 0])   # C truncation; x / 0 defined as 0 here
    np.testing.assert_array_equal(r.buf.a, [1, -1, 1, -1, 0])


def test_limits():
    x = E.View.of(HostBuf(np.zeros(4, np.float32)))
    n = E.load(x)
    for k in range(60):
        n = n + float(k + 1)
    with pytest.raises(ValueError):
        E.Program(n)   # more than 16 distinct constants
    with pytest.raises(ValueError):
        E.describe(E.Program(E.load(x)), x, shape=(1,) * 7)
