"""GPU tests of the generic schedule item (`caten_b200_eval_expr`): the interpreting kernel against
the numpy restatement of the rendered C, on the op patterns of the reference's
source/test-suite/test-ops.lisp and test-activations.lisp (element-wise, ax+b, broadcast, where,
cast, reductions), bit for bit where the arithmetic is fp32 / integer."""
import numpy as np
import pytest

from caten_b200 import expr as E
from caten_b200._lib import B200Error, EINVAL
from oracle import expr_ref as R

pytestmark = pytest.mark.gpu


class Pair:
    """A host array and its device copy under one view description."""

    def __init__(self, rt, a, strides=None, offset=0):
        self.host = np.ascontiguousarray(a)
        self.dev = rt.transfer_from_array(self.host)
        self.view = E.View(self.dev, strides, offset)

    def close(self):
        self.dev.close()


def check(rt, root, out: Pair, shape=None, n_reduce=0, reduce_op=None, accumulate=False, pairs=(), ulp=0):
    prog = E.Program(root)
    by_view = {id(p.view): p for p in pairs}
    ops = [(by_view[id(v)].host, E.DT_OF[np.dtype(v.buf.dtype)][0], v.offset, v.strides) for v in prog.operands]
    want = out.host.copy()
    R.eval_item(prog.code, prog.consts, ops, want, E.DT_OF[np.dtype(out.host.dtype)][0], out.view.offset, out.view.strides,
                shape if shape is not None else out.host.shape, n_reduce, E.RED[reduce_op], accumulate, prog.result_cls)
    E.run(rt, prog, out.view, shape, n_reduce, reduce_op, accumulate)
    got = out.dev.numpy()
    if ulp == 0:
        if got.dtype == np.float32:
            same = (got.view(np.uint32) == want.view(np.uint32)) | (np.isnan(got) & np.isnan(want))
            assert same.all(), f"{(~same).sum()} of {same.size} elements differ, first at {np.argwhere(~same)[0]}"
        else:
            np.testing.assert_array_equal(got, want)
    else:
        d = np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))
        d = np.where(np.isnan(got) & np.isnan(want), 0, d)
        assert d.max() <= ulp and (d == 0).mean() > 0.995
    return got, want


def test_elementwise_relu_axpb(rt):
    rng = np.random.Generator(np.random.PCG64(0))
    x, y = Pair(rt, rng.standard_normal((37, 129), dtype=np.float32)), Pair(rt, rng.standard_normal((37, 129), dtype=np.float32))
    out = Pair(rt, np.zeros((37, 129), np.float32))
    got, _ = check(rt, E.maximum(E.load(x.view) * 2.0 + E.load(y.view), E.const(0.0)), out, pairs=(x, y))
    np.testing.assert_array_equal(got, np.maximum(x.host * np.float32(2) + y.host, 0).astype(np.float32))


def test_broadcast_transpose_and_slices(rt):
    rng = np.random.Generator(np.random.PCG64(1))
    a = Pair(rt, rng.standard_normal((6, 10), dtype=np.float32), strides=(10, 0, 1))         # a[i, k] broadcast over j
    b = Pair(rt, rng.standard_normal((10, 8), dtype=np.float32), strides=(0, 1, 8))          # b[k, j] read transposed as [j, k]
    c = Pair(rt, rng.standard_normal((6, 8, 12), dtype=np.float32), strides=(96, 12, 1), offset=2)  # c[:, :, 2:12]
    out = Pair(rt, np.zeros((6, 8, 10), np.float32))
    got, _ = check(rt, E.load(a.view) * E.load(b.view) + E.load(c.view), out, pairs=(a, b, c))
    want = a.host[:, None, :] * b.host.T[None, :, :] + c.host[:, :, 2:12]
    np.testing.assert_array_equal(got, want.astype(np.float32))


def test_where_compare_not_cast_index(rt):
    rng = np.random.Generator(np.random.PCG64(2))
    x = Pair(rt, (rng.standard_normal((9, 33), dtype=np.float32) * 10).astype(np.float32))
    out = Pair(rt, np.zeros((9, 33), np.float32))
    lx = E.load(x.view)
    # |x| where x != trunc(x) else the flat index, as a float
    flat = E.cast(E.add(E.mul(E.index(0), E.const(33)), E.index(1)), E.F32)
    root = E.where(E.ne(E.cast(E.cast(lx, E.I32), E.F32), lx), E.where(lx < 0.0, -lx, lx), flat)
    got, _ = check(rt, root, out, pairs=(x,))
    np.testing.assert_array_equal(got, np.abs(x.host))   # no element is an exact integer
    mask = Pair(rt, np.zeros((9, 33), np.uint8))
    got, _ = check(rt, E.not_(lx < 0.0), mask, pairs=(x,))
    np.testing.assert_array_equal(got, (x.host >= 0).astype(np.uint8))
    idx = Pair(rt, np.zeros((9, 33), np.int64))
    got, _ = check(rt, E.add(E.mul(E.index(0), E.const(33)), E.index(1)), idx, pairs=())
    np.testing.assert_array_equal(got, np.arange(9 * 33).reshape(9, 33))


def test_integer_ops(rt):
    rng = np.random.Generator(np.random.PCG64(3))
    a = Pair(rt, rng.integers(-1000, 1000, (17, 40)).astype(np.int32))
    b = Pair(rt, rng.integers(-9, 9, (17, 40)).astype(np.int32))
    out = Pair(rt, np.zeros((17, 40), np.int32))
    la, lb = E.load(a.view), E.load(b.view)
    check(rt, E.add(E.mul(E.idiv(la, lb), lb), E.mod(la, lb)), out, pairs=(a, b))       # == a wherever b != 0
    nz = b.host != 0
    np.testing.assert_array_equal(out.dev.numpy()[nz], a.host[nz])
    check(rt, E.xor(E.and_(la, E.const(255)), E.or_(lb, E.const(3))), out, pairs=(a, b))
    check(rt, E.maximum(E.neg(la), lb), out, pairs=(a, b))


def test_transcendentals_round_once_from_double(rt):
    rng = np.random.Generator(np.random.PCG64(4))
    x = Pair(rt, (rng.standard_normal(20000, dtype=np.float32) * 4).astype(np.float32))
    out = Pair(rt, np.zeros(20000, np.float32))
    lx = E.load(x.view)
    for root in (E.sin(lx), E.exp2(lx), E.log2(lx * lx + 1e-3), E.sqrt(lx * lx), E.recip(lx)):
        check(rt, root, out, pairs=(x,), ulp=0 if root.op in ("SQRT", "RECIP") else 1)


def test_gelu_composed_like_the_reference_matches_the_c_oracle(rt, oracle):
    # source/nn/activations.lisp:202-204: x * 0.5 * (1 + tanh(sqrt(2/pi) * (x + 0.044715 x^3))), tanh through sigmoid/exp2
    rng = np.random.Generator(np.random.PCG64(5))
    x = Pair(rt, (rng.standard_normal(4096, dtype=np.float32) * 3).astype(np.float32))
    out = Pair(rt, np.zeros(4096, np.float32))
    lx = E.load(x.view)
    z = (lx + lx * lx * lx * 0.044715) * 0.7978845608028654
    sig = E.recip(E.exp2(z * 2.0 * (-1.0 / 0.6931472)) + 1.0)
    root = lx * 0.5 * (sig * 2.0 + (-1.0) + 1.0)
    got, _ = check(rt, root, out, pairs=(x,), ulp=1)
    np.testing.assert_allclose(got, oracle.gelu(x.host), atol=1e-6, rtol=0)   # tolerance of test-activations.lisp:176-184


def test_reductions_in_loop_order(rt):
    rng = np.random.Generator(np.random.PCG64(6))
    a = Pair(rt, (rng.standard_normal((13, 7, 300), dtype=np.float32) * 100).astype(np.float32))
    # sum over the last axis
    s1 = Pair(rt, np.zeros((13, 7), np.float32), strides=(7, 1, 0))
    check(rt, E.load(a.view), s1, shape=(13, 7, 300), n_reduce=1, reduce_op="sum", pairs=(a,))
    # max over the last two axes
    m2 = Pair(rt, np.zeros(13, np.float32), strides=(1, 0, 0))
    got, _ = check(rt, E.load(a.view), m2, shape=(13, 7, 300), n_reduce=2, reduce_op="max", pairs=(a,))
    np.testing.assert_array_equal(got, a.host.max((1, 2)))
    # everything into one scalar, on top of the old value (the :reduction store)
    tot = Pair(rt, np.array([5.0], np.float32), strides=(0, 0, 0))
    check(rt, E.load(a.view) * E.load(a.view), tot, shape=(13, 7, 300), n_reduce=3, reduce_op="sum", accumulate=True, pairs=(a,))
    # integer count of negatives per row
    cnt = Pair(rt, np.zeros((13, 7), np.int32), strides=(7, 1, 0))
    got, _ = check(rt, E.cast(E.load(a.view) < 0.0, E.I32), cnt, shape=(13, 7, 300), n_reduce=1, reduce_op="sum", pairs=(a,))
    np.testing.assert_array_equal(got, (a.host < 0).sum(2))


def test_softmax_from_four_items(rt):
    # max, exp2((x - m) / ln 2), sum, divide: the reference's softmax (source/nn/activations.lisp, atol 1e-5 in test-llm.lisp:28-80)
    rng = np.random.Generator(np.random.PCG64(7))
    x = Pair(rt, rng.standard_normal((64, 257), dtype=np.float32))
    m = Pair(rt, np.zeros(64, np.float32), strides=(1, 0))
    e = Pair(rt, np.zeros((64, 257), np.float32))
    s = Pair(rt, np.zeros(64, np.float32), strides=(1, 0))
    y = Pair(rt, np.zeros((64, 257), np.float32))
    check(rt, E.load(x.view), m, shape=(64, 257), n_reduce=1, reduce_op="max", pairs=(x,))
    m.host[:] = m.dev.numpy()
    check(rt, E.exp2((E.load(x.view) - E.load(m.view)) * (1.0 / 0.6931472)), e, pairs=(x, m), ulp=1)
    e.host[:] = e.dev.numpy()
    check(rt, E.load(e.view), s, shape=(64, 257), n_reduce=1, reduce_op="sum", pairs=(e,))
    s.host[:] = s.dev.numpy()
    got, _ = check(rt, E.load(e.view) / E.load(s.view), y, pairs=(e, s))
    x64 = x.host.astype(np.float64)
    want = np.exp(x64 - x64.max(1, keepdims=True))
    want /= want.sum(1, keepdims=True)
    np.testing.assert_allclose(got, want, atol=1e-5, rtol=0)


def test_random_expression_trees(rt):
    rng = np.random.Generator(np.random.PCG64(8))
    shape = (11, 5, 23)
    srcs = [Pair(rt, (rng.standard_normal(shape, dtype=np.float32) * 2).astype(np.float32)) for _ in range(2)]
    srcs.append(Pair(rt, rng.standard_normal((11, 23), dtype=np.float32), strides=(23, 0, 1)))
    srcs.append(Pair(rt, rng.standard_normal(5, dtype=np.float32), strides=(0, 1, 0)))
    out = Pair(rt, np.zeros(shape, np.float32))

    def tree(depth):
        if depth == 0 or rng.random() < 0.2:
            return E.load(srcs[int(rng.integers(len(srcs)))].view) if rng.random() < 0.8 else E.const(float(np.float32(rng.standard_normal())))
        k = int(rng.integers(7))
        a, b = tree(depth - 1), tree(depth - 1)
        if k == 0: return a + b
        if k == 1: return a * b
        if k == 2: return a - b
        if k == 3: return E.maximum(a, b)
        if k == 4: return E.where(a < b, a, b)
        if k == 5: return E.where(E.ne(a, b), -a, E.recip(b))
        return a / b
    built = 0
    while built < 25:
        try:
            root = tree(4)
            E.Program(root)
        except ValueError:
            continue   # more operands / constants than one item holds
        if root.op in ("CONST", "LOAD"):
            continue
        check(rt, root, out, pairs=srcs)
        built += 1


def test_empty_and_large(rt):
    x = Pair(rt, np.zeros((0, 8), np.float32))
    out = Pair(rt, np.zeros((0, 8), np.float32))
    E.run(rt, E.load(x.view) + 1.0, out.view)       # nothing to do, no launch error
    rng = np.random.Generator(np.random.PCG64(9))
    big = Pair(rt, rng.standard_normal(3_000_001, dtype=np.float32))
    res = Pair(rt, np.zeros(3_000_001, np.float32))
    check(rt, E.load(big.view) * E.load(big.view) + 1.0, res, pairs=(big,))


def test_malformed_programs_are_refused(rt):
    from caten_b200 import _lib as L
    x = Pair(rt, np.zeros(8, np.float32))
    out = Pair(rt, np.zeros(8, np.float32))
    d = E.describe(E.Program(E.load(x.view) + 1.0), out.view, (8,))

    def expect_einval(mutate):
        import ctypes as C
        dd = L.ExprDesc.from_buffer_copy(bytes(d))
        mutate(dd)
        rc = rt.lib.caten_b200_eval_expr(rt.ctx, C.byref(dd))
        assert rc == EINVAL, rt.lib.caten_b200_last_error(rt.ctx)

    expect_einval(lambda dd: dd.code.__setitem__(0, 1 | (5 << 8)))                 # loads operand 5 of 1
    expect_einval(lambda dd: dd.code.__setitem__(2, 30 | (E.I32 << 16)))           # integer add on floats
    expect_einval(lambda dd: setattr(dd, "n_code", 2))                             # leaves two values
    expect_einval(lambda dd: dd.code.__setitem__(0, 30))                           # add on an empty stack
    expect_einval(lambda dd: setattr(dd, "ndim", 9))
    expect_einval(lambda dd: setattr(dd, "reduce_op", 1))                          # reduce op without reduced loops
    expect_einval(lambda dd: dd.code.__setitem__(2, 99))                           # unknown opcode
    with pytest.raises(B200Error):
        E.run(rt, E.load(x.view), out.view, shape=(8,), n_reduce=1, reduce_op=None)
