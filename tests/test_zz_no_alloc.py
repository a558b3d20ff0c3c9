"""The allocation-free Linear entry point (`caten_b200_linear_noalloc`).

Some hosts of this library cannot let it call cudaMalloc behind their back: a runtime that plans
every device buffer itself, a token loop that cannot take the device-wide synchronisation an
allocation may cause, a process whose KV cache already fills HBM.  For them the tensor-core Linear
keeps its working memory in a fixed buffer inside the library.  This file checks, through the C
ABI, that the variant returns what `caten_b200_linear` returns — on two calls in a row, because
the buffer is shared and keeps the previous call's contents — and that it refuses shapes that do
not fit.  It is collected last on purpose.
"""
import numpy as np
import pytest

from caten_b200 import _lib as L
from caten_b200 import synthetic as S
from caten_b200._lib import B200Error

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("prec", ["bf16x3", "bf16"])
def test_noalloc_matches_linear_on_consecutive_calls(rt, oracle, prec):
    rng = np.random.Generator(np.random.PCG64(101))
    packed = S._rand_packed(rng, 1600, 1600, "q4_0", 0.05)
    w = rt.upload_weight(packed)   # few output tiles: split-K partials in use
    wf = oracle.dequant(packed.ggml_type, packed.data, 1600 * 1600).reshape(1600, 1600)
    bias_h = rng.standard_normal(1600, dtype=np.float32) * 0.1
    bias = rt.transfer_from_array(bias_h)
    p = L.PRECISIONS[prec]
    # second call: fewer rows and another activation, so stale bytes of the first call stay in the buffer
    for M, act in ((64, L.ACT_GELU), (24, L.ACT_NONE)):
        x_h = rng.standard_normal((M, 1600), dtype=np.float32)
        res_h = rng.standard_normal((M, 1600), dtype=np.float32) * 0.1
        x, res = rt.transfer_from_array(x_h), rt.transfer_from_array(res_h)
        want = rt.linear(w, x, bias, res, act, p).numpy()
        out = rt.open_buffer((M, 1600))
        got = rt.linear_noalloc(w, x, out, bias, res, act, p).numpy()
        rt.sync()
        # same kernels, same tile and split-K plan, only the working memory differs: the same bits
        np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
        # and the value itself against the CPU oracle (the reference's Linear, source/nn/linear.lisp:12-17)
        ref = oracle.linear(x_h, wf, bias_h, res_h, act)
        scale = max(1.0, float(np.abs(ref).max()))
        assert np.abs(got - ref).max() <= (2e-2 if prec == "bf16" else 1e-4) * scale
    w.close()


def test_noalloc_small_row_counts_use_the_gemv(rt):
    rng = np.random.Generator(np.random.PCG64(102))
    w = rt.upload_weight(S._rand_packed(rng, 300, 256, "q8_0", 0.05))
    x = rt.transfer_from_array(rng.standard_normal((3, 256), dtype=np.float32))
    want = rt.linear(w, x).numpy()
    got = rt.linear_noalloc(w, x, rt.open_buffer((3, 300))).numpy()
    np.testing.assert_array_equal(got, want)
    w.close()


def test_noalloc_rejects_working_sets_beyond_the_fixed_buffer(rt):
    rng = np.random.Generator(np.random.PCG64(103))
    w = rt.upload_weight(S._rand_packed(rng, 128, 6400, "q4_0"))
    x = rt.open_buffer((2048, 6400))          # 2048 x 6400 x 2 B x 2 = 50 MiB of bf16 copies > 32 MiB
    out = rt.open_buffer((2048, 128))
    with pytest.raises(B200Error) as e:
        rt.linear_noalloc(w, x, out, precision=L.PREC_BF16X3)
    assert e.value.code == L.EUNSUPPORTED and "built-in buffer" in str(e.value)
    rt.linear(w, x, precision=L.PREC_BF16X3)  # the allocating entry point still serves it
    rt.sync()
    w.close()
