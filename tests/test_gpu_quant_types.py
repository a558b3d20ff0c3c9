"""GPU tests of the GGUF block formats beyond Q4_0 / Q8_0: Q4_1, Q5_0 and Q5_1 stay packed in device
memory and are unpacked inside the GEMV / GEMM kernels; Q2_K, Q3_K, Q4_K, Q5_K and Q6_K are expanded to
fp32 at upload.  Either way the weight's values must be, bit for bit, what the Python `gguf` package's
dequantiser gives (the library the reference's own GGUF tests use as their oracle,
source/test-suite/external/test-gguf.lisp:53-75), and a Linear over such a weight must match the
product with those values on every kernel path."""
import numpy as np
import pytest

from caten_b200 import _lib as L
from caten_b200 import synthetic as S
from caten_b200.gguf import gguf_to_state_dict, load_gguf

pytestmark = pytest.mark.gpu
gguf = pytest.importorskip("gguf")
from gguf import GGMLQuantizationType as GT  # noqa: E402
from gguf.quants import dequantize  # noqa: E402

# type -> (elements per block, bytes per block, byte offsets of the fp16 fields)
FORMATS = {
    L.Q4_1: (32, 20, (0, 2)), L.Q5_0: (32, 22, (0,)), L.Q5_1: (32, 24, (0, 2)),
    L.Q2_K: (256, 84, (80, 82)), L.Q3_K: (256, 110, (108,)),
    L.Q4_K: (256, 144, (0, 2)), L.Q5_K: (256, 176, (0, 2)), L.Q6_K: (256, 210, (208,)),
}


def random_blocks(rng, t, rows, cols):
    per, nbytes, halfs = FORMATS[t]
    nb = rows * cols // per
    raw = rng.integers(0, 256, (nb, nbytes), dtype=np.uint8)
    for off in halfs:  # finite, weight-sized fp16 scales / minima (some negative)
        vals = (rng.standard_normal(nb) * 0.02).astype("<f2")
        raw[:, off:off + 2] = vals.view(np.uint8).reshape(nb, 2)
    return raw.reshape(-1)


@pytest.mark.parametrize("t", sorted(FORMATS))
def test_expansion_matches_gguf_package_bit_for_bit(rt, t):
    rng = np.random.Generator(np.random.PCG64(t))
    rows, cols = 37, 512
    raw = random_blocks(rng, t, rows, cols)
    per, nbytes, _ = FORMATS[t]
    want = dequantize(raw.reshape(rows, cols // per * nbytes), GT(t)).astype(np.float32)
    w = rt.upload_weight(S.Packed(t, rows, cols, raw))
    got = w.dequantize()
    np.testing.assert_array_equal(got.view(np.uint32), want.reshape(rows, cols).view(np.uint32))
    assert w.packed_nbytes == raw.size
    # the 32-weight formats keep the file's bytes on the device, the K formats hold fp32
    assert w.device_nbytes == (raw.size if per == 32 else rows * cols * 4)
    # one sequence (fp32 GEMV) and a small batch (tensor cores, split bf16)
    x1 = rng.standard_normal((1, cols), dtype=np.float32)
    y1 = rt.linear(w, rt.transfer_from_array(x1)).numpy()
    ref1 = x1.astype(np.float64) @ want.reshape(rows, cols).T.astype(np.float64)
    np.testing.assert_allclose(y1, ref1, atol=2e-6 * np.abs(ref1).max() + 1e-5, rtol=0)   # fp32 accumulation over 512 terms
    x8 = rng.standard_normal((8, cols), dtype=np.float32)
    y8 = rt.linear(w, rt.transfer_from_array(x8), precision=L.PREC_BF16X3).numpy()
    ref8 = x8.astype(np.float64) @ want.reshape(rows, cols).T.astype(np.float64)
    np.testing.assert_allclose(y8, ref8, atol=5e-5 * np.abs(ref8).max() + 1e-5, rtol=0)   # split bf16: about 2^-16 of the operands' scale
    w.close()


PACKED = {"q4_1": L.Q4_1, "q5_0": L.Q5_0, "q5_1": L.Q5_1}


@pytest.mark.parametrize("name", sorted(PACKED))
def test_packed_nibble_formats_golden_and_edge_scales(rt, golden, name):
    """Committed `gguf`-package vectors, including scales / minima from every fp16 class."""
    g = golden["gguf_dequant_nibble"]
    for kind in ("rand", "edge"):
        want = g[f"{kind}_{name}"]
        w = rt.upload_weight(S.Packed(PACKED[name], want.shape[0], want.shape[1], g[f"{kind}_{name}_raw"]))
        np.testing.assert_array_equal(w.dequantize().view(np.uint32), want.view(np.uint32))
        w.close()


@pytest.mark.parametrize("name", sorted(PACKED))
@pytest.mark.parametrize("rows,cols", [(37, 512), (1600, 1600), (130, 6400)])
def test_packed_nibble_formats_on_every_linear_path(rt, oracle, name, rows, cols):
    """GEMV (1 and 3 rows), the exact fp32 GEMM, and the tensor-core GEMM in both precisions with row counts
    that give one narrow tile, a ragged tile and several tiles; weight rows not a multiple of the 128-row tile."""
    rng = np.random.Generator(np.random.PCG64(rows + cols))
    p = S._rand_packed(rng, rows, cols, name, 0.05)
    wf = oracle.dequant(p.ggml_type, p.data, rows * cols).reshape(rows, cols)
    w = rt.upload_weight(p)
    assert w.device_nbytes == p.data.size
    np.testing.assert_array_equal(w.dequantize().view(np.uint32), wf.view(np.uint32))
    bias = rng.standard_normal(rows, dtype=np.float32)
    d_bias = rt.transfer_from_array(bias)
    w64 = wf.T.astype(np.float64)
    for M in (1, 3):
        x = rng.standard_normal((M, cols), dtype=np.float32)
        y = rt.linear(w, rt.transfer_from_array(x), d_bias).numpy()
        ref = x.astype(np.float64) @ w64 + bias
        np.testing.assert_allclose(y, ref, atol=3e-6 * np.abs(ref).max() + 1e-5, rtol=0)
    for M in (8, 70):
        x = rng.standard_normal((M, cols), dtype=np.float32)
        d_x = rt.transfer_from_array(x)
        ref = x.astype(np.float64) @ w64 + bias
        y32 = rt.linear(w, d_x, d_bias, precision=L.PREC_FP32).numpy()
        # the exact path: the oracle's own accumulation order over the same dequantised values
        np.testing.assert_array_equal(y32.view(np.uint32), oracle.linear(x, wf, bias).view(np.uint32))
        y3 = rt.linear(w, d_x, d_bias, precision=L.PREC_BF16X3).numpy()
        np.testing.assert_allclose(y3, ref, atol=5e-5 * np.abs(ref).max() + 1e-5, rtol=0)
        y1 = rt.linear(w, d_x, d_bias, precision=L.PREC_BF16).numpy()
        np.testing.assert_allclose(y1, ref, atol=2e-2 * np.abs(ref).max(), rtol=0)
    if cols <= 1600:
        x = rng.standard_normal((300, cols), dtype=np.float32)
        ref = x.astype(np.float64) @ w64 + bias
        y3 = rt.linear(w, rt.transfer_from_array(x), d_bias, precision=L.PREC_BF16X3).numpy()
        np.testing.assert_allclose(y3, ref, atol=5e-5 * np.abs(ref).max() + 1e-5, rtol=0)
    w.close()


def test_block_size_must_divide_the_row(rt):
    raw = np.zeros(144, np.uint8)
    with pytest.raises(L.B200Error) as e:
        rt.upload_weight(S.Packed(L.Q4_K, 2, 128, raw))   # 128 columns: not a multiple of 256
    assert e.value.code == L.EUNSUPPORTED


def test_k_quant_tensor_from_a_gguf_file(rt, tmp_path):
    rng = np.random.Generator(np.random.PCG64(3))
    rows, cols = 8, 256
    raw = random_blocks(rng, L.Q6_K, rows, cols)
    path = tmp_path / "k.gguf"
    w = gguf.GGUFWriter(str(path), "gpt2")
    w.add_tensor("blk.0.ffn_up.weight", raw.reshape(rows, 210), raw_dtype=GT.Q6_K)
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()
    g = load_gguf(path)
    sd = gguf_to_state_dict(g)
    p = sd["h.0.mlp.c_fc.weight"]
    assert isinstance(p, S.Packed) and (p.ggml_type, p.rows, p.cols) == (L.Q6_K, rows, cols)
    h = g.upload("blk.0.ffn_up.weight", rt)
    want = dequantize(raw.reshape(rows, 210), GT.Q6_K).astype(np.float32)
    np.testing.assert_array_equal(h.dequantize().view(np.uint32), want.view(np.uint32))
    h.close(); g.close()
