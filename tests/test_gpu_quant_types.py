"""GPU tests of the GGUF block formats that are expanded to fp32 at upload (Q4_1, Q5_0, Q5_1, Q2_K,
Q3_K, Q4_K, Q5_K, Q6_K): the device expansion must give, bit for bit, what the Python `gguf` package's
dequantiser gives (the library the reference's own GGUF tests use as their oracle,
source/test-suite/external/test-gguf.lisp:53-75), and a Linear over such a weight must match the
product with those values."""
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
