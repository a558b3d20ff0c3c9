import numpy as np
import pytest

from caten_b200 import synthetic as S


def test_generators_are_deterministic():
    p = S.GPT2Params(n_layers=1, n_heads=1, dim=64, vocab_size=97)
    a = S.synth_state_dict(p, "q4_0", seed=4, max_seq_len=16)
    b = S.synth_state_dict(p, "q4_0", seed=4, max_seq_len=16)
    for k in a:
        x, y = (a[k].data, b[k].data) if isinstance(a[k], S.Packed) else (a[k], b[k])
        np.testing.assert_array_equal(x, y)
    assert not np.array_equal(S.synth_prompts(2, 8, 97, 0), S.synth_prompts(2, 8, 97, 1))


@pytest.mark.parametrize("wtype,bb", [("q4_0", 18), ("q8_0", 34)])
def test_packed_shapes_and_value_ranges(wtype, bb):
    rng = np.random.Generator(np.random.PCG64(0))
    p = S._rand_packed(rng, 5, 128, wtype)
    assert p.data.size == 5 * 4 * bb
    blocks = p.data.reshape(-1, bb)
    scales = blocks[:, :2].copy().view(np.float16).astype(np.float32)
    assert (scales >= 0).all() and scales.max() < 0.02
    if wtype == "q8_0":
        assert blocks[:, 2:].view(np.int8).min() >= -127


def test_pack_q4_0_nibble_order_matches_gguf():
    gguf = pytest.importorskip("gguf")
    from gguf.quants import dequantize
    codes = np.arange(32, dtype=np.uint8).reshape(1, 32) % 16
    raw = S.pack_q4_0(codes, np.array([1.0], np.float16))
    got = dequantize(raw.reshape(1, 18), gguf.GGMLQuantizationType.Q4_0).reshape(-1)
    np.testing.assert_array_equal(got, codes.reshape(-1).astype(np.float32) - 8)


def test_benchmark_config_shapes():
    xl = S.GPT2_SIZES["gpt2-xl"]
    assert (xl.n_layers, xl.n_heads, xl.dim) == (48, 25, 1600) and xl.dim // xl.n_heads == 64
    a, b = S.synth_relu_gemm(M=8, K=64, N=16)
    assert a.shape == (8, 64) and b.shape == (64, 16)
