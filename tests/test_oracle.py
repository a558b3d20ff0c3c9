"""CPU tests of the oracle: pinned against the golden fixtures (made by tests/golden/make_golden.py
from the Python `gguf` package and PyTorch, the reference test-suite's own oracles) with the
tolerances the reference's tests use."""
import numpy as np
import pytest

from caten_b200 import synthetic as S


def test_dequant_arange_fixture(oracle, golden):
    # source/test-suite/external/test-gguf.lisp:53-75 (atol 1e-5); here the match is exact
    g = golden["gguf_dequant"]
    for name, t in (("f32", 0), ("f16", 1), ("q8_0", 8)):
        got = oracle.dequant(t, g[f"arange_{name}_raw"], 64)
        np.testing.assert_array_equal(got, g[f"arange_{name}"])


@pytest.mark.parametrize("name,t", [("q4_0", 2), ("q8_0", 8)])
def test_dequant_random_blocks_bit_exact(oracle, golden, name, t):
    g = golden["gguf_dequant"]
    want = g[f"rand_{name}"]
    got = oracle.dequant(t, g[f"rand_{name}_raw"], want.size).reshape(want.shape)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequant_q4_0_scale_edge_cases(oracle, golden):
    g = golden["gguf_dequant"]
    got = oracle.dequant(2, g["edge_q4_0_raw"], g["edge_q4_0"].size).reshape(g["edge_q4_0"].shape)
    np.testing.assert_array_equal(got.view(np.uint32), g["edge_q4_0"].view(np.uint32))


@pytest.mark.parametrize("name,t", [("q4_1", 3), ("q5_0", 6), ("q5_1", 7)])
def test_dequant_other_nibble_formats_bit_exact(oracle, golden, name, t):
    """Q4_1 / Q5_0 / Q5_1 against the Python `gguf` package: random blocks and the fp16 edge classes."""
    g = golden["gguf_dequant_nibble"]
    for kind in ("rand", "edge"):
        want = g[f"{kind}_{name}"]
        got = oracle.dequant(t, g[f"{kind}_{name}_raw"], want.size).reshape(want.shape)
        np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


def test_half_to_float_all_bit_patterns(oracle):
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    got = np.array([oracle.half_to_float(int(x)) for x in h], dtype=np.float32)
    ok = ~np.isnan(want)
    np.testing.assert_array_equal(got.view(np.uint32)[ok], want.view(np.uint32)[ok])
    assert np.isnan(got[~ok]).all()


def test_dequant_rejects_unknown(oracle):
    with pytest.raises(ValueError):
        oracle.dequant(12, np.zeros(64, np.uint8), 32)
    with pytest.raises(ValueError):
        oracle.dequant(2, np.zeros(18, np.uint8), 17)  # Q4_0 needs whole blocks


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_matmul_vs_torch(oracle, golden, mode):
    # test-gemm.lisp:3-22: atol 1e-5 / rtol 1e-5 against torch.matmul
    g = golden["torch_ops"]
    c = oracle.linear(g["mm_a"], np.ascontiguousarray(g["mm_b"].T), mode=mode)
    np.testing.assert_allclose(c, g["mm_c"], atol=1e-5, rtol=1e-5)
    r = oracle.relu_matmul(g["mm_a"], g["mm_b"], mode=mode)
    np.testing.assert_allclose(r, g["relu_mm_c"], atol=1e-5, rtol=1e-5)
    assert (r >= 0).all()


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_layernorm_vs_torch(oracle, golden, mode):
    # test-normalization.lisp:48-55: atol 1e-5 / rtol 1e-2
    g = golden["torch_ops"]
    y = oracle.layernorm(g["ln_x"], g["ln_g"], g["ln_b"], mode=mode)
    np.testing.assert_allclose(y, g["ln_y"], atol=1e-5, rtol=1e-2)


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_gelu_vs_torch(oracle, golden, mode):
    # test-activations.lisp:176-184 compares with the tanh formula at 1e-6 for inputs in [-1, 1);
    # the fixture spans |x| up to ~15, where values reach ~15, hence the relative part
    g = golden["torch_ops"]
    np.testing.assert_allclose(oracle.gelu(g["gelu_x"], mode=mode), g["gelu_y"], atol=2e-6, rtol=2e-6)


def _sdpa_via_oracle(oracle, q, k, v, causal, mode):
    # q,k,v [B,H,T,64] -> the oracle's fused qkv rows / [B,T,H,hd] cache protocol, prefill of T tokens
    B, H, T, hd = q.shape
    d = H * hd
    qkv = np.concatenate([x.transpose(0, 2, 1, 3).reshape(B * T, d) for x in (q, k, v)], axis=1)
    kc = np.zeros((B, T, H, hd), np.float32)
    vc = np.zeros_like(kc)
    if causal:
        o = oracle.attention(qkv, kc, vc, B, T, 0, H, mode=mode)
    else:  # one query at a time against the full cache: decode protocol, no future to mask
        oracle.attention(qkv, kc, vc, B, T, 0, H, mode=mode)
        o = np.empty((B * T, d), np.float32)
        for i in range(T):
            kc2, vc2 = kc.copy(), vc.copy()
            # move row i to the end so that the query at position T-1 sees every key
            perm = [j for j in range(T) if j != i] + [i]
            kc2, vc2 = np.ascontiguousarray(kc2[:, perm]), np.ascontiguousarray(vc2[:, perm])
            row = qkv.reshape(B, T, 3 * d)[:, i]
            o.reshape(B, T, d)[:, i] = oracle.attention(row, kc2, vc2, B, 1, T - 1, H, mode=mode)
    return o.reshape(B, T, H, hd).transpose(0, 2, 1, 3)


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_sdpa_vs_torch(oracle, golden, mode):
    # test-llm.lisp:28-62: atol 1e-5 / rtol 1e-5
    g = golden["torch_ops"]
    o = _sdpa_via_oracle(oracle, g["sdpa_q"], g["sdpa_k"], g["sdpa_v"], True, mode)
    np.testing.assert_allclose(o, g["sdpa_causal_o"], atol=1e-5, rtol=1e-5)
    o = _sdpa_via_oracle(oracle, g["sdpa_q"], g["sdpa_k"], g["sdpa_v"], False, mode)
    np.testing.assert_allclose(o, g["sdpa_o"], atol=1e-5, rtol=1e-5)


def test_argmax_first_index_on_ties(oracle):
    x = np.zeros((3, 10), np.float32)
    x[0, [4, 7]] = 2.0
    x[1, :] = -1.0
    x[2, 9] = 5.0
    np.testing.assert_array_equal(oracle.argmax(x), [4, 0, 9])


def test_embedding_ignores_ids_outside_vocab(oracle):
    # the one-hot compare of nn/embedding.lisp:17-25 matches nothing: zero token row + position row
    wte = np.arange(12, dtype=np.float32).reshape(4, 3) + 1
    wpe = np.full((5, 3), 100.0, np.float32)
    out = oracle.embedding(np.array([[2, 7, -1, 1.5]], np.float32), 1, wte, wpe)
    np.testing.assert_array_equal(out[0, 0], wte[2] + 100)
    for i in (1, 2, 3):
        np.testing.assert_array_equal(out[0, i], [100, 100, 100])


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_gpt2_tiny_vs_torch_f64(oracle, golden, mode):
    """Whole model, prefill then cached decode, against an uncached float64 PyTorch forward."""
    g = golden["gpt2_tiny_f64"]
    p = S.GPT2Params(n_layers=2, n_heads=2, dim=128, vocab_size=1003)
    sd = S.synth_state_dict(p, "f32", seed=int(g["seed"]), max_seq_len=int(g["max_seq_len"]), trivial_affine=False,
                            weight_std=float(g["weight_std"]))
    prompt = g["prompt"]
    m = oracle.GPT2(p.n_layers, p.dim, p.n_heads, p.vocab_size, int(g["max_seq_len"]), prompt.shape[0], sd, mode=mode)
    ids, logits = m.step(prompt, 0)
    pos = prompt.shape[1]
    for i in range(g["new_ids"].shape[1]):
        np.testing.assert_allclose(logits, g["logits"][i], atol=1e-3 if mode < 2 else 1e-6, rtol=0)
        np.testing.assert_array_equal(ids, g["new_ids"][:, i])
        ids, logits = m.step(ids.reshape(-1, 1), pos)
        pos += 1
    m.close()


def test_gpt2_rejects_positions_outside_cache(oracle):
    p = S.GPT2Params(n_layers=1, n_heads=1, dim=64, vocab_size=50)
    sd = S.synth_state_dict(p, "f32", seed=0, max_seq_len=8)
    m = oracle.GPT2(1, 64, 1, 50, 8, 1, sd)
    with pytest.raises(ValueError):
        m.step(np.zeros((1, 9)), 0)
    m.close()


def test_variants_agree_to_rounding(oracle):
    """The three numeric variants differ by rounding only (the spread that decides whether a
    greedy id is comparable at all)."""
    p = S.GPT2Params(n_layers=2, n_heads=2, dim=128, vocab_size=257)
    sd = S.synth_state_dict(p, "f32", seed=9, max_seq_len=32, trivial_affine=False, weight_std=0.08)
    toks = S.synth_prompts(2, 12, 257, seed=1)
    lg = []
    for mode in (0, 1, 2):
        m = oracle.GPT2(2, 128, 2, 257, 32, 2, sd, mode=mode)
        lg.append(m.step(toks, 0)[1])
        m.close()
    assert np.abs(lg[0] - lg[2]).max() < 1e-4 and np.abs(lg[1] - lg[2]).max() < 1e-4


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_attention_block_vs_torch(oracle, golden, mode):
    """source/test-suite/test-llm.lisp:257-301: c_attn -> heads -> softmax attention -> c_proj against
    `attn_impl_torch` at the reference test's shape (10 x 3 x 32, 4 heads, no mask) and tolerance
    (atol 1e-4, rtol 1e-4); then the same block at head dim 64 with the causal mask."""
    g = golden["attn_block"]
    for tag, causal in (("ref", False), ("hd64", True)):
        x, H = g[f"{tag}_x"], int(g[f"{tag}_heads"])
        B, T, d = x.shape
        qkv = oracle.linear(x.reshape(B * T, d), g[f"{tag}_wa"], g[f"{tag}_ba"], mode=mode)
        q, k, v = (qkv[:, i * d:(i + 1) * d].reshape(B, T, H, d // H).transpose(0, 2, 1, 3) for i in range(3))
        o = _sdpa_via_oracle(oracle, q, k, v, causal, mode)
        y = oracle.linear(o.transpose(0, 2, 1, 3).reshape(B * T, d), g[f"{tag}_wp"], g[f"{tag}_bp"], mode=mode)
        np.testing.assert_allclose(y.reshape(B, T, d), g[f"{tag}_y"], atol=1e-4, rtol=1e-4)


def test_kv_cache_protocol(oracle):
    """source/test-suite/test-dynamic-shape.lisp:189-222 (`symbolic-k-cache-test`): a prompt of 10
    rows at start_pos 0, then one row per call; after every call the cache rows [0, start_pos + seq_len)
    are exactly the rows fed so far, in order, and the rest of the cache is still zero."""
    rng = np.random.Generator(np.random.PCG64(4))
    B, T, H, hd = 1, 128, 4, 4
    d = H * hd
    kc, vc = np.zeros((B, T, H, hd), np.float32), np.zeros((B, T, H, hd), np.float32)
    fed_k, fed_v, start = [], [], 0
    for nth in range(10):
        s = 10 if nth == 0 else 1
        qkv = rng.random((B * s, 3 * d), dtype=np.float32)
        oracle.attention(qkv, kc, vc, B, s, start, H)
        fed_k.append(qkv[:, d:2 * d]); fed_v.append(qkv[:, 2 * d:])
        start += s
        np.testing.assert_array_equal(kc[0, :start].reshape(start, d), np.concatenate(fed_k))
        np.testing.assert_array_equal(vc[0, :start].reshape(start, d), np.concatenate(fed_v))
        assert not kc[0, start:].any() and not vc[0, start:].any()


@pytest.mark.parametrize("mode", [0, 2])
def test_rmsnorm_and_rope_vs_torch(oracle, golden, mode):
    """source/test-suite/test-normalization.lisp:57-63 (RMSNorm, atol 1e-3 / rtol 1e-6) and test-rope.lisp:60-66
    (RoPE, atol 1e-5 / rtol 5e-4) against the torchtune functions those tests import."""
    g = golden["llama_ops"]
    for tag in ("ref", "wide"):
        np.testing.assert_allclose(oracle.rmsnorm(g[f"rms_{tag}_x"], mode=mode), g[f"rms_{tag}_y"], atol=1e-5, rtol=1e-6)
    for tag in ("ref", "hd64"):
        np.testing.assert_allclose(oracle.rope(g[f"rope_{tag}_x"], mode=mode), g[f"rope_{tag}_y"], atol=1e-5, rtol=5e-4)
    # a weight multiplies after the normalisation; an odd head dim keeps its last element
    x = g["rms_ref_x"]
    w = np.linspace(0.5, 1.5, x.shape[1]).astype(np.float32)
    np.testing.assert_allclose(oracle.rmsnorm(x, w, mode=mode), g["rms_ref_y"] * w, atol=1e-5, rtol=1e-6)
    odd = np.random.Generator(np.random.PCG64(1)).random((1, 4, 2, 7), dtype=np.float32)
    out = oracle.rope(odd, mode=mode)
    np.testing.assert_array_equal(out[..., 6], odd[..., 6])
    np.testing.assert_array_equal(out[:, 0], odd[:, 0])   # position 0: no rotation
