"""GPU parity tests of the whole GPT-2 step (prefill + KV-cached greedy decode) through the
C ABI, against the CPU oracle, on the same seeded synthetic weights."""
import numpy as np
import pytest

from caten_b200 import synthetic as S
from caten_b200._lib import B200Error
from caten_b200.gpt2 import GPT2, gpt2_generate, make_gpt2

pytestmark = pytest.mark.gpu


def dequantised(oracle, sd):
    out = {}
    for k, v in sd.items():
        out[k] = oracle.dequant(v.ggml_type, v.data, v.rows * v.cols).reshape(v.rows, v.cols) if isinstance(v, S.Packed) else v
    return out


def comparable_rows(l32, lmix, l64, margin=8.0):
    """Rows whose greedy id is decided by more than rounding: all three oracle variants agree and
    the float64 top-2 gap exceeds `margin` x the largest disagreement between the variants."""
    spread = max(np.abs(l32 - l64).max(), np.abs(lmix - l64).max(), 1e-7)
    top2 = np.sort(l64, axis=1)[:, -2:]
    gap = top2[:, 1] - top2[:, 0]
    agree = (l32.argmax(1) == l64.argmax(1)) & (lmix.argmax(1) == l64.argmax(1))
    return agree & (gap > margin * spread)


def run_parity(rt, oracle, p, wtype, precision, B, prompt_len, steps, T, logit_tol, seed=3, rel=False):
    sd = S.synth_state_dict(p, wtype, seed=seed, max_seq_len=T, trivial_affine=False, weight_std=0.08)
    fsd = dequantised(oracle, sd)
    prompt = S.synth_prompts(B, prompt_len, p.vocab_size, seed=seed + 1)
    orcs = [oracle.GPT2(p.n_layers, p.dim, p.n_heads, p.vocab_size, T, B, fsd, eps=p.norm_eps, mode=m) for m in (0, 1, 2)]
    g = GPT2(rt, p, sd, max_seq_len=T, batch=B, precision=precision)
    tokens, pos, checked, total = prompt, 0, 0, 0
    for step in range(steps):
        s = tokens.shape[1] - pos
        res = [o.step(tokens[:, pos:], pos) for o in orcs]
        ids = g.forward(tokens[:, pos:], s, pos)
        logits = g.logits()
        l32, lmix, l64 = (r[1] for r in res)
        err = np.abs(logits - l32).max()
        bound = logit_tol * (np.abs(l32).max() if rel else 1.0)
        assert err <= bound, f"step {step}: logits differ by {err} (bound {bound})"
        ok = comparable_rows(l32, lmix, l64)
        # with logits within `err` of the oracle's, the greedy id is only determined where the
        # oracle's top-2 gap exceeds 2 * err (this matters for the bf16 class, whose err is large)
        top2 = np.sort(l32, axis=1)[:, -2:]
        ok &= (top2[:, 1] - top2[:, 0]) > 2.0 * err
        np.testing.assert_array_equal(ids[ok], res[0][0][ok])
        np.testing.assert_array_equal(ids, logits.argmax(1))  # the kernel's argmax agrees with its own logits
        checked += int(ok.sum()); total += B
        pos = tokens.shape[1]
        tokens = np.concatenate([tokens, res[0][0].reshape(-1, 1)], axis=1)  # teacher forcing on the oracle's ids
    assert checked >= total // 2, "too few rows had a decisive top-2 gap; enlarge weight_std"
    # the KV cache holds what the oracle's holds (device layout [B,H,T,64], oracle [B,T,H,64])
    k_dev, v_dev = g.kv_cache(p.n_layers - 1)
    g.close()
    for o in orcs:
        o.close()
    return k_dev, v_dev


TINY = S.GPT2Params(n_layers=2, n_heads=2, dim=128, vocab_size=1003)


@pytest.mark.parametrize("wtype", ["f32", "q8_0", "q4_0"])
def test_tiny_fp32_parity(rt, oracle, wtype):
    # logits: max-abs 1e-3 (fp32 accumulate); greedy ids identical wherever rounding cannot decide
    run_parity(rt, oracle, TINY, wtype, "fp32", B=3, prompt_len=9, steps=7, T=48, logit_tol=1e-3)


@pytest.mark.parametrize("wtype", ["f32", "q4_0"])
def test_tiny_single_sequence_uses_gemv(rt, oracle, wtype):
    run_parity(rt, oracle, TINY, wtype, "fp32", B=1, prompt_len=3, steps=8, T=32, logit_tol=1e-3)


@pytest.mark.parametrize("wtype", ["q8_0", "q4_0"])
def test_tiny_bf16x3_parity(rt, oracle, wtype):
    run_parity(rt, oracle, TINY, wtype, "bf16x3", B=6, prompt_len=9, steps=5, T=48, logit_tol=1e-3)


@pytest.mark.parametrize("wtype", ["f32", "q4_0"])
def test_tiny_bf16_parity(rt, oracle, wtype):
    # bf16 tensor-core class: relative 2e-2
    run_parity(rt, oracle, TINY, wtype, "bf16", B=6, prompt_len=9, steps=4, T=48, logit_tol=2e-2, rel=True)


@pytest.mark.parametrize("wtype", ["q4_1", "q5_0", "q5_1"])
def test_tiny_other_packed_formats(rt, oracle, wtype):
    """The other 32-weight GGUF formats are consumed packed by the same kernels: one sequence (GEMV, one
    kernel per operation), the exact fp32 GEMM, and the tensor-core GEMM."""
    run_parity(rt, oracle, TINY, wtype, "fp32", B=1, prompt_len=3, steps=5, T=32, logit_tol=1e-3)
    run_parity(rt, oracle, TINY, wtype, "fp32", B=5, prompt_len=7, steps=3, T=32, logit_tol=1e-3)
    run_parity(rt, oracle, TINY, wtype, "bf16x3", B=6, prompt_len=9, steps=4, T=48, logit_tol=1e-3)


def test_gpt2_small_width_one_layer(rt, oracle):
    """Real GPT-2 small widths (d=768, 12 heads, d_ff=3072), one layer, reduced vocabulary."""
    p = S.GPT2Params(n_layers=1, n_heads=12, dim=768, vocab_size=4099)
    run_parity(rt, oracle, p, "q8_0", "fp32", B=2, prompt_len=16, steps=4, T=64, logit_tol=1e-3)


def test_gpt2_xl_width_one_layer(rt, oracle):
    """GPT-2 XL widths (d=1600, 25 heads: rows of 900 / 1700 packed bytes), one layer."""
    p = S.GPT2Params(n_layers=1, n_heads=25, dim=1600, vocab_size=2053)
    run_parity(rt, oracle, p, "q4_0", "fp32", B=1, prompt_len=5, steps=3, T=32, logit_tol=1e-3)


def test_golden_fixture_float64_torch(rt, golden):
    """Against the committed float64 PyTorch run (tests/golden/gpt2_tiny_f64.npz)."""
    g = golden["gpt2_tiny_f64"]
    sd = S.synth_state_dict(TINY, "f32", seed=int(g["seed"]), max_seq_len=int(g["max_seq_len"]), trivial_affine=False,
                            weight_std=float(g["weight_std"]))
    m = GPT2(rt, TINY, sd, max_seq_len=int(g["max_seq_len"]), batch=g["prompt"].shape[0], precision="fp32")
    toks = gpt2_generate(m, g["prompt"], max_length=g["new_ids"].shape[1])
    np.testing.assert_array_equal(toks[:, g["prompt"].shape[1]:], g["new_ids"])
    np.testing.assert_allclose(m.logits(), g["logits"][-1], atol=1e-3, rtol=0)
    m.close()


def test_device_resident_decode_matches_host_loop(rt):
    sd = S.synth_state_dict(TINY, "q4_0", seed=5, max_seq_len=40, trivial_affine=False, weight_std=0.08)
    prompt = S.synth_prompts(2, 6, TINY.vocab_size, seed=2)
    a = GPT2(rt, TINY, sd, max_seq_len=40, batch=2)
    toks = gpt2_generate(a, prompt, max_length=10)
    b = GPT2(rt, TINY, sd, max_seq_len=40, batch=2)
    first = b.forward(prompt, 6, 0)
    rest = b.decode_device(first, 6, 9)
    np.testing.assert_array_equal(np.concatenate([first.reshape(-1, 1), rest], 1), toks[:, 6:])
    assert b.launch_count > 0
    a.close(); b.close()


@pytest.mark.parametrize("precision,batch", [("fp32", 1), ("bf16x3", 6)])
def test_graph_replayed_decode_is_repeatable(rt, precision, batch):
    """`caten_b200_gpt2_decode` captures the step once and replays it: a second call (graph reuse),
    a call under per-kernel timing (eager launches) and the host loop must give the same ids."""
    sd = S.synth_state_dict(TINY, "q8_0", seed=11, max_seq_len=40, trivial_affine=False, weight_std=0.08)
    prompt = S.synth_prompts(batch, 5, TINY.vocab_size, seed=7)
    ref = GPT2(rt, TINY, sd, max_seq_len=40, batch=batch, precision=precision)
    want = gpt2_generate(ref, prompt, max_length=12)[:, 5:]
    m = GPT2(rt, TINY, sd, max_seq_len=40, batch=batch, precision=precision)
    first = m.forward(prompt, 5, 0)
    np.testing.assert_array_equal(first, want[:, 0])
    a = m.decode_device(first, 5, 11)          # eager first step + capture + replays
    b = m.decode_device(first, 5, 11)          # replays only
    rt.profile_begin(["attn_decode", "decode_step"])
    c = m.decode_device(first, 5, 4)           # eager launches while timing is on
    prof = rt.profile_end()
    if batch <= 4:   # a few sequences: the whole step is one kernel, timed as such
        assert prof["decode_step"][1] == 4 and "attn_decode" not in prof
    else:
        assert prof["attn_decode"][1] == 4 * TINY.n_layers
    np.testing.assert_array_equal(a, want[:, 1:])
    np.testing.assert_array_equal(b, a)
    np.testing.assert_array_equal(c, a[:, :4])
    with pytest.raises(B200Error):
        m.decode_device(first, 38, 5)          # would run past the cache
    ref.close(); m.close()


WIDE = S.GPT2Params(n_layers=2, n_heads=8, dim=512, vocab_size=1003)  # wide enough for split-K linears


def test_wide_bf16x3_parity_with_split_k(rt, oracle):
    """d=512: the decode linears run split-K and their consumers (LayerNorm, attention) sum the
    partial tiles; same bounds as every other bf16x3 case."""
    run_parity(rt, oracle, WIDE, "q4_0", "bf16x3", B=6, prompt_len=7, steps=5, T=40, logit_tol=1e-3)


def test_deferred_split_k_reduction_is_bit_identical(rt, monkeypatch):
    """Summing the split-K partial tiles inside the consuming kernel gives the same bits as the
    separate reduction kernel (same order of additions)."""
    sd = S.synth_state_dict(WIDE, "q4_0", seed=9, max_seq_len=40, trivial_affine=False, weight_std=0.08)
    prompt = S.synth_prompts(6, 5, WIDE.vocab_size, seed=8)
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("CATEN_B200_DEFER_REDUCE", flag)
        m = GPT2(rt, WIDE, sd, max_seq_len=40, batch=6, precision="bf16x3")
        first = m.forward(prompt, 5, 0)
        ids = m.decode_device(first, 5, 6)
        launches = m.launch_count
        nxt = m.forward(ids[:, -1:], 1, 11)
        outs.append((first, ids, nxt, m.logits().copy(), launches))
        m.close()
    for a, b in zip(outs[0][:4], outs[1][:4]):
        np.testing.assert_array_equal(a.view(np.uint32) if a.dtype == np.float32 else a, b.view(np.uint32) if b.dtype == np.float32 else b)
    assert outs[0][4] < outs[1][4]  # fewer kernels per step


def test_prefill_in_chunks_equals_one_pass(rt):
    """max_rows forces the prefill to run sequence group by sequence group."""
    sd = S.synth_state_dict(TINY, "q8_0", seed=6, max_seq_len=32, trivial_affine=False, weight_std=0.08)
    prompt = S.synth_prompts(5, 8, TINY.vocab_size, seed=3)
    a = GPT2(rt, TINY, sd, max_seq_len=32, batch=5)
    b = GPT2(rt, TINY, sd, max_seq_len=32, batch=5, max_rows=16)  # two sequences at a time
    ia, ib = a.forward(prompt, 8, 0), b.forward(prompt, 8, 0)
    np.testing.assert_array_equal(ia, ib)
    np.testing.assert_array_equal(a.logits(), b.logits())
    a.close(); b.close()


def test_chunked_prompt_equals_whole_prompt(rt):
    """Feeding the prompt in two calls (n = 0 then n = 5) fills the cache like one call does."""
    sd = S.synth_state_dict(TINY, "f32", seed=7, max_seq_len=32, trivial_affine=False, weight_std=0.08)
    prompt = S.synth_prompts(2, 11, TINY.vocab_size, seed=4)
    a = GPT2(rt, TINY, sd, max_seq_len=32, batch=2)
    b = GPT2(rt, TINY, sd, max_seq_len=32, batch=2)
    a.forward(prompt, 11, 0)
    b.forward(prompt[:, :5], 5, 0)
    b.forward(prompt[:, 5:], 6, 5)
    np.testing.assert_allclose(a.logits(), b.logits(), atol=1e-5, rtol=0)
    ka, _ = a.kv_cache(1)
    kb, _ = b.kv_cache(1)
    np.testing.assert_allclose(ka[:, :, :11], kb[:, :, :11], atol=1e-5, rtol=0)
    assert not ka[:, :, 11:].any()  # untouched positions stay zero (layers.lisp:25-26)
    a.close(); b.close()


def test_step_errors(rt):
    sd = S.synth_state_dict(TINY, "f32", seed=8, max_seq_len=16)
    m = GPT2(rt, TINY, sd, max_seq_len=16, batch=1)
    with pytest.raises(B200Error):
        m.forward(np.zeros((1, 17)), 17, 0)       # longer than the cache
    with pytest.raises(B200Error):
        m.forward(np.zeros((1, 4)), 4, 14)        # runs past the end
    m.forward(np.zeros((1, 4)), 4, 0)             # still usable afterwards
    m.close()
    bad = S.GPT2Params(n_layers=1, n_heads=4, dim=128, vocab_size=50)  # head dim 32
    with pytest.raises(B200Error):
        GPT2(rt, bad, S.synth_state_dict(bad, "f32", seed=0, max_seq_len=8), max_seq_len=8)


def test_make_gpt2_by_name(rt):
    with pytest.raises(KeyError):
        make_gpt2("gpt3", {}, runtime=rt)


def test_closing_after_the_runtime_is_gone_is_harmless():
    """A model, weight or buffer that outlives its runtime (a failed test, interpreter exit) must
    not call into the library with a destroyed context."""
    from caten_b200.runtime import B200Runtime
    r = B200Runtime(0)
    sd = S.synth_state_dict(TINY, "q8_0", seed=1, max_seq_len=16, trivial_affine=False, weight_std=0.08)
    g = GPT2(r, TINY, sd, max_seq_len=16, batch=2)
    buf = r.open_buffer((4, 4))
    g.forward(S.synth_prompts(2, 3, TINY.vocab_size, seed=1), 3, 0)
    r.close()
    buf.close()
    g.close()
    del g


@pytest.mark.parametrize("wtype,batch,params,head", [("q4_0", 1, TINY, None), ("q8_0", 3, TINY, None), ("q4_0", 4, WIDE, None),
                                                     ("q8_0", 2, TINY, np.float32), ("q4_0", 1, WIDE, np.float16)])
def test_single_kernel_decode_step_matches_kernel_per_operation_path(rt, oracle, monkeypatch, wtype, batch, params, head):
    """With 1..4 sequences and block-quantised layers a single-token step is one kernel (weights streamed through shared memory,
    activations exchanged as tagged words); CATEN_B200_PERSISTENT=0 keeps the kernel-per-operation
    path.  Same inputs through both: logits within 1e-4, ids equal where the top-2 gap is decisive,
    identical KV cache rows, and the strict-fp32 oracle within 1e-3 (the bar of every fp32 path)."""
    T = 160
    sd = S.synth_state_dict(params, wtype, seed=13, max_seq_len=T, trivial_affine=False, weight_std=0.08)
    fsd = {k: (oracle.dequant(v.ggml_type, v.data, v.rows * v.cols).reshape(v.rows, v.cols) if isinstance(v, S.Packed) else v)
           for k, v in sd.items()}
    if head is not None:   # a dense output matrix (fp32 or fp16) behind quantised layers, as some GGUF files have
        sd["lm_head.weight"] = fsd["lm_head.weight"].astype(head)
        fsd["lm_head.weight"] = sd["lm_head.weight"].astype(np.float32)
    prompt = S.synth_prompts(batch, 70, params.vocab_size, seed=3)   # long enough for several context chunks per head
    monkeypatch.setenv("CATEN_B200_PERSISTENT", "0")
    old = GPT2(rt, params, sd, max_seq_len=T, batch=batch)
    monkeypatch.setenv("CATEN_B200_PERSISTENT", "1")
    new = GPT2(rt, params, sd, max_seq_len=T, batch=batch)
    ref = oracle.GPT2(params.n_layers, params.dim, params.n_heads, params.vocab_size, T, batch, fsd)
    ids_ref, _ = ref.step(prompt, 0)
    assert (old.forward(prompt, 70, 0) == new.forward(prompt, 70, 0)).all()   # the prompt runs the same kernels in both
    tok, pos = ids_ref.reshape(-1, 1), 70
    for step in range(12):
        ids_ref, lg_ref = ref.step(tok, pos)
        ia, ib = old.forward(tok, 1, pos), new.forward(tok, 1, pos)
        la, lb = old.logits(), new.logits()
        err = float(np.abs(la - lb).max())
        assert err <= 1e-4, (step, err)
        assert np.abs(lb - lg_ref).max() <= 1e-3
        top2 = np.sort(lg_ref, axis=1)[:, -2:]
        ok = (top2[:, 1] - top2[:, 0]) > 1e-3
        np.testing.assert_array_equal(ib[ok], ids_ref[ok])
        np.testing.assert_array_equal(ib[ok], ia[ok])
        tok, pos = ids_ref.reshape(-1, 1), pos + 1
    for layer in (0, params.n_layers - 1):
        (ka, va), (kb, vb) = old.kv_cache(layer), new.kv_cache(layer)
        np.testing.assert_allclose(kb[:, :, :pos], ka[:, :, :pos], atol=1e-4, rtol=0)
        np.testing.assert_allclose(vb[:, :, :pos], va[:, :, :pos], atol=1e-4, rtol=0)
        assert not kb[:, :, pos:].any() and not vb[:, :, pos:].any()
    # device-resident decode (ids and position never leave the GPU) gives the host loop's ids
    first = new.forward(prompt, 70, 0)
    want = [first]
    for i in range(5):
        want.append(new.forward(want[-1].reshape(-1, 1), 1, 70 + i))
    got = new.decode_device(first, 70, 5)
    np.testing.assert_array_equal(got, np.stack(want[1:], axis=1))
    old.close(); new.close(); ref.close()
