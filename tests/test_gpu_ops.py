"""GPU parity tests of the individual kernels, through the C ABI, against the CPU oracle."""
import numpy as np
import pytest

from caten_b200 import _lib as L
from caten_b200 import synthetic as S
from caten_b200._lib import B200Error

pytestmark = pytest.mark.gpu

TYPES = {"f32": 0, "f16": 1, "q4_0": 2, "q8_0": 8}


def make_weight(rng, rows, cols, wtype, std=0.05):
    """Returns (uploadable, ggml_type, raw bytes for the oracle)."""
    if wtype == "f32":
        a = (rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(std))
        return a, 0, a.view(np.uint8).reshape(-1)
    if wtype == "f16":
        a = (rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(std)).astype(np.float16)
        return a, 1, a.view(np.uint8).reshape(-1)
    p = S._rand_packed(rng, rows, cols, wtype, std)
    return p, p.ggml_type, p.data


def acc_check(got, ref32, ref64, slack=4.0, floor=1e-6):
    """`got` must be about as close to the float64 result as the strict-fp32 oracle is."""
    scale = max(1.0, float(np.abs(ref64).max()))
    e_ref = float(np.abs(ref32 - ref64).max())
    e_got = float(np.abs(got - ref64).max())
    assert e_got <= slack * e_ref + floor * scale, (e_got, e_ref)


@pytest.mark.parametrize("wtype", ["q4_0", "q8_0", "f16", "f32"])
def test_dequant_bit_exact(rt, oracle, wtype):
    rng = np.random.Generator(np.random.PCG64(1))
    up, t, raw = make_weight(rng, 37, 160, wtype)
    w = rt.upload_weight(up)
    got = w.dequantize()
    want = oracle.dequant(t, raw, 37 * 160).reshape(37, 160)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    w.close()


def test_dequant_golden_fixture(rt, golden):
    g = golden["gguf_dequant"]
    for name, t, bb in (("q4_0", 2, 18), ("q8_0", 8, 34)):
        w = rt.upload_weight(S.Packed(t, 6, 96, g[f"rand_{name}_raw"]))
        np.testing.assert_array_equal(w.dequantize().view(np.uint32), g[f"rand_{name}"].view(np.uint32))
        w.close()
    w = rt.upload_weight(S.Packed(2, 6, 32, g["edge_q4_0_raw"]))  # zero / subnormal / negative / max scales
    np.testing.assert_array_equal(w.dequantize().view(np.uint32), g["edge_q4_0"].view(np.uint32))
    w.close()
    w = rt.upload_weight(S.Packed(8, 1, 64, g["arange_q8_0_raw"]))  # the reference's own 64-element fixture
    np.testing.assert_array_equal(w.dequantize().reshape(-1), g["arange_q8_0"])
    w.close()


def test_weight_upload_rejects_bad_input(rt):
    with pytest.raises(B200Error) as e:
        rt.upload_weight(S.Packed(12, 4, 64, np.zeros(1000, np.uint8)))
    assert e.value.code == L.EUNSUPPORTED
    with pytest.raises(B200Error):
        rt.upload_weight(S.Packed(2, 4, 48, np.zeros(1000, np.uint8)))  # cols not a multiple of 32


@pytest.mark.parametrize("rows,d", [(1, 128), (7, 768), (33, 1600), (5, 2048)])
def test_layernorm(rt, oracle, rows, d):
    rng = np.random.Generator(np.random.PCG64(rows + d))
    x = rng.standard_normal((rows, d), dtype=np.float32) * 3 + 1
    g = rng.standard_normal(d, dtype=np.float32)
    b = rng.standard_normal(d, dtype=np.float32)
    y = rt.layernorm(rt.transfer_from_array(x), rt.transfer_from_array(g), rt.transfer_from_array(b)).numpy()
    np.testing.assert_allclose(y, oracle.layernorm(x, g, b, mode=0), atol=1e-5, rtol=1e-5)
    acc_check(y, oracle.layernorm(x, g, b, mode=0), oracle.layernorm(x, g, b, mode=2), slack=6.0)


def test_layernorm_golden(rt, golden):
    g = golden["torch_ops"]
    y = rt.layernorm(rt.transfer_from_array(g["ln_x"]), rt.transfer_from_array(g["ln_g"]), rt.transfer_from_array(g["ln_b"])).numpy()
    np.testing.assert_allclose(y, g["ln_y"], atol=1e-5, rtol=1e-2)  # the reference's tolerance


def test_layernorm_unsupported_width(rt):
    x = rt.open_buffer((2, 4100))
    with pytest.raises(B200Error) as e:
        rt.layernorm(x, x, x)
    assert e.value.code == L.EUNSUPPORTED


@pytest.mark.parametrize("dtype", [np.float32, np.int64])
def test_embed(rt, oracle, dtype):
    rng = np.random.Generator(np.random.PCG64(3))
    V, T, d = 301, 24, 192
    wte = rng.standard_normal((V, d), dtype=np.float32)
    wpe = rng.standard_normal((T, d), dtype=np.float32)
    ids = rng.integers(0, V, size=(3, 7))
    ids[1, 2] = V + 5      # outside the vocabulary: zero token row
    ids[2, 0] = -3
    got = rt.embed(rt.transfer_from_array(ids, dtype), rt.transfer_from_array(wte), rt.transfer_from_array(wpe), 5).numpy()
    want = oracle.embedding(ids.astype(np.float32), 5, wte, wpe)
    np.testing.assert_array_equal(got, want)
    if dtype == np.float32:
        frac = ids.astype(np.float32)
        frac[0, 0] += 0.5  # a non-integer id matches no row either
        got = rt.embed(rt.transfer_from_array(frac), rt.transfer_from_array(wte), rt.transfer_from_array(wpe), 5).numpy()
        np.testing.assert_array_equal(got, oracle.embedding(frac, 5, wte, wpe))


def test_argmax(rt, oracle):
    rng = np.random.Generator(np.random.PCG64(4))
    x = rng.standard_normal((5, 50257), dtype=np.float32)
    x[0, [100, 40000]] = 9.0          # tie: lowest index wins
    x[1, :] = 0.25                    # all equal
    x[2, 50256] = 11.0                # last element
    x[3, 0] = 12.0
    got = rt.argmax(rt.transfer_from_array(x)).numpy()
    np.testing.assert_array_equal(got, oracle.argmax(x))
    assert got[0] == 100 and got[1] == 0 and got[2] == 50256 and got[3] == 0


GEMV_SHAPES = [(96, 128), (200, 768), (1000, 1600), (130, 3072), (77, 6400)]


@pytest.mark.parametrize("wtype", ["q4_0", "q8_0", "f32", "f16"])
@pytest.mark.parametrize("N,K", GEMV_SHAPES)
def test_gemv(rt, oracle, wtype, N, K):
    rng = np.random.Generator(np.random.PCG64(N * 7 + K))
    up, t, raw = make_weight(rng, N, K, wtype)
    Wf = oracle.dequant(t, raw, N * K).reshape(N, K)
    x = rng.standard_normal((1, K), dtype=np.float32) * 2
    bias = rng.standard_normal(N, dtype=np.float32)
    res = rng.standard_normal((1, N), dtype=np.float32)
    w = rt.upload_weight(up)
    dx, db, dr = rt.transfer_from_array(x), rt.transfer_from_array(bias), rt.transfer_from_array(res)
    for act in (L.ACT_NONE, L.ACT_GELU):
        got = rt.linear(w, dx, db, dr, act).numpy()
        r32 = oracle.linear(x, Wf, bias, res, act, mode=0)
        r64 = oracle.linear(x, Wf, bias, res, act, mode=2)
        np.testing.assert_allclose(got, r32, atol=1e-4, rtol=1e-4)
        acc_check(got, r32, r64)
    got = rt.linear(w, dx).numpy()  # no bias, no residual
    np.testing.assert_allclose(got, oracle.linear(x, Wf, mode=0), atol=1e-4, rtol=1e-4)
    w.close()


def test_gemv_up_to_four_rows(rt, oracle):
    rng = np.random.Generator(np.random.PCG64(8))
    up, t, raw = make_weight(rng, 300, 1024, "q4_0")
    Wf = oracle.dequant(t, raw, 300 * 1024).reshape(300, 1024)
    x = rng.standard_normal((4, 1024), dtype=np.float32)
    res = rng.standard_normal((4, 300), dtype=np.float32)
    w = rt.upload_weight(up)
    got = rt.linear(w, rt.transfer_from_array(x), None, rt.transfer_from_array(res)).numpy()
    np.testing.assert_allclose(got, oracle.linear(x, Wf, None, res, mode=0), atol=1e-4, rtol=1e-4)
    w.close()


def test_gemv_large_activations_and_zero_scale(rt, oracle):
    """The Q4_0 path pre-scales x by powers of two: large and tiny activations must survive."""
    rng = np.random.Generator(np.random.PCG64(9))
    up, t, raw = make_weight(rng, 64, 256, "q4_0")
    Wf = oracle.dequant(t, raw, 64 * 256).reshape(64, 256)
    w = rt.upload_weight(up)
    for mag in (1e-12, 1e-3, 1e6, 1e12):
        x = rng.standard_normal((1, 256), dtype=np.float32) * np.float32(mag)
        got = rt.linear(w, rt.transfer_from_array(x)).numpy()
        ref = oracle.linear(x, Wf, mode=2)
        assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max()
    w.close()


SIMT_CASES = [("f32", 5, 96, 64), ("q4_0", 70, 200, 256), ("q8_0", 33, 130, 128), ("f16", 9, 64, 96)]


@pytest.mark.parametrize("wtype,M,N,K", SIMT_CASES)
def test_gemm_fp32_is_bit_exact(rt, oracle, wtype, M, N, K):
    """PREC_FP32 accumulates k in ascending order with a rounded multiply and a rounded add:
    the same arithmetic as the reference's rendered C loop, hence identical bits."""
    rng = np.random.Generator(np.random.PCG64(M + N + K))
    up, t, raw = make_weight(rng, N, K, wtype)
    Wf = oracle.dequant(t, raw, N * K).reshape(N, K)
    x = rng.standard_normal((M, K), dtype=np.float32)
    bias = rng.standard_normal(N, dtype=np.float32)
    res = rng.standard_normal((M, N), dtype=np.float32)
    w = rt.upload_weight(up)
    dx, db, dr = rt.transfer_from_array(x), rt.transfer_from_array(bias), rt.transfer_from_array(res)
    got = rt.linear(w, dx, db, dr, L.ACT_RELU, L.PREC_FP32).numpy()
    want = oracle.linear(x, Wf, bias, res, 2, mode=0)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    got = rt.linear(w, dx, db, None, L.ACT_GELU, L.PREC_FP32).numpy()
    np.testing.assert_allclose(got, oracle.linear(x, Wf, bias, None, 1, mode=0), atol=2e-6, rtol=2e-6)
    w.close()


TC_CASES = [("q4_0", 256, 1600, 6400), ("q4_0", 32, 1600, 1600), ("q4_0", 8, 128, 64), ("q4_0", 5, 200, 128), ("q4_0", 64, 4800, 1600), ("q8_0", 33, 130, 192),
            ("f32", 130, 256, 128), ("f16", 17, 128, 64), ("q4_0", 300, 384, 256), ("q8_0", 256, 256, 768)]


@pytest.mark.parametrize("wtype,M,N,K", TC_CASES)
@pytest.mark.parametrize("prec", ["bf16", "bf16x3"])
def test_gemm_tensor_core(rt, oracle, wtype, M, N, K, prec):
    rng = np.random.Generator(np.random.PCG64(M * 3 + N + K))
    up, t, raw = make_weight(rng, N, K, wtype)
    Wf = oracle.dequant(t, raw, N * K).reshape(N, K)
    x = rng.standard_normal((M, K), dtype=np.float32)
    bias = rng.standard_normal(N, dtype=np.float32) * 0.1
    res = rng.standard_normal((M, N), dtype=np.float32) * 0.1
    w = rt.upload_weight(up)
    dx, db, dr = rt.transfer_from_array(x), rt.transfer_from_array(bias), rt.transfer_from_array(res)
    oracle.set_threads(8)
    ref_lin = oracle.linear(x, Wf, mode=0)
    ref = oracle.linear(x, Wf, bias, res, 1, mode=0)
    oracle.set_threads(1)
    got_lin = rt.linear(w, dx, None, None, L.ACT_NONE, L.PRECISIONS[prec]).numpy()
    got = rt.linear(w, dx, db, dr, L.ACT_GELU, L.PRECISIONS[prec]).numpy()
    rt.sync()
    tol = 2e-2 if prec == "bf16" else 1e-4   # relative to the largest output
    assert np.abs(got_lin - ref_lin).max() <= tol * np.abs(ref_lin).max()
    assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())
    w.close()


# thousands of rows: the weights are expanded to bf16 once and both operands reach the tensor cores through TMA
# (persistent kernel, two accumulators).  Ragged rows and features, every weight format, both precisions.
MANY_ROW_CASES = [("q4_0", 2048, 2560, 1600), ("q4_0", 2000, 2500, 768), ("q8_0", 1100, 4800, 128), ("q5_1", 1500, 3200, 256),
                  ("f32", 1024, 4864, 192), ("f16", 4100, 1200, 64)]


@pytest.mark.parametrize("wtype,M,N,K", MANY_ROW_CASES)
@pytest.mark.parametrize("prec", ["bf16", "bf16x3"])
def test_gemm_tensor_core_many_rows(rt, oracle, wtype, M, N, K, prec):
    rng = np.random.Generator(np.random.PCG64(M + 7 * N + K))
    up, t, raw = make_weight(rng, N, K, wtype)
    Wf = oracle.dequant(t, raw, N * K).reshape(N, K)
    x = rng.standard_normal((M, K), dtype=np.float32)
    bias = rng.standard_normal(N, dtype=np.float32) * 0.1
    res = rng.standard_normal((M, N), dtype=np.float32) * 0.1
    w = rt.upload_weight(up)
    dx, db, dr = rt.transfer_from_array(x), rt.transfer_from_array(bias), rt.transfer_from_array(res)
    ref_lin = (x.astype(np.float64) @ Wf.T.astype(np.float64))
    got_lin = rt.linear(w, dx, None, None, L.ACT_NONE, L.PRECISIONS[prec]).numpy()
    got = rt.linear(w, dx, db, dr, L.ACT_GELU, L.PRECISIONS[prec]).numpy()
    rt.sync()
    tol = 2e-2 if prec == "bf16" else 1e-4   # relative to the largest output
    assert np.abs(got_lin - ref_lin).max() <= tol * np.abs(ref_lin).max()
    # bias, GELU (as the reference composes it) and residual on a sample of rows through the oracle
    rows = np.unique(np.concatenate([np.arange(0, 8), np.arange(M - 8, M), rng.integers(0, M, 48)]))
    ref = oracle.linear(x[rows], Wf, bias, res[rows], 1, mode=0)
    assert np.abs(got[rows] - ref).max() <= tol * max(1.0, np.abs(ref).max())
    # and everywhere against the kernel's own un-fused result
    z = got_lin + bias
    full = res + 0.5 * z * (1.0 + np.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
    assert np.abs(got - full).max() <= 1e-4 * max(1.0, np.abs(full).max())
    w.close()


def test_gemm_many_rows_matches_the_tile_per_cta_kernel(oracle, monkeypatch):
    """CATEN_B200_DENSE_GEMM=0 sends many-row linears through the decode GEMM (weights dequantised inside the
    kernel): the two kernels must agree to split-bf16 accuracy, and relu(matmul) likewise."""
    from caten_b200.runtime import B200Runtime
    rng = np.random.Generator(np.random.PCG64(91))
    up, _, _ = make_weight(rng, 2560, 1600, "q4_0")
    x = rng.standard_normal((2048, 1600), dtype=np.float32)
    a, b = S.synth_relu_gemm(seed=1, M=4096, K=768, N=3072)
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("CATEN_B200_DENSE_GEMM", flag)
        with B200Runtime(0) as r2:
            w = r2.upload_weight(up)
            y = r2.linear(w, r2.transfer_from_array(x), None, None, L.ACT_NONE, L.PREC_BF16X3).numpy()
            c = r2.relu_matmul(r2.transfer_from_array(a), r2.transfer_from_array(b), L.PREC_BF16X3).numpy()
            r2.sync()
            outs.append((y, c))
            w.close()
    assert np.abs(outs[0][0] - outs[1][0]).max() <= 1e-4 * np.abs(outs[1][0]).max()
    assert np.abs(outs[0][1] - outs[1][1]).max() <= 1e-4 * np.abs(outs[1][1]).max()
    ref = np.maximum(a[:64].astype(np.float64) @ b.astype(np.float64), 0.0)
    np.testing.assert_allclose(outs[0][1][:64], ref, atol=1e-5, rtol=1e-5)   # test-gemm.lisp:3-22


def test_gemm_tensor_core_split_k_is_deterministic(rt):
    """Few output tiles and a long inner dimension: several CTAs share a tile (split-K) and the
    last one to finish adds the partial tiles in a fixed order, so repeated runs give equal bits."""
    rng = np.random.Generator(np.random.PCG64(33))
    up, _, _ = make_weight(rng, 256, 6400, "q4_0")
    w = rt.upload_weight(up)
    dx = rt.transfer_from_array(rng.standard_normal((64, 6400), dtype=np.float32))
    first = rt.linear(w, dx, None, None, L.ACT_NONE, L.PREC_BF16X3).numpy()
    for _ in range(5):
        again = rt.linear(w, dx, None, None, L.ACT_NONE, L.PREC_BF16X3).numpy()
        np.testing.assert_array_equal(first.view(np.uint32), again.view(np.uint32))
    w.close()


def test_gemm_tensor_core_in_place_residual(rt, oracle):
    rng = np.random.Generator(np.random.PCG64(21))
    up, t, raw = make_weight(rng, 128, 128, "q4_0")
    Wf = oracle.dequant(t, raw, 128 * 128).reshape(128, 128)
    x = rng.standard_normal((40, 128), dtype=np.float32)
    h = rng.standard_normal((40, 128), dtype=np.float32)
    w = rt.upload_weight(up)
    dh = rt.transfer_from_array(h)
    rt.linear(w, rt.transfer_from_array(x), None, dh, L.ACT_NONE, L.PREC_BF16X3, out=dh)
    ref = oracle.linear(x, Wf, None, h, mode=0)
    assert np.abs(dh.numpy() - ref).max() <= 1e-4 * np.abs(ref).max()
    w.close()


@pytest.mark.parametrize("prec,tol", [("fp32", 0.0), ("bf16x3", 1e-5), ("bf16", 2e-2)])
def test_relu_matmul(rt, oracle, prec, tol):
    a, b = S.synth_relu_gemm(seed=1, M=200, K=768, N=384)
    oracle.set_threads(8)
    ref = oracle.relu_matmul(a, b, mode=0)
    oracle.set_threads(1)
    got = rt.relu_matmul(rt.transfer_from_array(a), rt.transfer_from_array(b), L.PRECISIONS[prec]).numpy()
    assert (got >= 0).all()
    if prec == "fp32":
        np.testing.assert_array_equal(got.view(np.uint32), ref.view(np.uint32))
    elif prec == "bf16x3":
        np.testing.assert_allclose(got, ref, atol=1e-5, rtol=1e-5)  # test-gemm.lisp:3-22
    else:
        assert np.abs(got - ref).max() <= tol * np.abs(ref).max()


def test_relu_matmul_golden(rt, golden):
    g = golden["torch_ops"]
    a = np.zeros((37, 64), np.float32); a[:] = g["mm_a"]
    got = rt.relu_matmul(rt.transfer_from_array(a), rt.transfer_from_array(g["mm_b"]), L.PREC_FP32).numpy()
    np.testing.assert_allclose(got, g["relu_mm_c"], atol=1e-5, rtol=1e-5)


def _to_gpu_cache(c):  # oracle [B,T,H,hd] -> device [B,H,T,hd]
    return np.ascontiguousarray(c.transpose(0, 2, 1, 3))


@pytest.mark.parametrize("B,H,T", [(1, 1, 16), (3, 2, 40), (2, 12, 300)])
def test_attention_decode_steps(rt, oracle, B, H, T):
    rng = np.random.Generator(np.random.PCG64(B + H + T))
    d = H * 64
    kc = np.zeros((B, T, H, 64), np.float32)
    vc = np.zeros_like(kc)
    dk, dv = rt.open_buffer((B, H, T, 64)), rt.open_buffer((B, H, T, 64))
    n0 = T - 6
    if n0 > 0:  # pre-existing context
        kc[:, :n0] = rng.standard_normal((B, n0, H, 64), dtype=np.float32)
        vc[:, :n0] = rng.standard_normal((B, n0, H, 64), dtype=np.float32)
        dk.close(); dv.close()
        dk, dv = rt.transfer_from_array(_to_gpu_cache(kc)), rt.transfer_from_array(_to_gpu_cache(vc))
    for n in range(max(n0, 0), T):
        qkv = rng.standard_normal((B, 3 * d), dtype=np.float32)
        want = oracle.attention(qkv, kc, vc, B, 1, n, H, mode=0)
        got = rt.attention(rt.transfer_from_array(qkv), dk, dv, B, 1, n).numpy()
        np.testing.assert_allclose(got, want, atol=1e-5, rtol=1e-5)
    np.testing.assert_array_equal(dk.numpy(), _to_gpu_cache(kc))
    np.testing.assert_array_equal(dv.numpy(), _to_gpu_cache(vc))


@pytest.mark.parametrize("B,H,T,s,n", [(2, 2, 64, 5, 0), (1, 3, 200, 64, 0), (2, 1, 200, 70, 9), (1, 2, 300, 130, 40), (1, 1, 8, 2, 6)])
def test_attention_prefill(rt, oracle, B, H, T, s, n):
    rng = np.random.Generator(np.random.PCG64(B + H + T + s + n))
    d = H * 64
    kc = np.zeros((B, T, H, 64), np.float32)
    vc = np.zeros_like(kc)
    kc[:, :n] = rng.standard_normal((B, n, H, 64), dtype=np.float32)
    vc[:, :n] = rng.standard_normal((B, n, H, 64), dtype=np.float32)
    dk, dv = rt.transfer_from_array(_to_gpu_cache(kc)), rt.transfer_from_array(_to_gpu_cache(vc))
    qkv = rng.standard_normal((B * s, 3 * d), dtype=np.float32)
    want = oracle.attention(qkv, kc, vc, B, s, n, H, mode=0)
    got = rt.attention(rt.transfer_from_array(qkv), dk, dv, B, s, n).numpy()
    np.testing.assert_allclose(got, want, atol=1e-5, rtol=1e-5)
    np.testing.assert_array_equal(dk.numpy(), _to_gpu_cache(kc))
    np.testing.assert_array_equal(dv.numpy(), _to_gpu_cache(vc))


@pytest.mark.parametrize("B,H,T,s,n", [(2, 2, 64, 5, 0), (1, 3, 200, 64, 0), (2, 1, 200, 70, 9), (1, 2, 300, 130, 40),
                                       (1, 1, 8, 2, 6), (2, 2, 600, 300, 0), (1, 2, 700, 257, 391), (1, 1, 1024, 128, 896),
                                       (3, 1, 520, 129, 127)])
def test_attention_prefill_tensor_cores(rt, oracle, B, H, T, s, n):
    """q.K^T and P.V as split-bf16 tensor-core products: within 2^-16-class error of the fp32
    statement, the cache append still exact; tiles of 128 queries x 128 keys, so the cases cover
    partial tiles, several tiles, and a history that starts inside a key step."""
    rng = np.random.Generator(np.random.PCG64(B + H + T + s + n))
    d = H * 64
    kc = np.zeros((B, T, H, 64), np.float32)
    vc = np.zeros_like(kc)
    kc[:, :n] = rng.standard_normal((B, n, H, 64), dtype=np.float32)
    vc[:, :n] = rng.standard_normal((B, n, H, 64), dtype=np.float32)
    # stale rows past the end of the context must not leak in (they are masked, and 0 * NaN would show)
    kg, vg = _to_gpu_cache(kc), _to_gpu_cache(vc)
    kg[:, :, n + s:] = np.nan
    vg[:, :, n + s:] = np.nan
    dk, dv = rt.transfer_from_array(kg), rt.transfer_from_array(vg)
    qkv = rng.standard_normal((B * s, 3 * d), dtype=np.float32)
    want = oracle.attention(qkv, kc, vc, B, s, n, H, mode=0)
    for prec in (L.PREC_BF16X3, L.PREC_BF16):
        got = rt.attention(rt.transfer_from_array(qkv), dk, dv, B, s, n, precision=prec).numpy()
        np.testing.assert_allclose(got, want, atol=2e-5, rtol=2e-5)
    np.testing.assert_array_equal(dk.numpy()[:, :, :n + s], _to_gpu_cache(kc)[:, :, :n + s])
    np.testing.assert_array_equal(dv.numpy()[:, :, :n + s], _to_gpu_cache(vc)[:, :, :n + s])


@pytest.mark.parametrize("B,H,T,s,n,grow", [(2, 2, 600, 300, 0, 1.0), (1, 2, 700, 257, 391, 1.02), (1, 1, 512, 512, 0, 1.01)])
def test_attention_prefill_tensor_cores_moving_maximum(rt, oracle, B, H, T, s, n, grow):
    """Large scores whose maximum keeps rising along the keys (key j scaled by grow^j on top of
    3x inputs): the kernel's reference maximum has to move, and O and the row sums have to be
    rescaled, many times per row."""
    rng = np.random.Generator(np.random.PCG64(7 + s + n))
    d = H * 64
    t = n + s
    ramp = (grow ** np.arange(t, dtype=np.float64)).astype(np.float32)
    ramp = ramp / ramp.max() * 3.0                         # the largest keys are 3x
    kc = np.zeros((B, T, H, 64), np.float32)
    vc = np.zeros_like(kc)
    kc[:, :n] = rng.standard_normal((B, n, H, 64), dtype=np.float32) * ramp[None, :n, None, None]
    vc[:, :n] = rng.standard_normal((B, n, H, 64), dtype=np.float32)
    dk, dv = rt.transfer_from_array(_to_gpu_cache(kc)), rt.transfer_from_array(_to_gpu_cache(vc))
    qkv = rng.standard_normal((B * s, 3 * d), dtype=np.float32)
    qkv[:, :d] *= 3.0
    qkv[:, d:2 * d] = (qkv[:, d:2 * d].reshape(B, s, d) * ramp[None, n:, None]).reshape(B * s, d)
    want = oracle.attention(qkv, kc, vc, B, s, n, H, mode=0)
    got = rt.attention(rt.transfer_from_array(qkv), dk, dv, B, s, n, precision=L.PREC_BF16X3).numpy()
    # scores reach the hundreds here, so the split-bf16 products carry an absolute error of a few 1e-4 in the
    # exponent; the outputs are convex combinations of unit-normal V rows
    np.testing.assert_allclose(got, want, atol=2e-3, rtol=0)


def test_attention_golden_sdpa(rt, golden):
    g = golden["torch_ops"]
    q, k, v = g["sdpa_q"], g["sdpa_k"], g["sdpa_v"]  # [4,4,8,64]
    B, H, T, hd = q.shape
    qkv = np.concatenate([x.transpose(0, 2, 1, 3).reshape(B * T, H * hd) for x in (q, k, v)], axis=1)
    dk, dv = rt.open_buffer((B, H, T, hd)), rt.open_buffer((B, H, T, hd))
    got = rt.attention(rt.transfer_from_array(qkv), dk, dv, B, T, 0).numpy()
    np.testing.assert_allclose(got.reshape(B, T, H, hd).transpose(0, 2, 1, 3), g["sdpa_causal_o"], atol=1e-5, rtol=1e-5)
    got = rt.attention(rt.transfer_from_array(qkv), dk, dv, B, T, 0, precision=L.PREC_BF16X3).numpy()
    np.testing.assert_allclose(got.reshape(B, T, H, hd).transpose(0, 2, 1, 3), g["sdpa_causal_o"], atol=2e-5, rtol=2e-5)


def test_attention_rejects_positions_outside_cache(rt):
    dk, dv = rt.open_buffer((1, 1, 8, 64)), rt.open_buffer((1, 1, 8, 64))
    qkv = rt.open_buffer((4, 192))
    with pytest.raises(B200Error) as e:
        rt.attention(qkv, dk, dv, 1, 4, 6)
    assert e.value.code == L.EINVAL


def test_open_buffer_is_zero_filled_and_roundtrips(rt):
    b = rt.open_buffer((1000,))
    assert not b.numpy().any()
    a = np.arange(1000, dtype=np.float32)
    c = rt.copy_buffer_value(rt.transfer_from_array(a))
    np.testing.assert_array_equal(c.numpy(), a)
    e = rt.open_buffer((0,))
    assert e.numpy().size == 0


def test_work_can_be_queued_on_a_stream_of_the_caller(oracle):
    """caten_b200_set_stream: the context queues its kernels on a stream the host owns (here a torch stream), then
    returns to its own."""
    torch = pytest.importorskip("torch")
    from caten_b200.runtime import B200Runtime
    rng = np.random.Generator(np.random.PCG64(9))
    up, t, raw = make_weight(rng, 384, 256, "q4_0")
    Wf = oracle.dequant(t, raw, 384 * 256).reshape(384, 256)
    x = rng.standard_normal((3, 256), dtype=np.float32)
    ref = oracle.linear(x, Wf, mode=0)
    with B200Runtime(0) as r2:
        own = r2.stream
        w = r2.upload_weight(up)
        dx = r2.transfer_from_array(x)
        host_stream = torch.cuda.Stream()
        L.check(r2.ctx, r2.lib.caten_b200_set_stream(r2.ctx, host_stream.cuda_stream))
        assert r2.stream == host_stream.cuda_stream
        y1 = r2.linear(w, dx).numpy()
        L.check(r2.ctx, r2.lib.caten_b200_set_stream(r2.ctx, None))
        assert r2.stream == own
        y2 = r2.linear(w, dx).numpy()
        w.close()
    np.testing.assert_array_equal(y1.view(np.uint32), y2.view(np.uint32))
    np.testing.assert_allclose(y1, ref, atol=1e-5, rtol=1e-5)


def test_large_copies_through_the_pinned_bounce_buffers(rt, oracle):
    """Copies of 4 MiB and more from pageable host memory are cut into 16 MiB pieces that alternate between two
    pinned buffers: sizes around the piece boundaries, and a packed weight larger than one piece."""
    rng = np.random.Generator(np.random.PCG64(5))
    for n in ((4 << 20) // 4, (16 << 20) // 4 + 3, (40 << 20) // 4 + 1):
        a = rng.integers(0, 2 ** 31, n, dtype=np.int64).astype(np.float32)
        buf = rt.transfer_from_array(a)
        np.testing.assert_array_equal(buf.numpy().view(np.uint32), a.view(np.uint32))
        buf.close()
    p = S._rand_packed(rng, 4100, 4096, "q8_0")      # 17.8 MB of blocks
    w = rt.upload_weight(p)
    want = oracle.dequant(p.ggml_type, p.data, p.rows * p.cols).reshape(p.rows, p.cols)
    np.testing.assert_array_equal(w.dequantize().view(np.uint32), want.view(np.uint32))
    w.close()


def test_gemm_split_k_cluster_reduction_matches_global_reduction(oracle, monkeypatch):
    """CATEN_B200_SPLITK_CLUSTER=1 reduces split-K partial tiles inside a thread-block cluster
    (distributed shared memory) instead of a second kernel: same splits order, same epilogue."""
    from caten_b200.runtime import B200Runtime
    rng = np.random.Generator(np.random.PCG64(77))
    up, t, raw = make_weight(rng, 1600, 1600, "q4_0")
    x = rng.standard_normal((40, 1600), dtype=np.float32)
    bias = rng.standard_normal(1600, dtype=np.float32) * 0.1
    res = rng.standard_normal((40, 1600), dtype=np.float32) * 0.1
    outs = []
    for flag in ("0", "1"):
        monkeypatch.setenv("CATEN_B200_SPLITK_CLUSTER", flag)
        with B200Runtime(0) as r2:
            w = r2.upload_weight(up)
            y = r2.linear(w, r2.transfer_from_array(x), r2.transfer_from_array(bias), r2.transfer_from_array(res), L.ACT_GELU,
                          L.PREC_BF16X3).numpy()
            r2.sync()
            outs.append(y)
            w.close()
    Wf = oracle.dequant(t, raw, 1600 * 1600).reshape(1600, 1600)
    oracle.set_threads(8)
    ref = oracle.linear(x, Wf, bias, res, 1, mode=0)
    oracle.set_threads(1)
    for y in outs:
        assert np.abs(y - ref).max() <= 1e-4 * max(1.0, np.abs(ref).max())
    assert np.abs(outs[0] - outs[1]).max() <= 1e-5


@pytest.mark.parametrize("prec", [L.PREC_FP32, L.PREC_BF16X3])
def test_attention_block_golden(rt, golden, prec):
    """The attention block of source/test-suite/test-llm.lisp:257-301 (c_attn -> heads -> softmax
    attention -> c_proj vs `attn_impl_torch`, atol 1e-4 / rtol 1e-4) at head dim 64 with the causal
    mask of external/llm/layers.lisp:86, through the three C-ABI calls the block lowers to."""
    g = golden["attn_block"]
    x, H = g["hd64_x"], int(g["hd64_heads"])
    B, T, d = x.shape
    wa, wp = rt.upload_weight(g["hd64_wa"]), rt.upload_weight(g["hd64_wp"])
    ba, bp = rt.transfer_from_array(g["hd64_ba"]), rt.transfer_from_array(g["hd64_bp"])
    qkv = rt.linear(wa, rt.transfer_from_array(x.reshape(B * T, d)), ba, precision=prec)
    dk, dv = rt.open_buffer((B, H, T, 64)), rt.open_buffer((B, H, T, 64))
    o = rt.attention(qkv, dk, dv, B, T, 0, precision=prec)
    y = rt.linear(wp, o, bp, precision=prec).numpy()
    np.testing.assert_allclose(y.reshape(B, T, d), g["hd64_y"], atol=1e-4, rtol=1e-4)
    wa.close(); wp.close()


def test_kv_cache_protocol(rt):
    """source/test-suite/test-dynamic-shape.lisp:189-222: a prompt of 10 rows at start_pos 0, then one
    row per call; after every call cache rows [0, start_pos + seq_len) are exactly the rows fed so
    far, in order, and the rest of the cache is still zero."""
    rng = np.random.Generator(np.random.PCG64(4))
    B, T, H = 1, 128, 4
    d = H * 64
    dk, dv = rt.open_buffer((B, H, T, 64)), rt.open_buffer((B, H, T, 64))
    fed_k, fed_v, start = [], [], 0
    for nth in range(10):
        s = 10 if nth == 0 else 1
        qkv = rng.random((B * s, 3 * d), dtype=np.float32)
        rt.attention(rt.transfer_from_array(qkv), dk, dv, B, s, start).close()
        fed_k.append(qkv[:, d:2 * d]); fed_v.append(qkv[:, 2 * d:])
        start += s
        k, v = dk.numpy(), dv.numpy()   # [B, H, T, 64]
        np.testing.assert_array_equal(k[0, :, :start].transpose(1, 0, 2).reshape(start, d), np.concatenate(fed_k))
        np.testing.assert_array_equal(v[0, :, :start].transpose(1, 0, 2).reshape(start, d), np.concatenate(fed_v))
        assert not k[0, :, start:].any() and not v[0, :, start:].any()


@pytest.mark.parametrize("rows,d", [(30, 40), (9, 1600), (3, 4096)])
def test_rmsnorm(rt, oracle, golden, rows, d):
    """`!rms-norm` (source/nn/normalization.lisp:70-85): the oracle within 1e-5, the torchtune function of
    source/test-suite/test-normalization.lisp:57-63 at its tolerance, with and without a weight."""
    g = golden["llama_ops"]
    rng = np.random.Generator(np.random.PCG64(rows + d))
    x = g["rms_ref_x"] if (rows, d) == (30, 40) else g["rms_wide_x"] if (rows, d) == (9, 1600) else rng.standard_normal((rows, d), dtype=np.float32) * 2
    w = (rng.random(d, dtype=np.float32) + 0.5)
    dx = rt.transfer_from_array(x)
    got = rt.rmsnorm(dx).numpy()
    np.testing.assert_allclose(got, oracle.rmsnorm(x), atol=1e-5, rtol=1e-5)
    acc_check(got, oracle.rmsnorm(x), oracle.rmsnorm(x, mode=2))
    if (rows, d) == (30, 40):
        np.testing.assert_allclose(got, g["rms_ref_y"], atol=1e-3, rtol=1e-6)
    np.testing.assert_allclose(rt.rmsnorm(dx, rt.transfer_from_array(w)).numpy(), oracle.rmsnorm(x, w), atol=1e-5, rtol=1e-5)
    with pytest.raises(B200Error):
        rt.rmsnorm(rt.open_buffer((2, 10)))    # d % 4 != 0


@pytest.mark.parametrize("tag", ["ref", "hd64"])
def test_rope(rt, oracle, golden, tag):
    """`!rope` (source/nn/positional-encoding.lisp:3-56): bit-exact against the oracle (the same fp32 formula,
    transcendentals through double), the torchtune function of source/test-suite/test-rope.lisp:60-66 at its
    tolerance, and a continued sequence (pos0 > 0) equal to the tail of the full one."""
    g = golden["llama_ops"]
    x = g[f"rope_{tag}_x"]
    got = rt.rope(rt.transfer_from_array(x)).numpy()
    np.testing.assert_allclose(got, oracle.rope(x), atol=1e-6, rtol=1e-6)
    np.testing.assert_allclose(got, g[f"rope_{tag}_y"], atol=1e-5, rtol=5e-4)
    tail = rt.rope(rt.transfer_from_array(x[:, 4:]), pos0=4).numpy()
    np.testing.assert_array_equal(tail, got[:, 4:])
    odd = np.random.Generator(np.random.PCG64(1)).random((2, 5, 3, 7), dtype=np.float32)
    np.testing.assert_allclose(rt.rope(rt.transfer_from_array(odd)).numpy(), oracle.rope(odd), atol=1e-6, rtol=1e-6)
