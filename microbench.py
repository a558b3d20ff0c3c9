"""Single-kernel timings through the C ABI (CUDA events on the library's stream).

    python microbench.py attn_decode --batch 64 --heads 25 --context 700
    python microbench.py attn_prefill --batch 16 --heads 25 --tokens 512 --precision bf16x3
    python microbench.py gemv --model gpt2-xl --wtype q4_0
    python microbench.py gemm --rows 256 --n 1600 --k 6400 --wtype q4_0 --precision bf16x3
    python microbench.py relu_matmul --precision bf16x3
    python microbench.py expr --elements 67108864
    python microbench.py decode_step --model gpt2-xl --wtype q4_0 --context 640 [--batch 1]
    python microbench.py layernorm --rows 8192 --n 1600
    python microbench.py gguf_load --model gpt2-xl --wtype q4_0
    python microbench.py sample --batch 256

Each prints one JSON line.  Operands are rotated over several copies larger in total than the
126 MB L2, so every launch streams from HBM.  Events bracket each launch (the profile API of the
library), so host launch pace does not enter; for kernels of a few microseconds the figure still
includes launch latency and an `ncu --metrics gpu__time_duration.sum` list is the better source.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from caten_b200 import _lib as L  # noqa: E402
from caten_b200 import synthetic as S  # noqa: E402
from caten_b200.runtime import B200Runtime  # noqa: E402


def _peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            j = json.load(f)
            return float(j["hbm_gbs"]), float(j["bf16_tflops"])
    except Exception:
        return 6650.0, 1590.0


def attn_decode(rt, a):
    B, H, T, n = a.batch, a.heads, a.context + 8, a.context
    d = H * 64
    copies = max(2, int(np.ceil(300e6 / (B * H * T * 64 * 4 * 2))))
    kv = [(rt.open_buffer((B, H, T, 64)), rt.open_buffer((B, H, T, 64))) for _ in range(copies)]
    rng = np.random.Generator(np.random.PCG64(0))
    qkv = rt.transfer_from_array(rng.standard_normal((B, 3 * d), dtype=np.float32))
    for i in range(a.warmup):
        rt.attention(qkv, *kv[i % copies], B, 1, n).close()
    rt.profile_begin(["attn_decode"])
    for i in range(a.iters):
        rt.attention(qkv, *kv[i % copies], B, 1, n).close()
    ms, calls = rt.profile_end()["attn_decode"]
    nbytes = B * 2 * (n + 1) * d * 4.0
    hbm, _ = _peak()
    return {"kernel": "attn_decode_kernel", "batch": B, "heads": H, "context": n + 1, "us": 1e3 * ms / calls,
            "algorithmic_bytes": nbytes, "GB/s": nbytes / (ms / calls / 1e3) / 1e9, "frac_of_measured_hbm": nbytes / (ms / calls / 1e3) / 1e9 / hbm}


def attn_prefill(rt, a):
    """One prefill step of `tokens` tokens after `context` cached ones; the figure of merit is the
    causal q.K^T + P.V work (4 * 64 flops per visible query-key pair) per second."""
    B, H, s, n = a.batch, a.heads, a.tokens, a.context
    T, d = n + s, H * 64
    prec = {"fp32": L.PREC_FP32, "bf16": L.PREC_BF16, "bf16x3": L.PREC_BF16X3}[a.precision]
    rng = np.random.Generator(np.random.PCG64(0))
    dk, dv = rt.open_buffer((B, H, T, 64)), rt.open_buffer((B, H, T, 64))
    qkv = rt.transfer_from_array(rng.standard_normal((B * s, 3 * d), dtype=np.float32))
    for i in range(a.warmup):
        rt.attention(qkv, dk, dv, B, s, n, precision=prec).close()
    rt.profile_begin(["attn_prefill"])
    for i in range(a.iters):
        rt.attention(qkv, dk, dv, B, s, n, precision=prec).close()
    ms, calls = rt.profile_end()["attn_prefill"]
    pairs = B * H * (s * n + s * (s + 1) / 2)
    flops = 4.0 * 64 * pairs
    return {"kernel": "attn_prefill_kernel" if prec == L.PREC_FP32 else "attn_prefill_tc_kernel", "batch": B, "heads": H,
            "tokens": s, "context": n, "precision": a.precision, "ms": ms / calls, "includes": "the cache append kernel",
            "useful_TFLOP/s": flops / (ms / calls / 1e3) / 1e12, "tokens_per_s": B * s / (ms / calls / 1e3)}


def gemv(rt, a):
    p = S.GPT2_SIZES[a.model]
    d = p.dim
    rng = np.random.Generator(np.random.PCG64(0))
    hbm, _ = _peak()
    out = {}
    for name, rows, cols in (("c_attn", 3 * d, d), ("attn.c_proj", d, d), ("c_fc", 4 * d, d), ("mlp.c_proj", d, 4 * d), ("lm_head", p.vocab_size, d)):
        one = S._rand_packed(rng, rows, cols, a.wtype) if a.wtype != "f32" else rng.standard_normal((rows, cols), dtype=np.float32)
        w0 = rt.upload_weight(one)
        copies = max(2, min(48, int(np.ceil(300e6 / w0.packed_nbytes))))
        ws = [w0] + [rt.upload_weight(one) for _ in range(copies - 1)]
        x = rt.transfer_from_array(rng.standard_normal((1, cols), dtype=np.float32))
        y = rt.open_buffer((1, rows))
        for i in range(copies):
            rt.linear(ws[i], x, out=y)
        rt.profile_begin(["gemv"])
        for i in range(a.iters):
            rt.linear(ws[i % copies], x, out=y)
        ms, calls = rt.profile_end()["gemv"]
        per = ms / calls / 1e3
        out[f"{name} {rows}x{cols}"] = {"us": per * 1e6, "GB/s": w0.packed_nbytes / per / 1e9, "frac_of_measured_hbm": w0.packed_nbytes / per / 1e9 / hbm}
        for w in ws:
            w.close()
    return {"kernel": "gemv", "model": a.model, "wtype": a.wtype, "shapes": out}


def gemm(rt, a):
    rng = np.random.Generator(np.random.PCG64(0))
    one = S._rand_packed(rng, a.n, a.k, a.wtype) if a.wtype != "f32" else rng.standard_normal((a.n, a.k), dtype=np.float32)
    w0 = rt.upload_weight(one)
    copies = max(2, min(48, int(np.ceil(300e6 / w0.packed_nbytes))))
    ws = [w0] + [rt.upload_weight(one) for _ in range(copies - 1)]
    x = rt.transfer_from_array(rng.standard_normal((a.rows, a.k), dtype=np.float32))
    y = rt.open_buffer((a.rows, a.n))
    prec = L.PRECISIONS[a.precision]
    for i in range(min(copies, 4)):
        rt.linear(ws[i], x, None, None, L.ACT_NONE, prec, out=y)
    rt.profile_begin(["gemm"])
    for i in range(a.iters):
        rt.linear(ws[i % copies], x, None, None, L.ACT_NONE, prec, out=y)
    ms, calls = rt.profile_end()["gemm"]
    per = ms / calls / 1e3
    flops = 2.0 * a.rows * a.n * a.k
    _, tf = _peak()
    return {"kernel": "gemm", "rows": a.rows, "n": a.n, "k": a.k, "wtype": a.wtype, "precision": a.precision, "us": per * 1e6,
            "useful_TFLOP/s": flops / per / 1e12, "frac_of_measured_bf16": flops / per / 1e12 / tf,
            "weight_GB/s": w0.packed_nbytes / per / 1e9}


def relu_matmul(rt, a):
    A, B = S.synth_relu_gemm(seed=1)
    da, db = rt.transfer_from_array(A), rt.transfer_from_array(B)
    prec = L.PRECISIONS[a.precision]
    for _ in range(a.warmup):
        rt.relu_matmul(da, db, prec).close()
    rt.profile_begin(["gemm"])
    for _ in range(a.iters):
        rt.relu_matmul(da, db, prec).close()
    ms, calls = rt.profile_end()["gemm"]
    per = ms / calls / 1e3
    flops = 2.0 * 4096 * 768 * 3072
    _, tf = _peak()
    return {"kernel": "relu_matmul 4096x768x3072", "precision": a.precision, "us": per * 1e6, "useful_TFLOP/s": flops / per / 1e12,
            "frac_of_measured_bf16": flops / per / 1e12 / tf}


def expr(rt, a):
    """Generic schedule items (`caten_b200_eval_expr`): algorithmic bytes = operand + output elements x 4."""
    import torch
    from caten_b200 import expr as E
    n = a.elements
    rng = np.random.Generator(np.random.PCG64(0))
    host = rng.standard_normal(n, dtype=np.float32)
    x, y, z = rt.transfer_from_array(host), rt.transfer_from_array(host[::-1].copy()), rt.open_buffer((n,))
    rows = n // 1024
    m2 = rt.open_buffer((rows,))
    x2 = E.View(x, strides=(1024, 1))
    cases = {
        "a*x+b (1 load, 1 store)": (E.load(E.View.of(x)) * 1.5 + 0.25, E.View.of(z), (n,), 0, None, 8.0 * n),
        "x*y+x (2 loads, 1 store)": (E.load(E.View.of(x)) * E.load(E.View.of(y)) + E.load(E.View.of(x)), E.View.of(z), (n,), 0, None, 12.0 * n),
        "relu(x)*y (where)": (E.where(E.load(E.View.of(x)) < 0.0, E.const(0.0), E.load(E.View.of(x))) * E.load(E.View.of(y)), E.View.of(z), (n,), 0, None, 12.0 * n),
        "row sum [n/1024, 1024]": (E.load(x2), E.View(m2, strides=(1, 0)), (rows, 1024), 1, "sum", 4.0 * n),
        "column sum [1024, n/1024] -> [n/1024]": (E.load(E.View(x, strides=(1, rows))), E.View(m2, strides=(1, 0)), (rows, 1024), 1, "sum", 4.0 * n),
    }
    hbm, _ = _peak()
    out = {}
    stream = torch.cuda.ExternalStream(rt.stream, device=f"cuda:{rt.device}")
    for name, (root, ov, shape, nr, op, nbytes) in cases.items():
        prog = E.Program(root)
        for _ in range(a.warmup):
            E.run(rt, prog, ov, shape, nr, op)
        with torch.cuda.stream(stream):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record(stream)
            for _ in range(a.iters):
                E.run(rt, prog, ov, shape, nr, op)
            t1.record(stream)
        rt.sync()
        per = t0.elapsed_time(t1) / a.iters / 1e3
        out[name] = {"us": per * 1e6, "GB/s": nbytes / per / 1e9, "frac_of_measured_hbm": nbytes / per / 1e9 / hbm, "program_words": len(prog.code)}
    return {"kernel": "expr_kernel", "elements": n, "cases": out}


def layernorm(rt, a):
    """LayerNorm over --rows rows of width --n through `caten_b200_layernorm` (fp32 in, fp32 out)."""
    rows, d = a.rows, a.n
    copies = max(2, int(np.ceil(300e6 / (rows * d * 8))))
    rng = np.random.Generator(np.random.PCG64(0))
    xs = [rt.transfer_from_array(rng.standard_normal((rows, d), dtype=np.float32)) for _ in range(copies)]
    ys = [rt.open_buffer((rows, d)) for _ in range(copies)]
    g = rt.transfer_from_array(np.ones(d, np.float32))
    b = rt.transfer_from_array(np.zeros(d, np.float32))

    def once(i):
        L.check(rt.ctx, rt.lib.caten_b200_layernorm(rt.ctx, xs[i % copies].ptr, g.ptr, b.ptr, ys[i % copies].ptr, rows, d, 1e-5))
    for i in range(a.warmup):
        once(i)
    rt.profile_begin(["layernorm"])
    for i in range(a.iters):
        once(i)
    ms, calls = rt.profile_end()["layernorm"]
    nbytes = rows * d * 8.0
    hbm, _ = _peak()
    return {"kernel": "layernorm_kernel", "rows": rows, "d": d, "us": 1e3 * ms / calls, "algorithmic_bytes": nbytes,
            "GB/s": nbytes / (ms / calls / 1e3) / 1e9, "frac_of_measured_hbm": nbytes / (ms / calls / 1e3) / 1e9 / hbm}


def gguf_load(rt, a):
    """File -> device: writes a synthetic GPT-2 GGUF file (--model, --wtype) with the Python `gguf` package, then
    times opening / parsing it in the library (mmap, header, metadata, tensor table) and building the model from
    it (every tensor uploaded straight from the mapping, quantised ones kept packed)."""
    import tempfile
    import time
    from gguf import GGMLQuantizationType as GT, GGUFWriter
    from caten_b200.gguf import REMAP, load_gguf, remap_key
    from caten_b200.gpt2 import make_gpt2_from_gguf

    def file_name(key):   # inverse of the reference's key remapping (apps/gpt2/gpt2.lisp:52-75)
        for before, after in reversed(REMAP):
            key = key.replace(after, before)
        return key
    p = S.GPT2_SIZES[a.model]
    T = 1024
    sd = S.synth_state_dict(p, a.wtype, seed=0, max_seq_len=T)
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "model.gguf")
        w = GGUFWriter(path, "gpt2")
        w.add_uint32("gpt2.block_count", p.n_layers)
        w.add_uint32("gpt2.embedding_length", p.dim)
        w.add_uint32("gpt2.attention.head_count", p.n_heads)
        w.add_uint32("gpt2.context_length", T)
        for k, v in sd.items():
            assert remap_key(file_name(k)) == k
            if isinstance(v, S.Packed):
                w.add_tensor(file_name(k), v.data.reshape(v.rows, v.cols // 32 * S.BLOCK_BYTES[v.ggml_type]), raw_dtype=GT(v.ggml_type))
            else:
                w.add_tensor(file_name(k), v)
        w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()
        size = os.path.getsize(path)
        del sd
        t0 = time.perf_counter()
        g = load_gguf(path)
        t_open = time.perf_counter() - t0
        n_tensors = len(g.tensors)
        g.close()
        best = None
        for _ in range(max(1, min(a.iters, 3))):   # the first pass also pages the file in
            t0 = time.perf_counter()
            m = make_gpt2_from_gguf(path, runtime=rt, batch=1, max_seq_len=64)
            rt.sync()
            dt = time.perf_counter() - t0
            m.close()
            best = dt if best is None else min(best, dt)
    return {"what": "gguf file -> model on the device", "model": a.model, "wtype": a.wtype, "file_bytes": size, "tensors": n_tensors,
            "open_parse_ms": 1e3 * t_open, "load_s": best, "GB/s": size / best / 1e9}


def sample(rt, a):
    """`caten_b200_sample`: temperature / top-k sampling of one id per row of [--batch, 50257] logits."""
    rows, V = a.batch, 50257
    rng = np.random.Generator(np.random.PCG64(0))
    copies = 4
    lg = [rt.transfer_from_array(rng.standard_normal((rows, V), dtype=np.float32) * 3) for _ in range(copies)]
    u = rt.transfer_from_array(rng.random(rows, dtype=np.float32))
    out = {}
    import torch
    for name, (temp, k) in {"temperature": (0.8, 0), "top_k_40": (0.8, 40)}.items():
        for i in range(a.warmup):
            rt.sample(lg[i % copies], u, temp, k).close()
        rt.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st = torch.cuda.ExternalStream(rt.stream)
        e0.record(st)
        for i in range(a.iters):
            rt.sample(lg[i % copies], u, temp, k).close()
        e1.record(st)
        rt.sync()
        us = 1e3 * e0.elapsed_time(e1) / a.iters
        out[name] = {"us": us, "GB/s": rows * V * 4 / (us / 1e6) / 1e9}
    return {"kernel": "sample", "rows": rows, "vocab": V, **out}


def decode_step(rt, a):
    """The single-kernel decode step (1..4 sequences): time per step from the library's per-class events and, when the
    loaded library is the timing build (`python -m caten_b200.build --timing`, CATEN_B200_LIB=...), the time CTA 0 spends
    in every phase of a Transformer block, averaged over the layers of the last step."""
    import ctypes as C
    from caten_b200.gpt2 import GPT2
    p = S.GPT2_SIZES[a.model]
    B = min(a.batch, 4)
    T = a.context + 40
    sd = S.synth_state_dict(p, a.wtype, seed=0, max_seq_len=T)
    m = GPT2(rt, p, sd, max_seq_len=T, batch=B)
    prompt = S.synth_prompts(B, a.context, p.vocab_size, seed=0)
    first = m.forward(prompt, a.context, 0)
    m.decode_device(first, a.context, 4)
    rt.profile_begin(["decode_step"])
    m.decode_device(first, a.context, a.iters if a.iters <= 32 else 32)
    prof = rt.profile_end()
    ms, calls = prof.get("decode_step", (0.0, 0))
    d, Ln, V = p.dim, p.n_layers, p.vocab_size
    bpw = {"f32": 4.0, "q8_0": 34 / 32, "q4_0": 18 / 32}[a.wtype]
    nbytes = (12 * d * d * Ln + V * d) * bpw + 4 * (13 * d * Ln + 2 * d) + B * (2 * d * 4 + Ln * 2 * (a.context + 1) * d * 4 + Ln * 2 * d * 4 + 8)
    hbm, _ = _peak()
    out = {"kernel": "decode_small_kernel", "model": a.model, "wtype": a.wtype, "batch": B, "context": a.context + 1,
           "us_per_step": 1e3 * ms / calls if calls else None, "algorithmic_bytes": nbytes,
           "frac_of_measured_hbm": (nbytes / (ms / calls / 1e3) / 1e9 / hbm) if calls else None}
    lib = L.load()
    if hasattr(lib, "cb_debug_ds_times"):
        names = ["P1 poll h", "P1 ln_1", "P1 c_attn", "P2 attention chunk", "P3 combine", "P4 poll att", "-", "P4 attn.c_proj",
                 "P5 poll h2", "P5 ln_2", "P5 c_fc+gelu", "P6 poll ff", "-", "P6 mlp.c_proj"]
        n = 1 + Ln * len(names) + 3
        buf = (C.c_ulonglong * n)()
        lib.cb_debug_ds_times.argtypes = [C.c_void_p, C.c_int]
        lib.cb_debug_ds_times(buf, n)
        t = np.array(list(buf), dtype=np.float64)
        per = np.diff(t[:1 + Ln * len(names)]).reshape(Ln, len(names)) / 1e3
        out["phase_us_mean_over_layers_cta0"] = {nm: round(float(per[:, i].mean()), 2) for i, nm in enumerate(names) if nm != "-"}
        k = Ln * len(names)
        out["head_us"] = {"poll h": (t[k + 1] - t[k]) / 1e3, "ln_f": (t[k + 2] - t[k + 1]) / 1e3, "lm_head + arg-max candidates": (t[k + 3] - t[k + 2]) / 1e3}
        out["step_us_cta0"] = (t[k + 3] - t[0]) / 1e3
    m.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["attn_decode", "attn_prefill", "gemv", "gemm", "relu_matmul", "expr", "decode_step", "layernorm", "gguf_load", "sample"])
    ap.add_argument("--elements", type=int, default=1 << 26)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--heads", type=int, default=25)
    ap.add_argument("--context", type=int, default=700)
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--model", default="gpt2-xl")
    ap.add_argument("--wtype", default="q4_0", choices=["q4_0", "q8_0", "f32"])
    ap.add_argument("--rows", type=int, default=256)
    ap.add_argument("--n", type=int, default=1600)
    ap.add_argument("--k", type=int, default=6400)
    ap.add_argument("--precision", default="bf16x3", choices=["fp32", "bf16", "bf16x3"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    with B200Runtime(0) as rt:
        print(json.dumps({"attn_decode": attn_decode, "attn_prefill": attn_prefill, "gemv": gemv, "gemm": gemm, "relu_matmul": relu_matmul, "expr": expr,
                          "decode_step": decode_step, "layernorm": layernorm, "gguf_load": gguf_load, "sample": sample}[a.what](rt, a)))


if __name__ == "__main__":
    main()
