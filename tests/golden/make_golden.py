"""Generates the golden fixtures in this directory.  Run from the repo root:

    python tests/golden/make_golden.py

The reference (hikettei/Caten) is Common Lisp and cannot be executed where this repository is
developed, so the fixtures come from the libraries the reference's own test-suite uses as ITS
oracle (source/test-suite/package.lisp:15-29 imports them through py4cl):

* ``gguf`` (Python): the 64-element ``arange`` tensor that external/test-gguf.lisp:8-32 writes
  as f32 / f16 / q8_0 and reads back with ``gguf.quants.dequantize``; Q4_0 blocks (which the
  reference cannot load, external/gguf/tensor-info.lisp:41) dequantised by the same package.
* PyTorch: matmul, softmax, scaled-dot-product attention, LayerNorm and tanh-GeLU on seeded
  inputs, the comparisons of test-gemm.lisp:3-22, test-llm.lisp:6-102, test-normalization.lisp:48-55
  and test-activations.lisp:176-184; and a float64 GPT-2 forward (prefill + cached decode) of a
  tiny random model, which pins the oracle's whole-model wiring; and the attention block of
  test-llm.lisp:257-301 (`attn_impl_torch`: c_attn, split into heads, softmax attention, c_proj)
  at the reference test's own shape (10 x 3 x 32, 4 heads, no mask) and at head dim 64 with the
  causal mask the Transformer passes (external/llm/layers.lisp:86), the shape the CUDA kernels cover.

Neither PyTorch nor gguf is needed to *use* the fixtures.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from caten_b200 import synthetic as S  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def gguf_fixtures():
    from gguf import GGMLQuantizationType as GT
    from gguf.quants import dequantize, quantize

    data = np.arange(64, dtype=np.float32)
    q8 = quantize(data, GT.Q8_0)
    out = {
        "arange_f32_raw": data.view(np.uint8), "arange_f32": data,
        "arange_f16_raw": data.astype(np.float16).view(np.uint8), "arange_f16": data.astype(np.float16).astype(np.float32),
        "arange_q8_0_raw": np.ascontiguousarray(q8).view(np.uint8).reshape(-1), "arange_q8_0": dequantize(q8, GT.Q8_0).reshape(-1),
    }
    rng = np.random.Generator(np.random.PCG64(7))
    for name, gt, bb in (("q4_0", GT.Q4_0, 18), ("q8_0", GT.Q8_0, 34)):
        p = S._rand_packed(rng, 6, 96, name)
        out[f"rand_{name}_raw"] = p.data
        out[f"rand_{name}"] = dequantize(p.data.reshape(-1, bb), gt).reshape(6, 96)
    # every fp16 scale class: subnormal, normal, negative, zero
    scales = np.array([0.0, 6e-8, 3e-5, 1.0, -2.5, 65504.0], dtype=np.float16)
    codes = rng.integers(0, 16, size=(6, 32), dtype=np.uint8)
    raw = S.pack_q4_0(codes, scales)
    out["edge_q4_0_raw"] = raw
    out["edge_q4_0"] = dequantize(raw.reshape(-1, 18), GT.Q4_0).reshape(6, 32)
    np.savez_compressed(os.path.join(OUT, "gguf_dequant.npz"), **out)


def gguf_nibble_formats():
    """Q4_1, Q5_0 and Q5_1 blocks (formats the reference lists, external/gguf/tensor-info.lisp:3-34,
    without implementing them) dequantised by the Python `gguf` package: random blocks, and blocks
    whose scale / minimum run through the fp16 classes (zero, subnormal, normal, negative, largest)."""
    from gguf import GGMLQuantizationType as GT
    from gguf.quants import dequantize

    rng = np.random.Generator(np.random.PCG64(11))
    out = {}
    for name, gt in (("q4_1", GT.Q4_1), ("q5_0", GT.Q5_0), ("q5_1", GT.Q5_1)):
        bb = S.BLOCK_BYTES[S.TYPE_IDS[name]]
        p = S._rand_packed(rng, 6, 96, name)
        out[f"rand_{name}_raw"] = p.data
        out[f"rand_{name}"] = dequantize(p.data.reshape(-1, bb), gt).astype(np.float32).reshape(6, 96)
        raw = rng.integers(0, 256, size=(6, bb), dtype=np.uint8)
        raw[:, 0:2] = np.array([0.0, 6e-8, 3e-5, 1.0, -2.5, 2047.0], dtype="<f2").reshape(6, 1).view(np.uint8)
        if name != "q5_0":
            raw[:, 2:4] = np.array([1.5, -6e-8, 0.0, -3e-5, 65504.0, -100.0], dtype="<f2").reshape(6, 1).view(np.uint8)
        out[f"edge_{name}_raw"] = raw.reshape(-1)
        out[f"edge_{name}"] = dequantize(raw, gt).astype(np.float32).reshape(6, 32)
    np.savez_compressed(os.path.join(OUT, "gguf_dequant_nibble.npz"), **out)


def torch_ops():
    g = torch.Generator().manual_seed(11)
    out = {}
    a, b = torch.randn(37, 64, generator=g), torch.randn(64, 29, generator=g)
    out["mm_a"], out["mm_b"], out["mm_c"] = a.numpy(), b.numpy(), (a @ b).numpy()
    out["relu_mm_c"] = torch.relu(a @ b).numpy()
    x = torch.randn(128, 128, generator=g)
    out["softmax_x"], out["softmax_y"] = x.numpy(), torch.softmax(x, -1).numpy()
    q, k, v = (torch.rand(4, 4, 8, 64, generator=g) for _ in range(3))
    sc = (q @ k.transpose(-1, -2)) * (1.0 / np.sqrt(64.0))
    out["sdpa_q"], out["sdpa_k"], out["sdpa_v"] = q.numpy(), k.numpy(), v.numpy()
    out["sdpa_o"] = (torch.softmax(sc, -1) @ v).numpy()
    mask = torch.full((8, 8), float("-inf")).triu(1)
    out["sdpa_causal_o"] = (torch.softmax(sc + mask, -1) @ v).numpy()
    x = torch.randn(30, 768, generator=g) * 3 + 1
    gm, bt = torch.randn(768, generator=g), torch.randn(768, generator=g)
    out["ln_x"], out["ln_g"], out["ln_b"] = x.numpy(), gm.numpy(), bt.numpy()
    out["ln_y"] = torch.nn.functional.layer_norm(x, (768,), gm, bt, 1e-5).numpy()
    x = torch.randn(4096, generator=g) * 4
    out["gelu_x"], out["gelu_y"] = x.numpy(), torch.nn.functional.gelu(x, approximate="tanh").numpy()
    np.savez_compressed(os.path.join(OUT, "torch_ops.npz"), **out)


def attn_block():
    """`attn_impl_torch` of source/test-suite/test-llm.lisp:273-287, restated: the projection to
    q, k, v, per-head softmax(q.k^T / sqrt(hd)) . v with the softmax composed as in the file's
    `softmax` helper (:9-13), heads merged, output projection."""
    def softmax(x):
        m = x - x.max(-1, keepdims=True)[0]
        e = m.exp()
        return e / e.sum(axis=-1, keepdims=True)

    def block(x, n_heads, wa, ba, wp, bp, causal):
        xqkv = torch.matmul(x, wa.T) + ba
        B, T, _ = x.size()
        shp = (B, T, n_heads, x.size(-1) // n_heads)
        q, k, v = (z.reshape(shp).transpose(1, 2) for z in xqkv.chunk(3, dim=2))
        qk = torch.matmul(q, k.transpose(-2, -1)) * (1 / np.sqrt(q.size(-1)))
        if causal:
            qk = qk + torch.full((T, T), float("-inf")).triu(1)
        o = torch.matmul(softmax(qk), v).permute(0, 2, 1, 3).reshape(B, T, -1)
        return torch.matmul(o, wp.T) + bp

    g = torch.Generator().manual_seed(23)
    out = {}
    for tag, (B, T, d, H, causal) in (("ref", (10, 3, 32, 4, False)), ("hd64", (3, 7, 128, 2, True))):
        x = torch.rand(B, T, d, generator=g)
        wa, ba = torch.rand(3 * d, d, generator=g) * (2.0 / d), torch.rand(3 * d, generator=g)
        wp, bp = torch.rand(d, d, generator=g) * (2.0 / d), torch.rand(d, generator=g)
        if tag == "ref":   # the reference test draws everything from rand() in [0, 1)
            wa, wp = wa * (d / 2.0), wp * (d / 2.0)
        out.update({f"{tag}_x": x.numpy(), f"{tag}_wa": wa.numpy(), f"{tag}_ba": ba.numpy(), f"{tag}_wp": wp.numpy(),
                    f"{tag}_bp": bp.numpy(), f"{tag}_heads": np.int64(H), f"{tag}_y": block(x, H, wa, ba, wp, bp, causal).numpy()})
    np.savez_compressed(os.path.join(OUT, "attn_block.npz"), **out)


def llama_ops():
    """RMSNorm and RoPE against the functions the reference's tests import from torchtune's documentation
    (source/test-suite/test-normalization.lisp:8-15, test-rope.lisp:38-56), restated; shapes of those tests
    (30 x 40; 1 x 10 x 10 x 10) plus head dim 64 rows."""
    def rms(x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5)

    def rope(x, base=10000):
        dim = x.shape[-1]
        theta = 1.0 / (base ** (torch.arange(0, dim, 2).float() / dim))
        idx_theta = torch.einsum("i,j->ij", torch.arange(x.size(1), dtype=theta.dtype), theta)
        cache = torch.stack([torch.cos(idx_theta), torch.sin(idx_theta)], dim=-1)
        xs = x.float().reshape(*x.shape[:-1], -1, 2)
        rc = cache.view(1, x.size(1), 1, xs.size(-2), 2)
        out = torch.stack([xs[..., 0] * rc[..., 0] - xs[..., 1] * rc[..., 1], xs[..., 1] * rc[..., 0] + xs[..., 0] * rc[..., 1]], dim=-1)
        return out.flatten(-2)

    g = torch.Generator().manual_seed(29)
    out = {}
    for tag, shape in (("ref", (30, 40)), ("wide", (9, 1600))):
        x = torch.rand(*shape, generator=g)
        out[f"rms_{tag}_x"], out[f"rms_{tag}_y"] = x.numpy(), rms(x).numpy()
    for tag, shape in (("ref", (1, 10, 10, 10)), ("hd64", (2, 33, 3, 64))):
        x = torch.rand(*shape, generator=g)
        out[f"rope_{tag}_x"], out[f"rope_{tag}_y"] = x.numpy(), rope(x).numpy()
    np.savez_compressed(os.path.join(OUT, "llama_ops.npz"), **out)


def torch_gpt2_f64(sd, tokens, p, n_new):
    """float64 GPT-2 (tanh GeLU, eps 1e-5, causal mask) recomputed from scratch for every new
    token: no KV cache, so it also checks the oracle's cache protocol."""
    d, H = p.dim, p.n_heads
    tt = {k: torch.tensor(v, dtype=torch.float64) for k, v in sd.items()}

    def fwd(ids):
        B, T = ids.shape
        h = tt["wte.weight"][ids] + tt["wpe.weight"][torch.arange(T)]
        mask = torch.full((T, T), float("-inf"), dtype=torch.float64).triu(1)
        for l in range(p.n_layers):
            pre = f"h.{l}."
            x = torch.nn.functional.layer_norm(h, (d,), tt[pre + "ln_1.affine"], tt[pre + "ln_1.bias"], 1e-5)
            qkv = x @ tt[pre + "attn.c_attn.weight"].T + tt[pre + "attn.c_attn.bias"]
            q, k, v = (z.view(B, T, H, -1).transpose(1, 2) for z in qkv.split(d, -1))
            a = torch.softmax(q @ k.transpose(-1, -2) / np.sqrt(d // H) + mask, -1) @ v
            h = h + a.transpose(1, 2).reshape(B, T, d) @ tt[pre + "attn.c_proj.weight"].T + tt[pre + "attn.c_proj.bias"]
            x = torch.nn.functional.layer_norm(h, (d,), tt[pre + "ln_2.affine"], tt[pre + "ln_2.bias"], 1e-5)
            f = torch.nn.functional.gelu(x @ tt[pre + "mlp.c_fc.weight"].T + tt[pre + "mlp.c_fc.bias"], approximate="tanh")
            h = h + f @ tt[pre + "mlp.c_proj.weight"].T + tt[pre + "mlp.c_proj.bias"]
        x = torch.nn.functional.layer_norm(h, (d,), tt["ln_f.affine"], tt["ln_f.bias"], 1e-5)
        return x[:, -1] @ tt["lm_head.weight"].T

    ids = torch.tensor(tokens)
    logits, new = [], []
    for _ in range(n_new):
        lg = fwd(ids)
        nxt = lg.argmax(-1)
        logits.append(lg.numpy())
        new.append(nxt.numpy())
        ids = torch.cat([ids, nxt[:, None]], 1)
    return np.stack(logits), np.stack(new, 1)


def gpt2_tiny():
    p = S.GPT2Params(n_layers=2, n_heads=2, dim=128, vocab_size=1003)
    sd = S.synth_state_dict(p, "f32", seed=3, max_seq_len=48, trivial_affine=False, weight_std=0.08)
    toks = S.synth_prompts(3, 9, p.vocab_size, seed=5)
    logits, new = torch_gpt2_f64(sd, toks, p, 6)
    np.savez_compressed(os.path.join(OUT, "gpt2_tiny_f64.npz"), prompt=toks, logits=logits.astype(np.float64), new_ids=new,
                        seed=3, weight_std=0.08, max_seq_len=48)


if __name__ == "__main__":
    only = sys.argv[1:]
    for fn in (gguf_fixtures, gguf_nibble_formats, torch_ops, gpt2_tiny, attn_block, llama_ops):
        if not only or fn.__name__ in only:
            fn()
    print("wrote", sorted(f for f in os.listdir(OUT) if f.endswith(".npz")))
