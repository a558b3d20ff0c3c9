"""Seeded synthetic GPT-2 state dicts and prompts.

Pre-trained GPT-2 GGUF files (apps/gpt2/gpt2.lisp:50 downloads them) are not available offline,
so every configuration is generated from ``numpy.random.Generator(PCG64(seed))`` with the shapes
and value distributions the benchmark configurations state.  Quantised weights are generated
directly in packed GGUF block form (codes + fp16 scale), so their dequantised values are exact.

State-dict keys are the reference's after `remap-state-dict-keys` (apps/gpt2/gpt2.lisp:52-80).
A quantised entry is a :class:`Packed` (raw GGUF block bytes, ggml type id, logical shape).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q4_1, GGML_Q5_0, GGML_Q5_1, GGML_Q8_0 = 0, 1, 2, 3, 6, 7, 8
BLOCK_BYTES = {GGML_Q4_0: 18, GGML_Q4_1: 20, GGML_Q5_0: 22, GGML_Q5_1: 24, GGML_Q8_0: 34}
TYPE_IDS = {"f32": GGML_F32, "f16": GGML_F16, "q4_0": GGML_Q4_0, "q4_1": GGML_Q4_1, "q5_0": GGML_Q5_0, "q5_1": GGML_Q5_1,
            "q8_0": GGML_Q8_0}


@dataclass(frozen=True)
class GPT2Params:
    """Model sizes of apps/gpt2/gpt2.lisp:36-41 (head dim is 64 for all of them)."""
    n_layers: int
    n_heads: int
    dim: int
    vocab_size: int = 50257
    norm_eps: float = 1e-5


GPT2_SIZES = {
    "gpt2": GPT2Params(12, 12, 768),
    "gpt2-medium": GPT2Params(24, 16, 1024),
    "gpt2-large": GPT2Params(36, 20, 1280),
    "gpt2-xl": GPT2Params(48, 25, 1600),
}


@dataclass
class Packed:
    """A weight matrix [rows, cols] kept as raw GGUF blocks (row-major, cols/32 blocks per row)."""
    ggml_type: int
    rows: int
    cols: int
    data: np.ndarray  # uint8, flat

    @property
    def shape(self):
        return (self.rows, self.cols)


def pack_q8_0(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """codes int8 [..., 32], scales float16 [...] -> uint8 [..., 34] (scale first, then 32 int8)."""
    nb = int(np.prod(scales.shape))
    out = np.empty((nb, 34), np.uint8)
    out[:, 0:2] = np.ascontiguousarray(scales, dtype="<f2").reshape(nb, 1).view(np.uint8)
    out[:, 2:] = np.ascontiguousarray(codes, dtype=np.int8).reshape(nb, 32).view(np.uint8)
    return out.reshape(-1)


def pack_q4_0(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """codes uint8 in [0,15] [..., 32], scales float16 [...] -> uint8 [..., 18].

    Byte j of a block holds element j in its low nibble and element j+16 in its high nibble."""
    nb = int(np.prod(scales.shape))
    c = np.ascontiguousarray(codes, dtype=np.uint8).reshape(nb, 32)
    out = np.empty((nb, 18), np.uint8)
    out[:, 0:2] = np.ascontiguousarray(scales, dtype="<f2").reshape(nb, 1).view(np.uint8)
    out[:, 2:] = (c[:, :16] & 0x0F) | (c[:, 16:] << 4)
    return out.reshape(-1)


def _rand_packed(rng: np.random.Generator, rows: int, cols: int, wtype: str, std: float = 0.02) -> Packed:
    assert cols % 32 == 0
    nb = rows * (cols // 32)
    if wtype == "q8_0":
        # 32 int8 uniform in [-127, 127]; scale = |N(0, 0.02)| / 127
        codes = rng.integers(-127, 128, size=(nb, 32), dtype=np.int8)
        scales = (np.abs(rng.standard_normal(nb, dtype=np.float32)) * np.float32(std / 127)).astype(np.float16)
        return Packed(GGML_Q8_0, rows, cols, pack_q8_0(codes, scales))
    if wtype == "q4_0":
        # 32 4-bit codes uniform in [0, 15] (offset 8); scale = |N(0, 0.02)| / 8.  A uniform byte
        # is two independent uniform nibbles, so the quant bytes are drawn directly.
        out = np.empty((nb, 18), np.uint8)
        out[:, 2:] = rng.integers(0, 256, size=(nb, 16), dtype=np.uint8)
        scales = (np.abs(rng.standard_normal(nb, dtype=np.float32)) * np.float32(std / 8)).astype("<f2")
        out[:, 0:2] = scales.reshape(nb, 1).view(np.uint8)
        return Packed(GGML_Q4_0, rows, cols, out.reshape(-1))
    if wtype in ("q4_1", "q5_0", "q5_1"):
        # uniform code bytes (and fifth bits); scale = |N(0, std)| / half the code range; the _1
        # formats get a minimum that centres the codes: m = -(range / 2) * d + N(0, std / 16)
        t = TYPE_IDS[wtype]
        levels = 16 if wtype == "q4_1" else 32
        out = rng.integers(0, 256, size=(nb, BLOCK_BYTES[t]), dtype=np.uint8)
        d = (np.abs(rng.standard_normal(nb, dtype=np.float32)) * np.float32(std / (levels / 2))).astype("<f2")
        out[:, 0:2] = d.reshape(nb, 1).view(np.uint8)
        if wtype != "q5_0":
            m = (-(levels / 2) * d.astype(np.float32) + rng.standard_normal(nb, dtype=np.float32) * np.float32(std / 16)).astype("<f2")
            out[:, 2:4] = m.reshape(nb, 1).view(np.uint8)
        return Packed(t, rows, cols, out.reshape(-1))
    raise ValueError(wtype)


def synth_state_dict(p: GPT2Params, wtype: str = "f32", seed: int = 0, max_seq_len: int = 1024,
                     trivial_affine: bool = True, weight_std: float = 0.02) -> dict:
    """Draw order (fixed): wte, wpe, then per layer c_attn, attn.c_proj, mlp.c_fc, mlp.c_proj
    (weight, then bias/affine extras when ``trivial_affine`` is False), then lm_head.

    wtype "f32": every matrix ~ N(0, 0.02).  "q8_0"/"q4_0"/"q4_1"/"q5_0"/"q5_1": the five kinds of Linear weight are
    packed blocks; embeddings, LayerNorm parameters and biases stay fp32.
    ``trivial_affine``: biases 0, LayerNorm gamma 1 / beta 0 (the benchmark configurations);
    False draws them at random so tests exercise those terms.  ``weight_std`` scales the fp32
    matrices and the quantisation scales (0.02 in the benchmark configurations; tests use a
    larger value so that sequences and logits differ visibly)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    d, L, V = p.dim, p.n_layers, p.vocab_size

    def normal(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(weight_std))

    def lin(rows, cols):
        return normal(rows, cols) if wtype == "f32" else _rand_packed(rng, rows, cols, wtype, weight_std)

    def vec(n, base):
        if trivial_affine:
            return np.full(n, base, np.float32)
        return (np.float32(base) + rng.standard_normal(n, dtype=np.float32) * np.float32(0.1))

    sd = {"wte.weight": normal(V, d), "wpe.weight": normal(max_seq_len, d)}
    for l in range(L):
        pre = f"h.{l}."
        sd[pre + "ln_1.affine"] = vec(d, 1.0)
        sd[pre + "ln_1.bias"] = vec(d, 0.0)
        sd[pre + "attn.c_attn.weight"] = lin(3 * d, d)
        sd[pre + "attn.c_attn.bias"] = vec(3 * d, 0.0)
        sd[pre + "attn.c_proj.weight"] = lin(d, d)
        sd[pre + "attn.c_proj.bias"] = vec(d, 0.0)
        sd[pre + "ln_2.affine"] = vec(d, 1.0)
        sd[pre + "ln_2.bias"] = vec(d, 0.0)
        sd[pre + "mlp.c_fc.weight"] = lin(4 * d, d)
        sd[pre + "mlp.c_fc.bias"] = vec(4 * d, 0.0)
        sd[pre + "mlp.c_proj.weight"] = lin(d, 4 * d)
        sd[pre + "mlp.c_proj.bias"] = vec(d, 0.0)
    sd["ln_f.affine"] = vec(d, 1.0)
    sd["ln_f.bias"] = vec(d, 0.0)
    sd["lm_head.weight"] = lin(V, d)
    return sd


def synth_prompts(batch: int, length: int, vocab: int, seed: int = 0) -> np.ndarray:
    """[batch, length] int64 token ids uniform in [0, vocab)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.integers(0, vocab, size=(batch, length), dtype=np.int64)


def synth_relu_gemm(seed: int = 1, M: int = 4096, K: int = 768, N: int = 3072):
    """A [M,K], B [K,N] with entries N(0,1)/sqrt(K) (the `!relu(!matmul)` configuration)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    sc = np.float32(1.0 / np.sqrt(K))
    return (rng.standard_normal((M, K), dtype=np.float32) * sc,
            rng.standard_normal((K, N), dtype=np.float32) * sc)
