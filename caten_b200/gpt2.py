"""GPT-2 on the B200 backend: the host-side counterpart of apps/gpt2/gpt2.lisp.

``make_gpt2`` plays the role of `make-gpt2` (gpt2.lisp:82-93: build the Transformer, load the
state dict, compile), ``GPT2.forward`` of ``(forward model (x . tokens) (s . len) (n . start-pos))``
(gpt2.lisp:104) and ``gpt2_generate`` of `gpt2-generate` (gpt2.lisp:97-113) without the tokenizer:
prompts are token ids.  Unlike the reference, whose compiled graph is fixed to batch 1
(gpt2.lisp:93), ``batch`` independent sequences advance together.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _lib as L
from .runtime import B200Buffer, B200Runtime, B200Weight
from .synthetic import GPT2_SIZES, GPT2Params, Packed


class GPT2:
    def __init__(self, runtime: B200Runtime, params: GPT2Params, state_dict: dict, max_seq_len: int = 1024,
                 batch: int = 1, precision: str = "fp32", max_rows: int = 0, device_blobs: Optional[dict] = None):
        """``state_dict``: reference keys -> fp32 arrays, or :class:`Packed` for Linear weights.

        ``device_blobs``: optional ``{key: device pointer}`` of raw GGUF blocks already resident on
        this GPU (e.g. received through an NCCL broadcast); those entries of ``state_dict`` then
        only need ``ggml_type/rows/cols`` and are not read from the host."""
        self.rt, self.params, self.batch, self.max_seq_len = runtime, params, batch, max_seq_len
        self.precision = L.PRECISIONS[precision] if isinstance(precision, str) else int(precision)
        self._bufs, self._weights, self._keep = [], [], []
        self.weights = {}  # state-dict key -> B200Weight
        p, rt = params, runtime
        Lr = p.n_layers

        def shape_of(key):
            a = state_dict[key]
            return (a.rows, a.cols) if hasattr(a, "ggml_type") and getattr(a, "ggml_type", -1) >= 0 else tuple(a.shape)

        # the embedding tables are indexed by the kernels: refuse tables that do not cover what will be read
        if shape_of("wte.weight") != (p.vocab_size, p.dim):
            raise ValueError(f"wte.weight is {shape_of('wte.weight')}, expected {(p.vocab_size, p.dim)}")
        if len(shape_of("wpe.weight")) != 2 or shape_of("wpe.weight")[1] != p.dim or shape_of("wpe.weight")[0] < max_seq_len:
            raise ValueError(f"wpe.weight is {shape_of('wpe.weight')}: need at least max_seq_len={max_seq_len} rows of {p.dim}")

        def f32(key) -> int:
            """fp32 device array.  A tensor stored in a GGUF block format or as F16 (what a quantised
            GPT-2 file holds for its embedding tables) is expanded on the device, which gives the values
            the reference's loader computes (external/gguf/dequantize.lisp:14-53)."""
            a = state_dict[key]
            packed = getattr(a, "ggml_type", -1) >= 0
            if packed or (isinstance(a, np.ndarray) and a.dtype == np.float16 and a.ndim == 2):
                if packed and device_blobs is not None and key in device_blobs:
                    w = rt.upload_weight_device(a.ggml_type, device_blobs[key], a.rows, a.cols)
                else:
                    w = rt.upload_weight(a)
                b = rt.open_buffer((w.rows, w.cols), np.float32)
                L.check(rt.ctx, rt.lib.caten_b200_weight_dequant(rt.ctx, w.handle, b.ptr))
                rt.sync()
                w.close()
            elif device_blobs is not None and key in device_blobs:
                b = rt.open_buffer(a.shape, np.float32)
                L.check(rt.ctx, rt.lib.caten_b200_d2d(rt.ctx, b.ptr, device_blobs[key], b.nbytes))
            else:
                b = rt.transfer_from_array(a, np.float32)
            self._bufs.append(b)
            return b.ptr

        def weight(key) -> int:
            w = state_dict[key]
            if device_blobs is not None and key in device_blobs:
                h = rt.upload_weight_device(w.ggml_type, device_blobs[key], w.rows, w.cols)
            else:
                h = rt.upload_weight(w)
            self._weights.append(h)
            self.weights[key] = h
            return h.handle

        def parr(vals):
            arr = (C.c_void_p * Lr)(*vals)
            self._keep.append(arr)
            return C.cast(arr, C.POINTER(C.c_void_p))

        d = L.GPT2Desc()
        d.n_layers, d.d_model, d.n_heads, d.vocab = p.n_layers, p.dim, p.n_heads, p.vocab_size
        d.max_seq_len, d.batch, d.eps, d.precision, d.max_rows = max_seq_len, batch, p.norm_eps, self.precision, max_rows
        d.wte, d.wpe = f32("wte.weight"), f32("wpe.weight")
        d.lnf_g, d.lnf_b = f32("ln_f.affine"), f32("ln_f.bias")
        d.lm_head = weight("lm_head.weight")
        d.ln1_g = parr([f32(f"h.{l}.ln_1.affine") for l in range(Lr)])
        d.ln1_b = parr([f32(f"h.{l}.ln_1.bias") for l in range(Lr)])
        d.ln2_g = parr([f32(f"h.{l}.ln_2.affine") for l in range(Lr)])
        d.ln2_b = parr([f32(f"h.{l}.ln_2.bias") for l in range(Lr)])
        d.attn_b = parr([f32(f"h.{l}.attn.c_attn.bias") for l in range(Lr)])
        d.proj_b = parr([f32(f"h.{l}.attn.c_proj.bias") for l in range(Lr)])
        d.fc_b = parr([f32(f"h.{l}.mlp.c_fc.bias") for l in range(Lr)])
        d.mproj_b = parr([f32(f"h.{l}.mlp.c_proj.bias") for l in range(Lr)])
        d.attn_w = parr([weight(f"h.{l}.attn.c_attn.weight") for l in range(Lr)])
        d.proj_w = parr([weight(f"h.{l}.attn.c_proj.weight") for l in range(Lr)])
        d.fc_w = parr([weight(f"h.{l}.mlp.c_fc.weight") for l in range(Lr)])
        d.mproj_w = parr([weight(f"h.{l}.mlp.c_proj.weight") for l in range(Lr)])
        self.linear_weight_bytes = sum(w.packed_nbytes for w in self._weights)
        self._desc = d
        h = C.c_void_p()
        L.check(rt.ctx, rt.lib.caten_b200_gpt2_create(rt.ctx, C.byref(d), C.byref(h)))
        self._h = h
        self._dev_ids = rt.open_buffer((2, batch), np.int64)  # ping-pong ids for device-resident decode

    # -- one step from host ids: the call the reference's token loop makes --
    def forward(self, x, s: Optional[int] = None, n: int = 0) -> np.ndarray:
        """x: [batch, s] token ids (any numeric dtype; sent as float32 like gpt2.lisp:95).
        Returns int64 [batch]: argmax of the logits at the last position."""
        tok = np.ascontiguousarray(x, dtype=np.float32).reshape(self.batch, -1)
        s = tok.shape[1] if s is None else int(s)
        if s != tok.shape[1]:
            raise ValueError("forward: s does not match x")
        out = np.empty(self.batch, np.int64)
        L.check(self.rt.ctx, self.rt.lib.caten_b200_gpt2_step(self._h, tok.ctypes.data, s, int(n), out.ctypes.data))
        return out

    # -- device-resident variants (ids never leave HBM) --
    def forward_device(self, ids: B200Buffer, s: int, n: int, out: B200Buffer) -> None:
        f32 = ids.ptr if ids.dtype == np.float32 else None
        i64 = ids.ptr if ids.dtype == np.int64 else None
        L.check(self.rt.ctx, self.rt.lib.caten_b200_gpt2_step_device(self._h, f32, i64, int(s), int(n), out.ptr))

    def decode_device(self, first_ids: np.ndarray, start_pos: int, steps: int) -> np.ndarray:
        """Greedy decode ``steps`` tokens with ids and position staying on the GPU (one C call; the
        step is replayed from a CUDA graph); returns [batch, steps]."""
        ids0 = self.rt.transfer_from_array(np.ascontiguousarray(first_ids, dtype=np.int64).reshape(self.batch))
        hist = self.rt.open_buffer((steps, self.batch), np.int64)
        self.decode_device_buffers(ids0, start_pos, steps, hist)
        out = hist.numpy().T.copy()
        hist.close()
        ids0.close()
        return out

    def decode_device_buffers(self, first_ids: B200Buffer, start_pos: int, steps: int, out: Optional[B200Buffer] = None) -> None:
        """Asynchronous form of :meth:`decode_device` on device buffers (``out``: [steps, batch] int64)."""
        L.check(self.rt.ctx, self.rt.lib.caten_b200_gpt2_decode(self._h, first_ids.ptr, int(start_pos), int(steps),
                                                                out.ptr if out is not None else None))

    def logits(self) -> np.ndarray:
        """[batch, vocab] fp32 logits of the last step."""
        ptr = self.rt.lib.caten_b200_gpt2_logits(self._h)
        return B200Buffer(self.rt, ptr, (self.batch, self.params.vocab_size), np.float32, owned=False).numpy()

    def sample(self, uniform, temperature: float = 1.0, top_k: int = 0) -> np.ndarray:
        """[batch] int64 ids drawn from the last step's logits (they stay on the device)."""
        ptr = self.rt.lib.caten_b200_gpt2_logits(self._h)
        lg = B200Buffer(self.rt, ptr, (self.batch, self.params.vocab_size), np.float32, owned=False)
        ids = self.rt.sample(lg, uniform, temperature, top_k)
        out = ids.numpy()
        ids.close()
        return out

    def kv_cache(self, layer: int):
        """(k, v) of one layer as numpy arrays [batch, heads, max_seq_len, 64]."""
        k, v = C.c_void_p(), C.c_void_p()
        L.check(self.rt.ctx, self.rt.lib.caten_b200_gpt2_kv(self._h, layer, C.byref(k), C.byref(v)))
        shp = (self.batch, self.params.n_heads, self.max_seq_len, 64)
        return (B200Buffer(self.rt, k.value, shp, np.float32, owned=False).numpy(),
                B200Buffer(self.rt, v.value, shp, np.float32, owned=False).numpy())

    @property
    def launch_count(self) -> int:
        return int(self.rt.lib.caten_b200_gpt2_launch_count(self._h))

    def close(self):
        if getattr(self, "_h", None):
            if self.rt.ctx is None:   # the runtime (and with it the stream the model uses) is already gone
                self._h = None
                return
            self.rt.lib.caten_b200_gpt2_destroy(self._h)
            self._h = None
            for w in self._weights:
                w.close()
            for b in self._bufs:
                b.close()
            self._dev_ids.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def make_gpt2(model_type, state_dict: dict, runtime: Optional[B200Runtime] = None, max_seq_len: int = 1024,
              batch: int = 1, precision: str = "fp32", **kw) -> GPT2:
    """`make-gpt2` (apps/gpt2/gpt2.lisp:82-93). ``model_type``: "gpt2", "gpt2-medium", "gpt2-large",
    "gpt2-xl" or a :class:`GPT2Params`."""
    params = model_type if isinstance(model_type, GPT2Params) else GPT2_SIZES[str(model_type).lstrip(":")]
    rt = runtime or B200Runtime(0)
    return GPT2(rt, params, state_dict, max_seq_len=max_seq_len, batch=batch, precision=precision, **kw)


def gpt2_generate(gpt2: GPT2, prompt_ids, max_length: int = 100, temperature: float = 0.0, top_k: int = 0, seed: int = 0) -> np.ndarray:
    """`gpt2-generate` (apps/gpt2/gpt2.lisp:97-113) on token ids: the first call feeds the whole
    prompt at start position 0, each later call one token; every call's argmax is appended.
    Returns [batch, prompt_len + max_length] int64.  With ``temperature`` > 0 the next id is drawn
    on the device from the step's logits instead (temperature / top-k sampling, seeded; beyond the
    reference, whose loop is greedy)."""
    tokens = np.ascontiguousarray(prompt_ids, dtype=np.int64).reshape(gpt2.batch, -1)
    start_pos = 0
    rng = np.random.Generator(np.random.PCG64(seed))
    for _ in range(max_length):
        in_tokens = tokens[:, start_pos:]
        out = gpt2.forward(in_tokens, in_tokens.shape[1], start_pos)
        if temperature > 0.0:
            out = gpt2.sample(rng.random(gpt2.batch, dtype=np.float32), temperature, top_k)
        start_pos = tokens.shape[1]
        tokens = np.concatenate([tokens, out.reshape(-1, 1)], axis=1)
    return tokens


def make_gpt2_from_gguf(path: str, runtime: Optional[B200Runtime] = None, max_seq_len: Optional[int] = None, batch: int = 1,
                        precision: str = "fp32", **kw) -> GPT2:
    """`make-gpt2` (apps/gpt2/gpt2.lisp:82-93) from a local GGUF file: parse, remap the tensor names,
    upload (quantised tensors stay packed) and build the model.  Sizes come from the file's
    metadata (`gpt2.block_count`, `gpt2.embedding_length`, `gpt2.attention.head_count`, ...) where the
    reference hard-codes them per model name (gpt2.lisp:38-41)."""
    from .gguf import gguf_to_state_dict, load_gguf
    g = load_gguf(path)
    try:
        sd = gguf_to_state_dict(g)
        md = g.metadata
        wte, wpe = sd["wte.weight"], sd["wpe.weight"]
        vocab, dim = (wte.rows, wte.cols) if isinstance(wte, Packed) else wte.shape
        wpe_rows = wpe.rows if isinstance(wpe, Packed) else wpe.shape[0]
        n_layers = int(md.get("gpt2.block_count", 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("h."))))
        n_heads = int(md.get("gpt2.attention.head_count", dim // 64))
        eps = float(md.get("gpt2.attention.layer_norm_epsilon", 1e-5))
        T = int(max_seq_len) if max_seq_len else min(int(md.get("gpt2.context_length", wpe_rows)), wpe_rows)
        if T > wpe_rows:
            raise ValueError(f"max_seq_len={T} exceeds the {wpe_rows} rows of the file's position table")
        if "lm_head.weight" not in sd:   # GGUF exports of GPT-2 may tie the output matrix to the embeddings
            sd["lm_head.weight"] = sd["wte.weight"]
        params = GPT2Params(n_layers, n_heads, int(dim), int(vocab), eps)
        if not isinstance(wpe, Packed):
            sd["wpe.weight"] = wpe[:T]
        return GPT2(runtime or B200Runtime(0), params, sd, max_seq_len=T, batch=batch, precision=precision, **kw)
    finally:
        g.close()
