"""TEST INFRASTRUCTURE: ctypes front end of the CPU oracle (``libcaten_oracle.so``).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` import
this package.  The CUDA library and the ``caten_b200`` package never do.

The oracle restates hikettei/Caten's GPT-2 path (external/llm/layers.lisp, source/nn/*.lisp,
external/gguf/dequantize.lisp) op by op; see caten_oracle.c for what pins it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libcaten_oracle.so")

# numeric variants (see caten_oracle.c)
STRICT_F32, C_PROMOTED, ALL_F64 = 0, 1, 2

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0 = 0, 1, 2, 8


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc -O3, no fast-math)."""
    srcs = [os.path.join(_HERE, f) for f in ("caten_oracle.c", "gpt2_impl.inc", "Makefile")]
    stale = not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in srcs
    )
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "libcaten_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


class _Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("n_layers", "d_model", "n_heads", "vocab", "max_seq_len", "batch")] + [("eps", C.c_float)]


_PF = C.POINTER(C.c_float)
_PPF = C.POINTER(_PF)


class _Weights(C.Structure):
    _fields_ = [(n, _PF) for n in ("wte", "wpe", "lnf_g", "lnf_b", "lm_head")] + [
        (n, _PPF) for n in ("ln1_g", "ln1_b", "attn_w", "attn_b", "proj_w", "proj_b",
                            "ln2_g", "ln2_b", "fc_w", "fc_b", "mproj_w", "mproj_b")]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_half_to_float.restype = C.c_float
        _lib.orc_half_to_float.argtypes = [C.c_uint16]
        _lib.orc_gpt2_create.restype = C.c_void_p
        _lib.orc_gpt2_create.argtypes = [C.POINTER(_Config), C.POINTER(_Weights), C.c_int]
        _lib.orc_gpt2_step.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]
        _lib.orc_gpt2_destroy.argtypes = [C.c_void_p]
        _lib.orc_gpt2_fill_cache.argtypes = [C.c_void_p, C.c_float]
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def set_threads(n: int) -> None:
    lib().orc_set_threads(int(n))


def max_threads() -> int:
    return int(lib().orc_max_threads())


def half_to_float(h: int) -> float:
    return float(lib().orc_half_to_float(int(h)))


def dequant(ggml_type: int, blocks: np.ndarray, n: int) -> np.ndarray:
    """Dequantise ``n`` elements of raw GGUF block bytes to fp32."""
    src = np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
    out = np.empty(n, dtype=np.float32)
    rc = lib().orc_dequant(C.c_int(ggml_type), _p(src), C.c_int64(n), _p(out))
    if rc:
        raise ValueError(f"orc_dequant: unsupported type/size (rc={rc})")
    return out


def embedding(tok, n, wte, wpe):
    tok = _f32(tok); wte = _f32(wte); wpe = _f32(wpe)
    B, s = tok.shape
    V, d = wte.shape
    out = np.empty((B, s, d), np.float32)
    lib().orc_embedding(_p(tok), C.c_int64(B), C.c_int64(s), C.c_int64(n), _p(wte), _p(wpe),
                        C.c_int64(V), C.c_int64(wpe.shape[0]), C.c_int64(d), _p(out))
    return out


def layernorm(x, g, b, eps=1e-5, mode=STRICT_F32):
    x = _f32(x); g = _f32(g); b = _f32(b)
    rows, d = x.reshape(-1, x.shape[-1]).shape
    y = np.empty_like(x)
    lib().orc_layernorm(C.c_int(mode), _p(x), _p(g), _p(b), C.c_int64(rows), C.c_int64(d),
                        C.c_float(eps), _p(y))
    return y


def linear(x, W, bias=None, res=None, act=0, mode=STRICT_F32):
    """y = act(x @ W.T + bias) + res ; act 0 none, 1 GeLU, 2 ReLU."""
    x = _f32(x); W = _f32(W)
    M, K = x.shape
    N = W.shape[0]
    assert W.shape[1] == K
    bias = None if bias is None else _f32(bias)
    res = None if res is None else _f32(res)
    y = np.empty((M, N), np.float32)
    lib().orc_linear(C.c_int(mode), _p(x), _p(W), _p(bias), _p(res), C.c_int(act), C.c_int64(M),
                     C.c_int64(N), C.c_int64(K), _p(y))
    return y


def relu_matmul(a, b, mode=STRICT_F32):
    a = _f32(a); b = _f32(b)
    M, K = a.shape
    N = b.shape[1]
    c = np.empty((M, N), np.float32)
    lib().orc_relu_matmul(C.c_int(mode), _p(a), _p(b), C.c_int64(M), C.c_int64(K), C.c_int64(N), _p(c))
    return c


def gelu(x, mode=STRICT_F32):
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_gelu(C.c_int(mode), _p(x), C.c_int64(x.size), _p(y))
    return y


def attention(qkv, kc, vc, B, s, n, H, mode=STRICT_F32):
    """qkv [B*s, 3d]; kc/vc [B, T, H, hd] float32 arrays updated in place. Returns [B*s, d]."""
    qkv = _f32(qkv)
    assert kc.dtype == np.float32 and kc.flags.c_contiguous and vc.flags.c_contiguous
    T, hd = kc.shape[1], kc.shape[3]
    out = np.empty((B * s, H * hd), np.float32)
    lib().orc_attention(C.c_int(mode), _p(qkv), _p(kc), _p(vc), C.c_int64(B), C.c_int64(s),
                        C.c_int64(n), C.c_int64(H), C.c_int64(hd), C.c_int64(T), _p(out))
    return out


def rmsnorm(x, weight=None, eps=1e-5, mode=STRICT_F32):
    x = _f32(x)
    weight = None if weight is None else _f32(weight)
    rows, d = x.reshape(-1, x.shape[-1]).shape
    y = np.empty_like(x)
    lib().orc_rmsnorm(C.c_int(mode), _p(x), _p(weight), C.c_int64(rows), C.c_int64(d), C.c_float(eps), _p(y))
    return y


def rope(x, base=10000.0, pos0=0, mode=STRICT_F32):
    """x [B, S, H, head_dim] -> rotated copy (`!rope x (head_dim / 2)`)."""
    x = _f32(x)
    B, S, H, hd = x.shape
    y = np.empty_like(x)
    lib().orc_rope(C.c_int(mode), _p(x), C.c_int64(B), C.c_int64(S), C.c_int64(H), C.c_int64(hd), C.c_float(base),
                   C.c_int64(pos0), _p(y))
    return y


def argmax(x):
    x = _f32(x)
    rows, V = x.shape
    out = np.empty(rows, np.int64)
    lib().orc_argmax(_p(x), C.c_int64(rows), C.c_int64(V), _p(out))
    return out


class GPT2:
    """Whole-model oracle. ``sd`` maps the reference's state-dict keys (after the remapping of
    apps/gpt2/gpt2.lisp:52-70) to fp32 arrays, i.e. weights already dequantised, as the reference
    holds them."""

    def __init__(self, n_layers, d_model, n_heads, vocab, max_seq_len, batch, sd, eps=1e-5,
                 mode=STRICT_F32):
        self.cfg = _Config(n_layers, d_model, n_heads, vocab, max_seq_len, batch, eps)
        self.batch, self.vocab = batch, vocab
        self._keep = []

        def one(key):
            a = _f32(sd[key])
            self._keep.append(a)
            return a.ctypes.data_as(_PF)

        def per_layer(fmt):
            arr = (_PF * n_layers)(*[one(fmt.format(l)) for l in range(n_layers)])
            self._keep.append(arr)
            return C.cast(arr, _PPF)

        w = _Weights(
            one("wte.weight"), one("wpe.weight"), one("ln_f.affine"), one("ln_f.bias"),
            one("lm_head.weight"),
            per_layer("h.{}.ln_1.affine"), per_layer("h.{}.ln_1.bias"),
            per_layer("h.{}.attn.c_attn.weight"), per_layer("h.{}.attn.c_attn.bias"),
            per_layer("h.{}.attn.c_proj.weight"), per_layer("h.{}.attn.c_proj.bias"),
            per_layer("h.{}.ln_2.affine"), per_layer("h.{}.ln_2.bias"),
            per_layer("h.{}.mlp.c_fc.weight"), per_layer("h.{}.mlp.c_fc.bias"),
            per_layer("h.{}.mlp.c_proj.weight"), per_layer("h.{}.mlp.c_proj.bias"))
        self._h = lib().orc_gpt2_create(C.byref(self.cfg), C.byref(w), C.c_int(mode))
        if not self._h:
            raise ValueError("orc_gpt2_create failed")

    def step(self, tokens, n, want_logits=True):
        """tokens [B, s] (any numeric dtype; passed as float32 like apps/gpt2/gpt2.lisp:95)."""
        tok = _f32(tokens)
        assert tok.shape[0] == self.batch
        ids = np.empty(self.batch, np.int64)
        logits = np.empty((self.batch, self.vocab), np.float32) if want_logits else None
        rc = lib().orc_gpt2_step(self._h, _p(tok), C.c_int64(tok.shape[1]), C.c_int64(n), _p(ids),
                                 _p(logits))
        if rc:
            raise ValueError(f"orc_gpt2_step rc={rc}")
        return ids, logits

    def fill_cache(self, value=0.01):
        lib().orc_gpt2_fill_cache(self._h, C.c_float(value))

    def close(self):
        if self._h:
            lib().orc_gpt2_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
