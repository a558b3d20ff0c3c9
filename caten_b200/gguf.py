"""GGUF loading for the B200 backend: host-side counterpart of the reference's `caten/gguf`
package (external/gguf/gguf-file.lisp, metadata.lisp, tensor-info.lisp).

``load_gguf`` plays `load-gguf` (gguf-file.lisp:83-91), ``GGUF.metadata`` the parsed key/values
(metadata.lisp:58-87), ``gguf_to_state_dict`` plays `gguf->state-dict` (gguf-file.lisp:93-104)
followed by the GPT-2 key remapping of apps/gpt2/gpt2.lisp:52-80 — except that quantised
tensors are NOT dequantised: they come back as :class:`Packed` views of the memory-mapped file,
ready for ``caten_b200_weight_upload``.  Parsing happens in the C library (`csrc/gguf.cu`).
"""
from __future__ import annotations

import ctypes as C
import struct
from typing import Dict

import numpy as np

from . import _lib as L
from .synthetic import Packed

_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}

# GGUF tensor name -> reference state-dict key (apps/gpt2/gpt2.lisp:52-70), applied in this order
REMAP = [("blk.", "h."), ("token_embd.weight", "wte.weight"), ("position_embd.weight", "wpe.weight"),
         (".attn_norm.weight", ".ln_1.affine"), (".attn_norm.bias", ".ln_1.bias"),
         (".attn_qkv.weight", ".attn.c_attn.weight"), (".attn_qkv.bias", ".attn.c_attn.bias"),
         (".ffn_down.weight", ".mlp.c_proj.weight"), (".ffn_down.bias", ".mlp.c_proj.bias"),
         (".ffn_norm.weight", ".ln_2.affine"), (".ffn_norm.bias", ".ln_2.bias"),
         (".ffn_up.weight", ".mlp.c_fc.weight"), (".ffn_up.bias", ".mlp.c_fc.bias"),
         (".attn_output.weight", ".attn.c_proj.weight"), (".attn_output.bias", ".attn.c_proj.bias"),
         ("output.weight", "lm_head.weight"), ("output_norm.bias", "ln_f.bias"), ("output_norm.weight", "ln_f.affine")]


def remap_key(key: str) -> str:
    """`remap-key` (apps/gpt2/gpt2.lisp:72-75)."""
    for before, after in REMAP:
        key = key.replace(before, after)
    return key


class TensorInfo:
    """One entry of the tensor table (`tensor-info`, external/gguf/tensor-info.lisp:43-69)."""

    def __init__(self, name, ggml_type, dims, data_ptr, nbytes, owner):
        self.name, self.ggml_type, self.dims, self._ptr, self.nbytes, self._owner = name, ggml_type, dims, data_ptr, nbytes, owner

    @property
    def shape(self):
        """Row-major shape (GGUF lists dimensions innermost first; tensor-info.lisp:108 reverses them)."""
        return tuple(reversed(self.dims))

    def raw(self) -> np.ndarray:
        """uint8 view of the tensor's bytes inside the memory map (no copy)."""
        if self.nbytes < 0:
            raise L.B200Error(L.EUNSUPPORTED, f"{self.name}: ggml type {self.ggml_type} is not held by this library")
        buf = (C.c_uint8 * self.nbytes).from_address(self._ptr)
        a = np.frombuffer(buf, dtype=np.uint8)
        a.flags.writeable = False
        return a


class GGUF:
    def __init__(self, path: str):
        self.lib = L.load()
        h = C.c_void_p()
        L.check(None, self.lib.caten_b200_gguf_open(str(path).encode(), C.byref(h)))
        self._h = h
        self.version = int(self.lib.caten_b200_gguf_version(h))
        self.alignment = int(self.lib.caten_b200_gguf_alignment(h))
        self.tensors: Dict[str, TensorInfo] = {}
        self.order = []
        for i in range(int(self.lib.caten_b200_gguf_tensor_count(h))):
            name, t, nd, data, nb = C.c_char_p(), C.c_int(), C.c_int(), C.c_void_p(), C.c_int64()
            dims = (C.c_int64 * 4)()
            L.check(None, self.lib.caten_b200_gguf_tensor(h, i, C.byref(name), C.byref(t), C.byref(nd), dims, C.byref(data), C.byref(nb)))
            info = TensorInfo(name.value.decode(), t.value, tuple(dims[k] for k in range(nd.value)), data.value, nb.value, self)
            self.tensors[info.name] = info
            self.order.append(info.name)
        self.metadata = {}
        for i in range(int(self.lib.caten_b200_gguf_meta_count(h))):
            key, t, et, cnt, val, sl = C.c_char_p(), C.c_int(), C.c_int(), C.c_int64(), C.c_void_p(), C.c_int64()
            L.check(None, self.lib.caten_b200_gguf_meta(h, i, C.byref(key), C.byref(t), C.byref(et), C.byref(cnt), C.byref(val), C.byref(sl)))
            self.metadata[key.value.decode()] = self._decode(t.value, et.value, cnt.value, val.value, sl.value)

    @staticmethod
    def _decode(t, et, count, ptr, str_len):
        if t == 8:
            return C.string_at(ptr, str_len).decode("utf-8", "replace")
        if t == 9:
            if et == 8:
                out, p = [], ptr
                for _ in range(count):
                    n = struct.unpack("<Q", C.string_at(p, 8))[0]
                    out.append(C.string_at(p + 8, n).decode("utf-8", "replace"))
                    p += 8 + n
                return out
            fmt = _SCALAR[et]
            sz = struct.calcsize(fmt)
            return list(struct.unpack("<" + fmt[1] * count, C.string_at(ptr, sz * count)))
        fmt = _SCALAR[t]
        return struct.unpack(fmt, C.string_at(ptr, struct.calcsize(fmt)))[0]

    def upload(self, name: str, runtime):
        """Uploads a 2-D tensor as a Linear weight straight from the mapping."""
        from .runtime import B200Weight
        i = int(self.lib.caten_b200_gguf_find_tensor(self._h, name.encode()))
        if i < 0:
            raise KeyError(name)
        w = C.c_void_p()
        L.check(runtime.ctx, self.lib.caten_b200_gguf_upload(runtime.ctx, self._h, i, C.byref(w)))
        info = self.tensors[name]
        return B200Weight(runtime, w.value, info.ggml_type, info.dims[1], info.dims[0])

    def close(self):
        if getattr(self, "_h", None):
            self.lib.caten_b200_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def load_gguf(path: str) -> GGUF:
    """`load-gguf` (external/gguf/gguf-file.lisp:83-91)."""
    return GGUF(path)


def gguf_to_state_dict(g: GGUF, remap=remap_key) -> dict:
    """`gguf->state-dict` + `remap-state-dict-keys`.  2-D F16 and block-quantised tensors stay packed
    (:class:`Packed`, zero-copy); F32 tensors and all 1-D tensors become float32 arrays (1-D F16 is
    widened).  The arrays are views of the mapping: keep ``g`` open while they are in use."""
    sd = {}
    for name in g.order:
        t = g.tensors[name]
        raw = t.raw()
        key = remap(name) if remap else name
        if len(t.dims) == 2 and t.ggml_type in L.BLOCK_FORMATS:
            sd[key] = Packed(t.ggml_type, t.dims[1], t.dims[0], raw)
        elif t.ggml_type == L.F32:
            sd[key] = raw.view(np.float32).reshape(t.shape)
        elif t.ggml_type == L.F16:
            a = raw.view(np.float16).reshape(t.shape)
            sd[key] = a if len(t.dims) == 2 else a.astype(np.float32)
        else:
            raise L.B200Error(L.EUNSUPPORTED, f"{name}: ggml type {t.ggml_type} with {len(t.dims)} dims")
    return sd
