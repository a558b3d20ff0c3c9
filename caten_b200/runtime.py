"""Host-side mirror of the interface a Caten backend implements, over ``libcaten_b200.so``.

The reference registers a backend with ``(define-backend name buffer runtime renderer
auto-scheduler jit-p)`` (source/codegen/backend.lisp:22-34); its buffer class answers
``open-buffer / close-buffer / transfer-from-array / transfer-into-array / copy-buffer-value``
(source/runtime/buffer.lisp:78-89) and its runtime runs the kernels.  A Common Lisp image is not
available where this package is developed, so the same roles are written in Python over the C
ABI with the reference's names: :class:`B200Runtime` (context + kernel calls) and
:class:`B200Buffer` (shape/dtype/device pointer).  The Common Lisp glue that binds the same C symbols
through CFFI is ``lisp/b200.lisp`` at the top of this repository.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _lib as L
from .synthetic import Packed


class B200Buffer:
    """Device array: the counterpart of ``AbstractBuffer`` (source/runtime/buffer.lisp:46-52)."""

    def __init__(self, runtime: "B200Runtime", ptr: int, shape: Sequence[int], dtype, owned: bool = True):
        self.runtime, self.ptr, self.shape, self.dtype, self.owned = runtime, ptr, tuple(int(x) for x in shape), np.dtype(dtype), owned

    @property
    def nbytes(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize

    def numpy(self) -> np.ndarray:
        return self.runtime.transfer_into_array(self)

    def close(self):
        if self.owned and self.ptr and self.runtime.ctx is not None:
            self.runtime.close_buffer(self)

    def view(self, offset_elems: int, shape: Sequence[int]) -> "B200Buffer":
        return B200Buffer(self.runtime, self.ptr + offset_elems * self.dtype.itemsize, shape, self.dtype, owned=False)


class B200Weight:
    """Handle of a Linear weight kept in GGUF block form on the device."""

    def __init__(self, runtime: "B200Runtime", handle: int, ggml_type: int, rows: int, cols: int):
        self.runtime, self.handle, self.ggml_type, self.rows, self.cols = runtime, handle, ggml_type, rows, cols

    @property
    def packed_nbytes(self) -> int:
        return int(L.load().caten_b200_weight_nbytes(self.ggml_type, self.rows, self.cols))

    @property
    def device_nbytes(self) -> int:
        """Bytes held in device memory: ``packed_nbytes`` when the kernels read the format packed."""
        return int(L.load().caten_b200_weight_device_nbytes(self.handle))

    def dequantize(self) -> np.ndarray:
        """fp32 [rows, cols], the values external/gguf/dequantize.lisp:14-53 would produce."""
        rt = self.runtime
        out = rt.open_buffer((self.rows, self.cols), np.float32)
        L.check(rt.ctx, rt.lib.caten_b200_weight_dequant(rt.ctx, self.handle, out.ptr))
        a = out.numpy()
        out.close()
        return a

    def close(self):
        if self.handle and self.runtime.ctx is not None:
            self.runtime.lib.caten_b200_weight_free(self.runtime.ctx, self.handle)
        self.handle = 0


class B200Runtime:
    """One CUDA device + stream; the counterpart of a ``GraphRuntime`` subclass
    (source/runtime/runtime.lisp:39-54) reduced to what the GPT-2 path calls."""

    def __init__(self, device: int = 0):
        self.lib = L.load()
        ctx = C.c_void_p()
        L.check(None, self.lib.caten_b200_init(int(device), C.byref(ctx)))
        self.ctx = ctx
        self.device = device

    def close(self):
        if getattr(self, "ctx", None):
            self.lib.caten_b200_destroy(self.ctx)
            self.ctx = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- buffers (source/runtime/buffer.lisp:78-89) ----
    def open_buffer(self, shape, dtype=np.float32) -> B200Buffer:
        shape = tuple(int(x) for x in (shape if hasattr(shape, "__len__") else (shape,)))
        nbytes = int(np.prod(shape, dtype=np.int64)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        L.check(self.ctx, self.lib.caten_b200_malloc(self.ctx, nbytes, C.byref(p)))
        return B200Buffer(self, p.value, shape, dtype)

    def close_buffer(self, buf: B200Buffer):
        L.check(self.ctx, self.lib.caten_b200_free(self.ctx, buf.ptr))
        buf.ptr = 0

    def transfer_from_array(self, array, dtype=None) -> B200Buffer:
        a = np.ascontiguousarray(array, dtype=dtype)
        buf = self.open_buffer(a.shape, a.dtype)
        if a.nbytes:
            L.check(self.ctx, self.lib.caten_b200_h2d(self.ctx, buf.ptr, a.ctypes.data, a.nbytes))
        return buf

    def transfer_into_array(self, buf: B200Buffer) -> np.ndarray:
        out = np.empty(buf.shape, buf.dtype)
        if out.nbytes:
            L.check(self.ctx, self.lib.caten_b200_d2h(self.ctx, out.ctypes.data, buf.ptr, out.nbytes))
        return out

    def copy_buffer_value(self, buf: B200Buffer) -> B200Buffer:
        out = self.open_buffer(buf.shape, buf.dtype)
        L.check(self.ctx, self.lib.caten_b200_d2d(self.ctx, out.ptr, buf.ptr, buf.nbytes))
        return out

    def sync(self):
        L.check(self.ctx, self.lib.caten_b200_sync(self.ctx))

    def profile_begin(self, classes=None):
        """Starts CUDA-event timing of the given kernel classes (names of ``_lib.KERNEL_CLASSES``;
        all when None): the counterpart of PROFILE=1 (source/runtime/profile.lisp:15-39)."""
        names = L.KERNEL_CLASSES if classes is None else classes
        mask = 0
        for nme in names:
            mask |= 1 << L.KERNEL_CLASSES.index(nme)
        L.check(self.ctx, self.lib.caten_b200_profile_begin(self.ctx, mask))

    def profile_end(self) -> dict:
        """Stops timing; returns {class: (milliseconds, calls)} for classes that ran."""
        ms = (C.c_double * L.K_COUNT)()
        calls = (C.c_int64 * L.K_COUNT)()
        L.check(self.ctx, self.lib.caten_b200_profile_end(self.ctx, ms, calls))
        return {L.KERNEL_CLASSES[i]: (ms[i], calls[i]) for i in range(L.K_COUNT) if calls[i]}

    @property
    def stream(self) -> int:
        return int(self.lib.caten_b200_stream(self.ctx) or 0)

    # ---- weights ----
    def upload_weight(self, w) -> B200Weight:
        """``w``: :class:`Packed` raw GGUF blocks, or a 2-D float32/float16 array."""
        if isinstance(w, Packed):
            t, rows, cols, data = w.ggml_type, w.rows, w.cols, np.ascontiguousarray(w.data)
        else:
            a = np.ascontiguousarray(w)
            if a.ndim != 2 or a.dtype not in (np.float32, np.float16):
                raise ValueError("upload_weight: expected Packed or a 2-D float32/float16 array")
            t, (rows, cols), data = (L.F32 if a.dtype == np.float32 else L.F16), a.shape, a
        h = C.c_void_p()
        L.check(self.ctx, self.lib.caten_b200_weight_upload(self.ctx, t, data.ctypes.data, rows, cols, C.byref(h)))
        return B200Weight(self, h.value, t, rows, cols)

    def upload_weight_device(self, ggml_type: int, d_blocks_ptr: int, rows: int, cols: int) -> B200Weight:
        h = C.c_void_p()
        L.check(self.ctx, self.lib.caten_b200_weight_upload_device(self.ctx, ggml_type, d_blocks_ptr, rows, cols, C.byref(h)))
        return B200Weight(self, h.value, ggml_type, rows, cols)

    # ---- kernels ----
    def linear(self, w: B200Weight, x: B200Buffer, bias: Optional[B200Buffer] = None,
               residual: Optional[B200Buffer] = None, act: int = L.ACT_NONE, precision: int = L.PREC_FP32,
               out: Optional[B200Buffer] = None) -> B200Buffer:
        M = int(np.prod(x.shape[:-1], dtype=np.int64))
        if x.shape[-1] != w.cols:
            raise ValueError(f"linear: x has {x.shape[-1]} features, weight expects {w.cols}")
        y = out or self.open_buffer(x.shape[:-1] + (w.rows,), np.float32)
        L.check(self.ctx, self.lib.caten_b200_linear(self.ctx, w.handle, x.ptr, bias.ptr if bias else None,
                                                     residual.ptr if residual else None, act, y.ptr, M, precision))
        return y

    def linear_noalloc(self, w: B200Weight, x: B200Buffer, out: B200Buffer, bias: Optional[B200Buffer] = None,
                       residual: Optional[B200Buffer] = None, act: int = L.ACT_NONE, precision: int = L.PREC_BF16X3) -> B200Buffer:
        """``linear`` for callers that must not trigger an allocation: the caller supplies ``out`` and
        the library keeps its working memory in a fixed 32 MiB buffer of its own image
        (``caten_b200_linear_noalloc``).  Larger working sets raise ``B200Error`` (EUNSUPPORTED).
        Calls that may overlap on the GPU share that buffer and must be serialised by the caller."""
        M = int(np.prod(x.shape[:-1], dtype=np.int64))
        if x.shape[-1] != w.cols or out.shape[-1] != w.rows:
            raise ValueError("linear_noalloc: shape mismatch")
        L.check(self.ctx, self.lib.caten_b200_linear_noalloc(self.ctx, w.handle, x.ptr, bias.ptr if bias else None,
                                                             residual.ptr if residual else None, act, out.ptr, M, precision))
        return out

    def relu_matmul(self, a: B200Buffer, b: B200Buffer, precision: int = L.PREC_BF16X3) -> B200Buffer:
        (M, K), (K2, N) = a.shape, b.shape
        if K != K2:
            raise ValueError("relu_matmul: inner dimensions differ")
        c = self.open_buffer((M, N), np.float32)
        L.check(self.ctx, self.lib.caten_b200_relu_matmul(self.ctx, a.ptr, b.ptr, c.ptr, M, K, N, precision))
        return c

    def layernorm(self, x: B200Buffer, gamma: B200Buffer, beta: B200Buffer, eps: float = 1e-5) -> B200Buffer:
        d = x.shape[-1]
        rows = int(np.prod(x.shape[:-1], dtype=np.int64))
        y = self.open_buffer(x.shape, np.float32)
        L.check(self.ctx, self.lib.caten_b200_layernorm(self.ctx, x.ptr, gamma.ptr, beta.ptr, y.ptr, rows, d, eps))
        return y

    def rmsnorm(self, x: B200Buffer, weight: Optional[B200Buffer] = None, eps: float = 1e-5) -> B200Buffer:
        """`!rms-norm` (source/nn/normalization.lisp:70-85) over the last axis."""
        d = x.shape[-1]
        rows = int(np.prod(x.shape[:-1], dtype=np.int64))
        y = self.open_buffer(x.shape, np.float32)
        L.check(self.ctx, self.lib.caten_b200_rmsnorm(self.ctx, x.ptr, weight.ptr if weight else None, y.ptr, rows, d, eps))
        return y

    def rope(self, x: B200Buffer, base: float = 10000.0, pos0: int = 0) -> B200Buffer:
        """`!rope` (source/nn/positional-encoding.lisp:3-56) on x [B, S, H, head_dim]."""
        B, S_, H, hd = x.shape
        y = self.open_buffer(x.shape, np.float32)
        L.check(self.ctx, self.lib.caten_b200_rope(self.ctx, x.ptr, y.ptr, B, S_, H, hd, float(base), int(pos0)))
        return y

    def embed(self, ids: B200Buffer, wte: B200Buffer, wpe: B200Buffer, n: int) -> B200Buffer:
        B, s = ids.shape
        V, d = wte.shape
        out = self.open_buffer((B, s, d), np.float32)
        f32 = ids.ptr if ids.dtype == np.float32 else None
        i64 = ids.ptr if ids.dtype == np.int64 else None
        if f32 is None and i64 is None:
            raise ValueError("embed: ids must be float32 or int64")
        L.check(self.ctx, self.lib.caten_b200_embed(self.ctx, f32, i64, wte.ptr, wpe.ptr, out.ptr, B, s, n, d, V, wpe.shape[0]))
        return out

    def attention(self, qkv: B200Buffer, kcache: B200Buffer, vcache: B200Buffer, B: int, s: int, n: int,
                  precision: int = L.PREC_FP32) -> B200Buffer:
        """kcache/vcache: [B, H, T, 64]; qkv: [B*s, 3*H*64].  A tensor-core precision selects the
        split-bf16 tensor-core kernel for steps of more than one token."""
        _, H, T, hd = kcache.shape
        out = self.open_buffer((B * s, H * hd), np.float32)
        L.check(self.ctx, self.lib.caten_b200_attention_ex(self.ctx, qkv.ptr, kcache.ptr, vcache.ptr, out.ptr, B, s, n, H, T, precision))
        return out

    def argmax(self, x: B200Buffer) -> B200Buffer:
        rows, V = x.shape
        out = self.open_buffer((rows,), np.int64)
        L.check(self.ctx, self.lib.caten_b200_argmax(self.ctx, x.ptr, rows, V, out.ptr))
        return out

    def sample(self, logits: B200Buffer, uniform, temperature: float = 1.0, top_k: int = 0) -> B200Buffer:
        """One id per row by temperature / top-k sampling (`caten_b200_sample`; the reference only has the
        greedy argmax).  ``uniform``: one number in [0, 1) per row (array or device buffer)."""
        rows, V = logits.shape
        u = uniform if isinstance(uniform, B200Buffer) else self.transfer_from_array(np.asarray(uniform, np.float32).reshape(rows))
        out = self.open_buffer((rows,), np.int64)
        L.check(self.ctx, self.lib.caten_b200_sample(self.ctx, logits.ptr, rows, V, float(temperature), int(top_k), u.ptr, out.ptr))
        return out
