"""ctypes bindings of ``libcaten_b200.so`` (the C ABI declared in include/caten_b200.h).

There is no fallback: if the library is missing or fails to load, importing a compute entry
point raises, and every non-zero status becomes a :class:`B200Error` carrying
``caten_b200_last_error``.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# CATEN_B200_LIB: load another build of the library (e.g. one with development instrumentation)
LIB_PATH = os.environ.get("CATEN_B200_LIB") or os.path.join(HERE, "libcaten_b200.so")

OK, EINVAL, ECUDA, EUNSUPPORTED, EDEVICE = 0, 1, 2, 3, 4
F32, F16, Q4_0, Q8_0 = 0, 1, 2, 8
Q4_1, Q5_0, Q5_1 = 3, 6, 7                                # kept packed, like Q4_0 and Q8_0
Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 10, 11, 12, 13, 14        # expanded to fp32 at upload
BLOCK_FORMATS = (Q4_0, Q8_0, Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K)
ACT_NONE, ACT_GELU, ACT_RELU = 0, 1, 2
PREC_FP32, PREC_BF16, PREC_BF16X3 = 0, 1, 2
K_EMBED, K_LAYERNORM, K_GEMV, K_GEMM, K_ATTN_DECODE, K_ATTN_PREFILL, K_ARGMAX, K_COUNT = 0, 1, 2, 3, 4, 5, 6, 8
KERNEL_CLASSES = ["embed", "layernorm", "gemv", "gemm", "attn_decode", "attn_prefill", "argmax", "decode_step"]
DIST_ID_BYTES = 128
PRECISIONS = {"fp32": PREC_FP32, "bf16": PREC_BF16, "bf16x3": PREC_BF16X3}


class B200Error(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"caten_b200 error {code}: {msg}")
        self.code = code


_vp = C.c_void_p
_i64 = C.c_int64
_PFP = C.POINTER(_vp)


class GPT2Desc(C.Structure):
    """Mirror of ``caten_b200_gpt2_desc``."""
    _fields_ = [
        ("n_layers", C.c_int32), ("d_model", C.c_int32), ("n_heads", C.c_int32), ("vocab", C.c_int32),
        ("max_seq_len", C.c_int32), ("batch", C.c_int32), ("eps", C.c_float), ("precision", C.c_int32),
        ("max_rows", C.c_int32),
        ("wte", _vp), ("wpe", _vp), ("lnf_g", _vp), ("lnf_b", _vp), ("lm_head", _vp),
        ("ln1_g", _PFP), ("ln1_b", _PFP), ("attn_b", _PFP), ("proj_b", _PFP),
        ("ln2_g", _PFP), ("ln2_b", _PFP), ("fc_b", _PFP), ("mproj_b", _PFP),
        ("attn_w", _PFP), ("proj_w", _PFP), ("fc_w", _PFP), ("mproj_w", _PFP),
    ]


EXPR_MAX_DIMS, EXPR_MAX_OPERANDS, EXPR_MAX_CODE, EXPR_MAX_CONSTS = 6, 8, 96, 16


class ExprDesc(C.Structure):
    """Mirror of ``caten_b200_expr``."""
    _fields_ = [
        ("ndim", C.c_int32), ("shape", _i64 * EXPR_MAX_DIMS), ("n_reduce", C.c_int32), ("reduce_op", C.c_int32),
        ("accumulate", C.c_int32), ("n_operands", C.c_int32),
        ("operand", _vp * EXPR_MAX_OPERANDS), ("operand_dtype", C.c_int32 * EXPR_MAX_OPERANDS),
        ("operand_offset", _i64 * EXPR_MAX_OPERANDS), ("operand_stride", (_i64 * EXPR_MAX_DIMS) * EXPR_MAX_OPERANDS),
        ("out", _vp), ("out_dtype", C.c_int32), ("out_offset", _i64), ("out_stride", _i64 * EXPR_MAX_DIMS),
        ("n_code", C.c_int32), ("code", C.c_uint32 * EXPR_MAX_CODE), ("consts", C.c_uint32 * EXPR_MAX_CONSTS),
    ]


# name -> (restype, argtypes); every name here must be declared in include/caten_b200.h
SIGNATURES = {
    "caten_b200_eval_expr": (C.c_int, [_vp, C.POINTER(ExprDesc)]),
    "caten_b200_init": (C.c_int, [C.c_int, _PFP]),
    "caten_b200_destroy": (C.c_int, [_vp]),
    "caten_b200_last_error": (C.c_char_p, [_vp]),
    "caten_b200_malloc": (C.c_int, [_vp, C.c_size_t, _PFP]),
    "caten_b200_free": (C.c_int, [_vp, _vp]),
    "caten_b200_h2d": (C.c_int, [_vp, _vp, _vp, C.c_size_t]),
    "caten_b200_d2h": (C.c_int, [_vp, _vp, _vp, C.c_size_t]),
    "caten_b200_d2d": (C.c_int, [_vp, _vp, _vp, C.c_size_t]),
    "caten_b200_memset": (C.c_int, [_vp, _vp, C.c_int, C.c_size_t]),
    "caten_b200_sync": (C.c_int, [_vp]),
    "caten_b200_stream": (_vp, [_vp]),
    "caten_b200_set_stream": (C.c_int, [_vp, _vp]),
    "caten_b200_weight_upload": (C.c_int, [_vp, C.c_int, _vp, _i64, _i64, _PFP]),
    "caten_b200_weight_upload_device": (C.c_int, [_vp, C.c_int, _vp, _i64, _i64, _PFP]),
    "caten_b200_weight_free": (C.c_int, [_vp, _vp]),
    "caten_b200_weight_nbytes": (_i64, [C.c_int, _i64, _i64]),
    "caten_b200_weight_device_nbytes": (_i64, [_vp]),
    "caten_b200_weight_dequant": (C.c_int, [_vp, _vp, _vp]),
    "caten_b200_gguf_open": (C.c_int, [C.c_char_p, _PFP]),
    "caten_b200_gguf_close": (C.c_int, [_vp]),
    "caten_b200_gguf_version": (C.c_int, [_vp]),
    "caten_b200_gguf_alignment": (_i64, [_vp]),
    "caten_b200_gguf_tensor_count": (_i64, [_vp]),
    "caten_b200_gguf_meta_count": (_i64, [_vp]),
    "caten_b200_gguf_tensor": (C.c_int, [_vp, _i64, C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                         C.POINTER(_i64), _PFP, C.POINTER(_i64)]),
    "caten_b200_gguf_find_tensor": (_i64, [_vp, C.c_char_p]),
    "caten_b200_gguf_meta": (C.c_int, [_vp, _i64, C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                       C.POINTER(_i64), _PFP, C.POINTER(_i64)]),
    "caten_b200_gguf_upload": (C.c_int, [_vp, _vp, _i64, _PFP]),
    "caten_b200_linear": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_int, _vp, _i64, C.c_int]),
    "caten_b200_linear_noalloc": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_int, _vp, _i64, C.c_int]),
    "caten_b200_relu_matmul": (C.c_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, C.c_int]),
    "caten_b200_layernorm": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, C.c_float]),
    "caten_b200_embed": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64]),
    "caten_b200_attention": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64]),
    "caten_b200_attention_ex": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, C.c_int]),
    "caten_b200_argmax": (C.c_int, [_vp, _vp, _i64, _i64, _vp]),
    "caten_b200_rmsnorm": (C.c_int, [_vp, _vp, _vp, _vp, _i64, _i64, C.c_float]),
    "caten_b200_rope": (C.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, C.c_float, _i64]),
    "caten_b200_sample": (C.c_int, [_vp, _vp, _i64, _i64, C.c_float, C.c_int, _vp, _vp]),
    "caten_b200_gpt2_create": (C.c_int, [_vp, C.POINTER(GPT2Desc), _PFP]),
    "caten_b200_gpt2_destroy": (C.c_int, [_vp]),
    "caten_b200_gpt2_step": (C.c_int, [_vp, _vp, _i64, _i64, _vp]),
    "caten_b200_gpt2_step_device": (C.c_int, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "caten_b200_gpt2_decode": (C.c_int, [_vp, _vp, _i64, _i64, _vp]),
    "caten_b200_gpt2_logits": (_vp, [_vp]),
    "caten_b200_gpt2_kv": (C.c_int, [_vp, C.c_int, _PFP, _PFP]),
    "caten_b200_gpt2_launch_count": (_i64, [_vp]),
    "caten_b200_dist_unique_id": (C.c_int, [_vp]),
    "caten_b200_dist_init": (C.c_int, [_vp, C.c_int, C.c_int, _vp]),
    "caten_b200_dist_finalize": (C.c_int, [_vp]),
    "caten_b200_dist_rank": (C.c_int, [_vp]),
    "caten_b200_dist_world": (C.c_int, [_vp]),
    "caten_b200_dist_shard": (C.c_int, [_i64, C.c_int, C.c_int, C.POINTER(_i64), C.POINTER(_i64)]),
    "caten_b200_dist_bcast_weights": (C.c_int, [_vp, _vp, C.c_size_t, C.c_int]),
    "caten_b200_dist_gather_ids": (C.c_int, [_vp, _vp, _i64, _vp]),
    "caten_b200_profile_begin": (C.c_int, [_vp, C.c_uint]),
    "caten_b200_profile_end": (C.c_int, [_vp, _vp, _vp]),
    "caten_b200_arch": (C.c_char_p, []),
}

_lib = None


def load():
    """Loads the shared library (building nothing: run ``python -m caten_b200.build`` first)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200Error(ECUDA, f"{LIB_PATH} is missing: build it with `python -m caten_b200.build`")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(ctx, rc: int):
    if rc != 0:
        msg = load().caten_b200_last_error(ctx)
        raise B200Error(rc, (msg or b"").decode("utf-8", "replace"))
