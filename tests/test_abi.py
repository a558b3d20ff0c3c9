"""CPU checks of the C-ABI boundary: the library builds, loads, and exports exactly what
include/caten_b200.h declares.  No kernel is launched here."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "caten_b200.h")


def _declared():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(caten_b200_[a-z0-9_]+)\s*\(", src)))


@pytest.fixture(scope="module")
def lib():
    from caten_b200 import _lib, build
    build.build()
    return _lib.load()


def test_header_symbols_are_exported(lib):
    names = _declared()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in caten_b200.h but not exported"


def test_bindings_cover_the_header(lib):
    from caten_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared()


def test_header_cites_the_reference_for_every_entry_group():
    src = open(HEADER).read()
    for needle in ("source/runtime/buffer.lisp", "external/gguf/dequantize.lisp", "source/nn/linear.lisp",
                   "source/nn/normalization.lisp", "external/llm/layers.lisp", "apps/gpt2/gpt2.lisp",
                   "api/high-level-ops.lisp", "source/byoc/clang.lisp"):
        assert needle in src


def test_weight_nbytes(lib):
    assert lib.caten_b200_weight_nbytes(0, 3, 64) == 3 * 64 * 4
    assert lib.caten_b200_weight_nbytes(1, 3, 64) == 3 * 64 * 2
    assert lib.caten_b200_weight_nbytes(2, 3, 64) == 3 * 2 * 18
    assert lib.caten_b200_weight_nbytes(8, 3, 64) == 3 * 2 * 34
    assert lib.caten_b200_weight_nbytes(2, 3, 48) == -1   # not whole blocks
    assert lib.caten_b200_weight_nbytes(12, 3, 64) == -1  # Q4_K super-blocks hold 256 weights: 64 columns are not whole blocks
    assert lib.caten_b200_weight_nbytes(12, 3, 256) == 3 * 144
    assert lib.caten_b200_weight_nbytes(99, 3, 256) == -1  # unknown type id
    assert lib.caten_b200_arch() == b"sm_100a"


def test_null_arguments_are_rejected_without_touching_a_gpu(lib):
    from caten_b200 import _lib
    assert lib.caten_b200_init(0, None) == _lib.EINVAL
    assert b"NULL" in lib.caten_b200_last_error(None)
    assert lib.caten_b200_sync(None) == _lib.EINVAL
    assert lib.caten_b200_gpt2_step(None, None, 1, 0, None) == _lib.EINVAL
    assert lib.caten_b200_destroy(None) == 0


def test_init_fails_loudly_without_a_device(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from caten_b200.runtime import B200Runtime
    from caten_b200._lib import B200Error
    with pytest.raises(B200Error):
        B200Runtime(0)


def test_missing_library_is_an_error(monkeypatch):
    from caten_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libcaten_b200.so")
    with pytest.raises(_lib.B200Error):
        _lib.load()


def test_product_code_never_touches_the_oracle():
    for dirpath, _, files in os.walk(os.path.join(ROOT, "caten_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".lisp")):
                txt = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in txt and "from oracle" not in txt and "libcaten_oracle" not in txt, f
