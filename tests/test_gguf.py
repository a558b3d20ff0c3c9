"""CPU tests of the GGUF reader (C parser + Python host) against files written by the Python
`gguf` package, the way source/test-suite/external/test-gguf.lisp:8-32 writes its dummy files."""
import os
import struct

import numpy as np
import pytest

from caten_b200 import synthetic as S
from caten_b200._lib import B200Error
from caten_b200.gguf import gguf_to_state_dict, load_gguf, remap_key

gguf = pytest.importorskip("gguf")
from gguf import GGMLQuantizationType as GT  # noqa: E402
from gguf import GGUFReader, GGUFWriter  # noqa: E402


def write_file(path, tensors, meta=None, alignment=None):
    w = GGUFWriter(str(path), "gpt2")
    if alignment:
        w.add_custom_alignment(alignment)
    for k, v in (meta or {}).items():
        if isinstance(v, str):
            w.add_string(k, v)
        elif isinstance(v, float):
            w.add_float32(k, v)
        elif isinstance(v, list):
            w.add_array(k, v)
        else:
            w.add_uint32(k, v)
    for name, (arr, raw_dtype) in tensors.items():
        w.add_tensor(name, arr, raw_dtype=raw_dtype)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def packed_as_writer_array(p: S.Packed):
    bb = S.BLOCK_BYTES[p.ggml_type]
    return p.data.reshape(p.rows, p.cols // 32 * bb)


@pytest.fixture()
def sample(tmp_path):
    rng = np.random.Generator(np.random.PCG64(0))
    q4 = S._rand_packed(rng, 6, 64, "q4_0")
    q8 = S._rand_packed(rng, 5, 96, "q8_0")
    tensors = {
        "blk.0.attn_norm.bias": (rng.standard_normal(7, dtype=np.float32), None),
        "token_embd.weight": (rng.standard_normal((9, 16), dtype=np.float32), None),
        "blk.0.attn_output.weight": (rng.standard_normal((4, 8), dtype=np.float32).astype(np.float16), None),
        "blk.0.ffn_up.weight": (packed_as_writer_array(q8), GT.Q8_0),
        "blk.0.attn_qkv.weight": (packed_as_writer_array(q4), GT.Q4_0),
    }
    meta = {"gpt2.block_count": 12, "general.name": "tiny", "gpt2.attention.layer_norm_epsilon": 1e-5,
            "tokenizer.ggml.tokens": ["a", "bc", "é"], "tokenizer.ggml.token_type": [1, 2, 3]}
    path = tmp_path / "t.gguf"
    write_file(path, tensors, meta)
    return path, tensors, meta, q4, q8


def test_tensor_table_matches_gguf_reader(sample):
    path, tensors, _, q4, q8 = sample
    g = load_gguf(path)
    ref = GGUFReader(str(path))
    assert g.version == 3 and g.alignment == 32
    assert g.order == [t.name for t in ref.tensors]
    for t in ref.tensors:
        mine = g.tensors[t.name]
        assert mine.ggml_type == int(t.tensor_type)
        assert list(mine.dims) == [int(x) for x in t.shape]
        np.testing.assert_array_equal(mine.raw(), np.ascontiguousarray(t.data).view(np.uint8).reshape(-1))
        assert (mine._ptr - g.tensors[g.order[0]]._ptr) % 32 == 0   # the 32-byte alignment rule
    assert g.tensors["blk.0.attn_qkv.weight"].shape == (6, 64)
    g.close()


def test_metadata_values(sample):
    path, _, meta, _, _ = sample
    g = load_gguf(path)
    assert g.metadata["general.architecture"] == "gpt2"
    assert g.metadata["gpt2.block_count"] == 12
    assert g.metadata["general.name"] == "tiny"
    assert abs(g.metadata["gpt2.attention.layer_norm_epsilon"] - 1e-5) < 1e-12
    assert g.metadata["tokenizer.ggml.tokens"] == ["a", "bc", "é"]
    assert g.metadata["tokenizer.ggml.token_type"] == [1, 2, 3]
    g.close()


def test_state_dict_keeps_quantised_blocks_packed(sample, oracle):
    path, tensors, _, q4, q8 = sample
    g = load_gguf(path)
    sd = gguf_to_state_dict(g)
    assert set(sd) == {"h.0.ln_1.bias", "wte.weight", "h.0.attn.c_proj.weight", "h.0.mlp.c_fc.weight", "h.0.attn.c_attn.weight"}
    p = sd["h.0.attn.c_attn.weight"]
    assert isinstance(p, S.Packed) and (p.ggml_type, p.rows, p.cols) == (2, 6, 64)
    np.testing.assert_array_equal(p.data, q4.data)
    np.testing.assert_array_equal(sd["h.0.mlp.c_fc.weight"].data, q8.data)
    np.testing.assert_array_equal(sd["wte.weight"], tensors["token_embd.weight"][0])
    assert sd["h.0.attn.c_proj.weight"].dtype == np.float16
    # what the reference would hold after its dequantising load (external/gguf/dequantize.lisp:40-53)
    want = oracle.dequant(8, q8.data, 5 * 96)
    got = oracle.dequant(8, sd["h.0.mlp.c_fc.weight"].data, 5 * 96)
    np.testing.assert_array_equal(got, want)
    g.close()


def test_custom_alignment(tmp_path):
    path = tmp_path / "a.gguf"
    write_file(path, {"x": (np.arange(5, dtype=np.float32), None), "y": (np.arange(3, dtype=np.float32), None)}, alignment=64)
    g = load_gguf(path)
    assert g.alignment == 64
    np.testing.assert_array_equal(g.tensors["y"].raw().view(np.float32), [0, 1, 2])
    assert (g.tensors["y"]._ptr - g.tensors["x"]._ptr) == 64
    g.close()


def test_remap_key_follows_the_reference_table():
    assert remap_key("blk.11.attn_qkv.weight") == "h.11.attn.c_attn.weight"
    assert remap_key("blk.3.ffn_down.bias") == "h.3.mlp.c_proj.bias"
    assert remap_key("output_norm.weight") == "ln_f.affine"
    assert remap_key("output.weight") == "lm_head.weight"
    assert remap_key("position_embd.weight") == "wpe.weight"


def test_malformed_files_are_rejected(tmp_path, sample):
    path = sample[0]
    blob = open(path, "rb").read()
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + blob[4:])
    with pytest.raises(B200Error) as e:
        load_gguf(bad)
    assert "magic" in str(e.value)
    bad.write_bytes(blob[:4] + struct.pack("<I", 1) + blob[8:])
    with pytest.raises(B200Error):
        load_gguf(bad)                       # version 1
    bad.write_bytes(blob[: len(blob) - 40])
    with pytest.raises(B200Error) as e:
        load_gguf(bad)                       # tensor data cut off
    assert "past the end" in str(e.value)
    bad.write_bytes(blob[:60])
    with pytest.raises(B200Error):
        load_gguf(bad)                       # cut inside the metadata
    with pytest.raises(B200Error):
        load_gguf(tmp_path / "missing.gguf")


def test_types_outside_the_supported_set_are_listed_but_not_served(tmp_path):
    path = tmp_path / "q.gguf"
    raw = np.zeros((2, 136), np.uint8)   # one IQ4_XS block (136 bytes) per row of 256 elements
    write_file(path, {"w": (raw, GT.IQ4_XS)})
    g = load_gguf(path)
    assert g.tensors["w"].ggml_type == int(GT.IQ4_XS) and g.tensors["w"].nbytes == -1
    with pytest.raises(B200Error):
        g.tensors["w"].raw()
    g.close()
