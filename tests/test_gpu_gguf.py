"""GPU test of the file path: GGUF written by the Python `gguf` package -> C parser -> packed
upload -> GPT-2 decode, compared with the oracle fed by `gguf.quants.dequantize` of the same file."""
import numpy as np
import pytest

from caten_b200 import synthetic as S
from caten_b200.gguf import load_gguf, remap_key
from caten_b200.gpt2 import gpt2_generate, make_gpt2_from_gguf

pytestmark = pytest.mark.gpu
gguf = pytest.importorskip("gguf")

INVERSE = {"wte.weight": "token_embd.weight", "wpe.weight": "position_embd.weight", "ln_f.affine": "output_norm.weight",
           "ln_f.bias": "output_norm.bias", "lm_head.weight": "output.weight"}
LAYER = {"ln_1.affine": "attn_norm.weight", "ln_1.bias": "attn_norm.bias", "attn.c_attn.weight": "attn_qkv.weight",
         "attn.c_attn.bias": "attn_qkv.bias", "attn.c_proj.weight": "attn_output.weight", "attn.c_proj.bias": "attn_output.bias",
         "ln_2.affine": "ffn_norm.weight", "ln_2.bias": "ffn_norm.bias", "mlp.c_fc.weight": "ffn_up.weight",
         "mlp.c_fc.bias": "ffn_up.bias", "mlp.c_proj.weight": "ffn_down.weight", "mlp.c_proj.bias": "ffn_down.bias"}


def gguf_name(key):
    if key in INVERSE:
        return INVERSE[key]
    _, l, rest = key.split(".", 2)
    return f"blk.{l}.{LAYER[rest]}"


@pytest.mark.parametrize("wtype", ["q4_0", "q8_0"])
def test_gpt2_from_gguf_file(rt, oracle, tmp_path, wtype):
    from gguf import GGMLQuantizationType as GT
    from gguf import GGUFReader, GGUFWriter
    from gguf.quants import dequantize
    p = S.GPT2Params(n_layers=2, n_heads=2, dim=128, vocab_size=515)
    T = 40
    sd = S.synth_state_dict(p, wtype, seed=21, max_seq_len=T, trivial_affine=False, weight_std=0.08)
    path = tmp_path / "gpt2-tiny.gguf"
    w = GGUFWriter(str(path), "gpt2")
    w.add_uint32("gpt2.block_count", p.n_layers)
    w.add_uint32("gpt2.embedding_length", p.dim)
    w.add_uint32("gpt2.attention.head_count", p.n_heads)
    w.add_uint32("gpt2.context_length", T)
    w.add_float32("gpt2.attention.layer_norm_epsilon", 1e-5)
    for k, v in sd.items():
        assert remap_key(gguf_name(k)) == k
        if isinstance(v, S.Packed):
            bb = S.BLOCK_BYTES[v.ggml_type]
            w.add_tensor(gguf_name(k), v.data.reshape(v.rows, v.cols // 32 * bb), raw_dtype=GT(v.ggml_type))
        else:
            w.add_tensor(gguf_name(k), v)
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()

    # oracle weights: what the reference's loader would hold, via the gguf package's own dequantiser
    fsd = {}
    for t in GGUFReader(str(path)).tensors:
        a = np.asarray(t.data)
        if t.tensor_type in (GT.Q4_0, GT.Q8_0):
            a = dequantize(a, t.tensor_type)
        fsd[remap_key(t.name)] = np.ascontiguousarray(a, dtype=np.float32).reshape([int(x) for x in reversed(t.shape)])
    B = 3
    prompt = S.synth_prompts(B, 6, p.vocab_size, seed=4)
    ref = oracle.GPT2(p.n_layers, p.dim, p.n_heads, p.vocab_size, T, B, fsd)
    m = make_gpt2_from_gguf(str(path), runtime=rt, batch=B)
    assert (m.params.n_layers, m.params.n_heads, m.params.dim, m.params.vocab_size) == (p.n_layers, p.n_heads, p.dim, p.vocab_size)
    assert abs(m.params.norm_eps - 1e-5) < 1e-9 and m.max_seq_len == T
    tokens, pos = prompt, 0
    for _ in range(5):
        ids_ref, lg_ref = ref.step(tokens[:, pos:], pos)
        ids = m.forward(tokens[:, pos:], tokens.shape[1] - pos, pos)
        assert np.abs(m.logits() - lg_ref).max() <= 1e-3
        top2 = np.sort(lg_ref, axis=1)[:, -2:]
        ok = (top2[:, 1] - top2[:, 0]) > 1e-4
        np.testing.assert_array_equal(ids[ok], ids_ref[ok])
        pos = tokens.shape[1]
        tokens = np.concatenate([tokens, ids_ref.reshape(-1, 1)], 1)
    # a weight uploaded straight from the mapping dequantises to the gguf package's values, bit for bit
    g = load_gguf(str(path))
    h = g.upload("blk.1.ffn_up.weight", rt)
    np.testing.assert_array_equal(h.dequantize().view(np.uint32), fsd["h.1.mlp.c_fc.weight"].view(np.uint32))
    h.close(); g.close(); m.close(); ref.close()


def test_text_in_text_out_from_one_gguf_file(rt, tmp_path):
    """The whole caller-side flow of apps/gpt2/gpt2.lisp:97-113 from one file: tokenizer metadata ->
    ids -> greedy loop on the GPU -> text.  The weights are random, so only the plumbing is checked:
    the prompt survives the round trip and every generated id decodes."""
    from gguf import GGMLQuantizationType as GT
    from gguf import GGUFWriter
    from caten_b200.bpe import BYTE2UNICODE, gguf_to_bpe_tokenizer
    tokens = [BYTE2UNICODE[b] for b in range(256)] + ["th", "the", "Ġthe", "he", "ll", "hell", "hello"]
    merges = ["t h", "th e", "Ġ the", "h e", "l l", "he ll", "hell o"]
    p = S.GPT2Params(n_layers=1, n_heads=2, dim=128, vocab_size=len(tokens))
    T = 48
    sd = S.synth_state_dict(p, "q8_0", seed=3, max_seq_len=T, trivial_affine=False, weight_std=0.08)
    path = tmp_path / "tiny-text.gguf"
    w = GGUFWriter(str(path), "gpt2")
    w.add_uint32("gpt2.block_count", p.n_layers)
    w.add_uint32("gpt2.embedding_length", p.dim)
    w.add_uint32("gpt2.attention.head_count", p.n_heads)
    w.add_uint32("gpt2.context_length", T)
    w.add_array("tokenizer.ggml.tokens", tokens)
    w.add_array("tokenizer.ggml.merges", merges)
    for k, v in sd.items():
        if isinstance(v, S.Packed):
            w.add_tensor(gguf_name(k), v.data.reshape(v.rows, v.cols // 32 * S.BLOCK_BYTES[v.ggml_type]), raw_dtype=GT(v.ggml_type))
        else:
            w.add_tensor(gguf_name(k), v)
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()

    g = load_gguf(str(path))
    tok = gguf_to_bpe_tokenizer(g)
    g.close()
    ids = tok.encode("hello the")
    assert ids == [tokens.index("hello"), tokens.index("Ġthe")]
    m = make_gpt2_from_gguf(str(path), runtime=rt, batch=1)
    out = gpt2_generate(m, [ids], max_length=12)
    assert out.shape == (1, len(ids) + 12) and out.min() >= 0 and out.max() < len(tokens)
    text = tok.decode(out[0])
    assert isinstance(text, str) and tok.decode(out[0, :len(ids)]) == "hello the"
    m.close()


def test_gpt2_from_gguf_with_quantised_embeddings_and_tied_output(rt, oracle, tmp_path):
    """What llama.cpp's quantiser writes for GPT-2: token_embd.weight in Q8_0, position_embd.weight in
    F16, and no output.weight (the output matrix is the token embedding).  The reference dequantises
    such tables at load (external/gguf/dequantize.lisp:27-53); here they are expanded on the device."""
    from gguf import GGMLQuantizationType as GT
    from gguf import GGUFWriter
    from gguf.quants import dequantize
    p = S.GPT2Params(n_layers=1, n_heads=2, dim=128, vocab_size=300)
    T = 24
    sd = S.synth_state_dict(p, "q8_0", seed=31, max_seq_len=T, trivial_affine=False, weight_std=0.08)
    rng = np.random.Generator(np.random.PCG64(32))
    wte = S._rand_packed(rng, p.vocab_size, p.dim, "q8_0", 0.08)
    wpe16 = sd["wpe.weight"].astype(np.float16)
    del sd["lm_head.weight"]
    path = tmp_path / "gpt2-tied.gguf"
    w = GGUFWriter(str(path), "gpt2")
    w.add_uint32("gpt2.block_count", p.n_layers)
    w.add_uint32("gpt2.embedding_length", p.dim)
    w.add_uint32("gpt2.attention.head_count", p.n_heads)
    w.add_uint32("gpt2.context_length", T)
    for k, v in sd.items():
        if k == "wte.weight":
            w.add_tensor(gguf_name(k), wte.data.reshape(wte.rows, wte.cols // 32 * 34), raw_dtype=GT.Q8_0)
        elif k == "wpe.weight":
            w.add_tensor(gguf_name(k), wpe16)
        elif isinstance(v, S.Packed):
            w.add_tensor(gguf_name(k), v.data.reshape(v.rows, v.cols // 32 * S.BLOCK_BYTES[v.ggml_type]), raw_dtype=GT(v.ggml_type))
        else:
            w.add_tensor(gguf_name(k), v)
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()

    fsd = {k: (oracle.dequant(v.ggml_type, v.data, v.rows * v.cols).reshape(v.rows, v.cols) if isinstance(v, S.Packed) else v)
           for k, v in sd.items()}
    fsd["wte.weight"] = dequantize(wte.data.reshape(-1, 34), GT.Q8_0).reshape(p.vocab_size, p.dim)
    fsd["lm_head.weight"] = fsd["wte.weight"]
    fsd["wpe.weight"] = wpe16.astype(np.float32)
    B = 2
    prompt = S.synth_prompts(B, 5, p.vocab_size, seed=6)
    ref = oracle.GPT2(p.n_layers, p.dim, p.n_heads, p.vocab_size, T, B, fsd)
    m = make_gpt2_from_gguf(str(path), runtime=rt, batch=B)
    tokens, pos = prompt, 0
    for _ in range(4):
        ids_ref, lg_ref = ref.step(tokens[:, pos:], pos)
        m.forward(tokens[:, pos:], tokens.shape[1] - pos, pos)
        assert np.abs(m.logits() - lg_ref).max() <= 1e-3
        pos = tokens.shape[1]
        tokens = np.concatenate([tokens, ids_ref.reshape(-1, 1)], 1)
    m.close(); ref.close()
    # a position table shorter than the requested context is refused, not read past its end
    with pytest.raises(ValueError):
        make_gpt2_from_gguf(str(path), runtime=rt, batch=1, max_seq_len=T + 8)
