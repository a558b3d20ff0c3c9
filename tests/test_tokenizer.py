"""CPU tests of the BPE tokenizer against `tiktoken`, the checker the reference's own tokenizer
test uses (source/test-suite/external/test-tokenizer.lisp:26-37): on the GPT-2 vocabulary files
that test loads (kept compressed under tests/golden/gpt2_tokenizer/) with its three sentences, and
on a small vocabulary trained here on a fixed text (edge cases of the merge rule)."""
import collections
import gzip
import os

import numpy as np
import pytest

from caten_b200.bpe import (BYTE2UNICODE, PAT, UNICODE2BYTE, gguf_to_bpe_tokenizer, make_bpe_tokenizer,
                            make_bpe_tokenizer_from_text)

tiktoken = pytest.importorskip("tiktoken")

CORPUS = (
    "the quick brown fox jumps over the lazy dog. The dog didn't mind; it's used to foxes. "
    "We'll count: 1, 22, 333 and 4444 sheep, then they've gone home. I'm sure she'd say the same. "
    "Tokenizers split text into pieces, and pieces into bytes; bytes merge back into pieces. "
    "café naïve über straße 日本語 текст "
    "tabs\tand\nnewlines\n\n  and   runs of   spaces  .\n"
) * 3


def train(n_merges):
    """Plain BPE training over the pre-tokenised corpus; returns (tokens, merges) in GGUF's form."""
    words = collections.Counter(tuple(BYTE2UNICODE[b] for b in piece.encode("utf-8")) for piece in PAT.findall(CORPUS))
    tokens = [BYTE2UNICODE[b] for b in range(256)]
    merges = []
    for _ in range(n_merges):
        pairs = collections.Counter()
        for w, c in words.items():
            for a, b in zip(w, w[1:]):
                pairs[(a, b)] += c
        if not pairs:
            break
        (a, b), _ = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))
        merges.append(f"{a} {b}")
        tokens.append(a + b)
        new = collections.Counter()
        for w, c in words.items():
            out, i = [], 0
            while i < len(w):
                if i < len(w) - 1 and w[i] == a and w[i + 1] == b:
                    out.append(a + b); i += 2
                else:
                    out.append(w[i]); i += 1
            new[tuple(out)] += c
        words = new
    return tokens, merges


@pytest.fixture(scope="module")
def pair():
    tokens, merges = train(300)
    mine = make_bpe_tokenizer(tokens, merges)
    ranks = {bytes(UNICODE2BYTE[c] for c in t): i for i, t in enumerate(tokens)}
    theirs = tiktoken.Encoding("tiny", pat_str=PAT.pattern, mergeable_ranks=ranks, special_tokens={})
    return mine, theirs, tokens, merges


SENTENCES = [
    "the quick brown fox",
    "The dog didn't mind, it's fine; we'll see, they've gone, I'm here, she'd know, you're right.",
    "Count 1 22 333 4444 55555 sheep",
    "  leading spaces and trailing   ",
    "tabs\tand\nnewlines\n\n\n  mixed \t \n",
    "café naïve straße 日本語 текст \U0001f600",
    "symbols!!! ... ??? $%^&*() [brackets] {braces} <tags/>",
    "unseenwordsthatneverappearedinthetrainingtext zzzqqq",
    "",
    " ",
    "a",
]


@pytest.mark.parametrize("text", SENTENCES)
def test_encode_matches_tiktoken(pair, text):
    mine, theirs, _, _ = pair
    assert mine.encode(text) == theirs.encode(text)


@pytest.mark.parametrize("text", SENTENCES)
def test_decode_round_trip_and_matches_tiktoken(pair, text):
    mine, theirs, _, _ = pair
    ids = theirs.encode(text)
    assert mine.decode(ids) == theirs.decode(ids) == text


def test_random_byte_strings_match_tiktoken(pair):
    mine, theirs, _, _ = pair
    rng = np.random.Generator(np.random.PCG64(5))
    alphabet = list("abcdefghij  \n\t'.,0123456789ABCéü日т!?-")
    for _ in range(200):
        text = "".join(rng.choice(alphabet, size=int(rng.integers(1, 60))))
        ids = mine.encode(text)
        assert ids == theirs.encode(text)
        assert mine.decode(ids) == text


def test_merges_apply_in_rank_order_not_left_to_right():
    # "b c" outranks "a b": the word abc must become a + bc, as bpe-split's lowest-rank rule says
    tokens = ["a", "b", "c", "bc", "ab"]
    t = make_bpe_tokenizer(tokens, ["b c", "a b"])
    assert t.encode("abc") == [0, 3]
    t = make_bpe_tokenizer(tokens, ["a b", "b c"])
    assert t.encode("abc") == [4, 2]
    # every occurrence of the chosen pair merges in one pass
    assert t.encode("abab") == [4, 4]


def test_unknown_piece_maps_to_id_zero():
    t = make_bpe_tokenizer(["<unk>", "a"], [])
    assert t.encode("ab") == [1, 0]


def test_tokenizer_from_gguf_metadata(tmp_path, pair):
    gguf = pytest.importorskip("gguf")
    from caten_b200.gguf import load_gguf
    mine, theirs, tokens, merges = pair
    path = tmp_path / "tok.gguf"
    w = gguf.GGUFWriter(str(path), "gpt2")
    w.add_array("tokenizer.ggml.tokens", tokens)
    w.add_array("tokenizer.ggml.merges", merges)
    w.add_tensor("x", np.zeros(4, np.float32))
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()
    g = load_gguf(path)
    t = gguf_to_bpe_tokenizer(g)
    text = "The dog didn't count 333 sheep at the café."
    assert t.encode(text) == theirs.encode(text) and t.decode(t.encode(text)) == text
    g.close()
    path2 = tmp_path / "none.gguf"
    w = gguf.GGUFWriter(str(path2), "gpt2")
    w.add_tensor("x", np.zeros(4, np.float32))
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()
    g = load_gguf(path2)
    with pytest.raises(KeyError):
        gguf_to_bpe_tokenizer(g)
    g.close()


# ---- the reference's own vocabulary and sentences ---------------------------------------------------
GPT2_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gpt2_tokenizer")


@pytest.fixture(scope="module")
def gpt2_pair():
    def read(name):
        with gzip.open(os.path.join(GPT2_DIR, name + ".gz"), "rt", encoding="utf-8", newline="") as f:
            return f.read()
    mine = make_bpe_tokenizer_from_text(read("tokens.txt"), read("merges.txt"))   # make-bpe-gpt2, test-tokenizer.lisp:19-24
    assert len(mine.encoder) == 50257 and len(mine.merges) == 50000
    special = {"<|endoftext|>": mine.encoder["<|endoftext|>"]}
    ranks = {bytes(UNICODE2BYTE[c] for c in t): i for t, i in mine.encoder.items() if t not in special}
    theirs = tiktoken.Encoding("gpt2-offline", pat_str=PAT.pattern, mergeable_ranks=ranks, special_tokens=special)
    return mine, theirs


REFERENCE_SENTENCES = ["Say hello to me", "Hello world", "What is the answer to the life, the world, and everything?"]   # test-tokenizer.lisp:35-37


@pytest.mark.parametrize("text", REFERENCE_SENTENCES + SENTENCES)
def test_gpt2_vocabulary_matches_tiktoken(gpt2_pair, text):
    mine, theirs = gpt2_pair
    ids = mine.encode(text)
    assert ids == theirs.encode(text)
    assert mine.decode(ids) == theirs.decode(ids) == text


def test_gpt2_vocabulary_known_ids(gpt2_pair):
    """Ids of GPT-2's published vocabulary for the second reference sentence: a fixed point that does
    not depend on tiktoken being importable in the same way elsewhere."""
    mine, _ = gpt2_pair
    assert mine.encode("Hello world") == [15496, 995]
    assert mine.decode([15496, 995]) == "Hello world"
