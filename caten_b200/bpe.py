"""Byte-pair-encoding tokenizer: host-side counterpart of external/llm/bpe.lisp (the step either
side of the token loop, apps/gpt2/gpt2.lisp:101,108-109).  CPU work, no GPU involved.

`make_bpe_tokenizer` mirrors `make-bpe-tokenizer` (bpe.lisp:12-36), `BPETokenizer.encode/decode`
mirror `encode`/`decode` (bpe.lisp:86-114) and `gguf_to_bpe_tokenizer` mirrors
`gguf->bpe-tokenizer` (external/gguf/gguf-file.lisp:118-153).  The pre-tokenisation pattern is
the reference's (bpe.lisp:3).  One deliberate difference: a piece is mapped to the printable
alphabet byte by byte over its UTF-8 encoding, as GPT-2 and `tiktoken` (the reference's test
oracle, test-tokenizer.lisp:26-37) do, whereas the reference maps character codes
(bpe.lisp:97-99), which only coincides for code points below 128.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Sequence, Tuple

import regex

PAT = regex.compile(r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+")


def bytes_to_unicode() -> Dict[int, str]:
    """The reversible byte -> printable character table GPT-2 vocabularies are written in
    (what external/llm/utils.lisp:15-274 tabulates): printable Latin-1 bytes map to themselves,
    the remaining 68 bytes to code points 256.. in increasing byte order."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


BYTE2UNICODE = bytes_to_unicode()
UNICODE2BYTE = {c: b for b, c in BYTE2UNICODE.items()}


class BPETokenizer:
    def __init__(self, encoder: Dict[str, int], merges: Dict[Tuple[str, str], int]):
        self.encoder = encoder
        self.decoder = {i: t for t, i in encoder.items()}
        self.merges = merges
        self.cache: Dict[str, List[str]] = {}

    def bpe_split(self, token: str) -> List[str]:
        """`bpe-split` (bpe.lisp:45-84): repeatedly merge the adjacent pair with the lowest merge rank."""
        hit = self.cache.get(token)
        if hit is not None:
            return hit
        word = list(token)
        while len(word) > 1:
            ranked = [(self.merges.get((a, b)), i) for i, (a, b) in enumerate(zip(word, word[1:]))]
            ranked = [(r, i) for r, i in ranked if r is not None]
            if not ranked:
                break
            best = min(ranked)[0]
            first, second = next((a, b) for (a, b) in zip(word, word[1:]) if self.merges.get((a, b)) == best)
            out, i = [], 0
            while i < len(word):
                if i < len(word) - 1 and word[i] == first and word[i + 1] == second:
                    out.append(first + second)
                    i += 2
                else:
                    out.append(word[i])
                    i += 1
            word = out
        self.cache[token] = word
        return word

    def encode(self, text: str) -> List[int]:
        ids: List[int] = []
        for piece in PAT.findall(text):
            mapped = "".join(BYTE2UNICODE[b] for b in piece.encode("utf-8"))
            for t in self.bpe_split(mapped):
                ids.append(self.encoder.get(t, 0))   # unknown piece -> id 0, as bpe.lisp:101 does
        return ids

    def decode(self, ids: Iterable[int]) -> str:
        text = "".join(self.decoder.get(int(i), "") for i in ids)
        return bytes(UNICODE2BYTE.get(c, 0x20) for c in text).decode("utf-8", errors="replace")


def make_bpe_tokenizer(tokens: Sequence[str], merges: Sequence[str]) -> BPETokenizer:
    """``tokens``: vocabulary, index = id.  ``merges``: "left right" strings, index = rank."""
    encoder = {t: i for i, t in enumerate(tokens)}
    ranks = {}
    for r, m in enumerate(merges):
        a, _, b = m.partition(" ")
        if a and b:
            ranks[(a, b)] = r
    return BPETokenizer(encoder, ranks)


def make_bpe_tokenizer_from_text(tokens: str, merges: str) -> BPETokenizer:
    """`make-bpe-tokenizer` on its own argument form (bpe.lisp:12-36): ``tokens`` is one string of
    tokens separated by single spaces, ``merges`` one string of "left right" lines; as there, the
    piece before the first separator of each is dropped (both files start with a separator)."""
    tok = tokens.split(" ")[1:]
    if tok and tok[-1].endswith("\n"):
        tok[-1] = tok[-1].rstrip("\n")
    lines = [" ".join(part for part in line.split(" ") if part) for line in merges.split("\n")[1:]]
    return make_bpe_tokenizer(tok, [ln for ln in lines if ln])


def gguf_to_bpe_tokenizer(gguf, metadata_tokens: str = "tokenizer.ggml.tokens",
                          metadata_merges: str = "tokenizer.ggml.merges") -> BPETokenizer:
    md = gguf.metadata
    if metadata_tokens not in md or metadata_merges not in md:
        raise KeyError(f"the GGUF file has no tokenizer metadata ({metadata_tokens}, {metadata_merges})")
    return make_bpe_tokenizer(md[metadata_tokens], md[metadata_merges])
