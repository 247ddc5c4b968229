"""SentencePiece and RWKV-trie tokenizers behind the common tokenizer interface."""
import io
import os

import pytest

from xllm_b200.utils.tokenizer import load_tokenizer
from xllm_b200.utils.tokenizer_extra import PyIncrementalDecoder, RwkvTokenizer, SentencePieceTokenizer


def test_rwkv_trie_longest_match_roundtrip(tmp_path):
    toks = ["a", "b", "ab", "abc", " ", "hello", "he", "l", "o", "é", "\n"]
    lines, idx = [], 1
    for b in range(256):                       # single bytes first, like the real vocabulary
        lit = repr(bytes([b]))
        lines.append(f"{idx} {lit} 1")
        idx += 1
    for t in toks:
        if len(t.encode()) > 1:
            lines.append(f"{idx} {t!r} {len(t.encode())}")
            idx += 1
    d = tmp_path / "m"
    d.mkdir()
    (d / "rwkv_vocab_v20230424.txt").write_text("\n".join(lines), encoding="utf-8")
    tw = load_tokenizer(str(d))
    tok = tw.impl
    assert isinstance(tok, RwkvTokenizer)
    ids = tw.encode("abcab hello é!")
    assert tok.id2bytes[ids[0]] == b"abc" and tok.id2bytes[ids[1]] == b"ab"     # longest match wins
    assert tw.decode(ids) == "abcab hello é!"
    inc = tw.incremental_decoder()
    assert isinstance(inc, PyIncrementalDecoder)
    streamed = "".join(inc.push(i) for i in tok.encode("héllo"))
    assert streamed == "héllo"


def test_sentencepiece_roundtrip(tmp_path):
    spm = pytest.importorskip("sentencepiece")
    corpus = tmp_path / "c.txt"
    corpus.write_text("\n".join(["the quick brown fox jumps over the lazy dog", "hello world of tokens",
                                 "paged attention keeps the cache in blocks"] * 50))
    d = tmp_path / "m"
    d.mkdir()
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(d / "tokenizer"), vocab_size=64,
                                   model_type="bpe", minloglevel=2)
    tw = load_tokenizer(str(d))
    assert isinstance(tw.impl, SentencePieceTokenizer) and tw.vocab_size == 64
    ids = tw.encode("the quick dog")
    assert tw.decode(ids) == "the quick dog"
    assert tw.token_to_id("▁the") >= 0
