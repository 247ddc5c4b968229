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


def test_clip_bpe_matches_huggingface(tmp_path):
    """CLIP's tokenizer from vocab.json + merges.txt against transformers' slow CLIPTokenizer."""
    import json

    transformers = pytest.importorskip("transformers")
    from xllm_b200.utils.tokenizer import load_tokenizer
    from xllm_b200.utils.tokenizer_extra import ClipBpeTokenizer
    probe = ClipBpeTokenizer.__new__(ClipBpeTokenizer)
    # a small vocabulary: all byte symbols (plain and end-of-word), a few merges, the two specials
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    cs, n = bs[:], 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    symbols = [chr(c) for c in cs]
    merges = [("h", "o"), ("ho", "u"), ("hou", "se</w>"), ("s", "e</w>"), ("r", "e"), ("re", "d</w>"), ("t", "h"), ("th", "e</w>"),
              ("a</w>",) * 1 + ("x",)][:-1]
    vocab = {}
    for s in symbols:
        vocab[s] = len(vocab)
    for s in symbols:
        vocab[s + "</w>"] = len(vocab)
    for a, b in merges:
        vocab[a + b] = len(vocab)
    vocab["<|startoftext|>"] = len(vocab)
    vocab["<|endoftext|>"] = len(vocab)
    (tmp_path / "vocab.json").write_text(json.dumps(vocab))
    (tmp_path / "merges.txt").write_text("#version: 0.2\n" + "\n".join(f"{a} {b}" for a, b in merges) + "\n")
    (tmp_path / "tokenizer_config.json").write_text(json.dumps({"tokenizer_class": "CLIPTokenizer"}))
    hf = transformers.CLIPTokenizer(str(tmp_path / "vocab.json"), str(tmp_path / "merges.txt"))
    mine = load_tokenizer(str(tmp_path))
    assert isinstance(mine.impl, ClipBpeTokenizer)
    for text in ("The red house", "  a  RED   house, the sea!  ", "it's 42 houses: théâtre", "x"):
        want = hf(text, add_special_tokens=False)["input_ids"]
        assert mine.encode(text) == want, text
    assert mine.impl.encode("the house", add_special=True) == hf("the house")["input_ids"]
    assert mine.decode(mine.encode("the red house")) == "the red house"
