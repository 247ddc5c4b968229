"""Tokenizers beyond byte-level BPE: SentencePiece models and the RWKV "world" trie vocabulary.

Parity: `SentencePieceTokenizer`, `RWKVTokenizer` and their selection in `TokenizerFactory`
(xllm/core/framework/tokenizer/{sentencepiece_tokenizer,rwkv_tokenizer,tokenizer_factory}.cpp).
Both expose the interface of the native BPE tokenizer (`encode`, `decode`, `token_to_id`,
`vocab_size`), so `TokenizerWrapper` and the serving front end use them unchanged.
"""
from __future__ import annotations

import ast
from typing import Dict, List, Optional


class SentencePieceTokenizer:
    def __init__(self, model_file: str, add_bos: bool = False, add_eos: bool = False):
        import sentencepiece as spm
        self.sp = spm.SentencePieceProcessor(model_file=model_file)
        self.add_bos, self.add_eos = add_bos, add_eos
        self.bos_id, self.eos_id = self.sp.bos_id(), self.sp.eos_id()

    @property
    def vocab_size(self) -> int:
        return self.sp.get_piece_size()

    def encode(self, text: str, add_special: bool = False) -> List[int]:
        ids = list(self.sp.encode(text))
        if add_special and self.add_bos and self.bos_id >= 0:
            ids.insert(0, self.bos_id)
        if add_special and self.add_eos and self.eos_id >= 0:
            ids.append(self.eos_id)
        return ids

    def decode(self, ids, skip_special: bool = True) -> str:
        ids = [int(i) for i in ids]
        if skip_special:
            ids = [i for i in ids if not self.sp.is_control(i)]
        return self.sp.decode(ids)

    def token_to_id(self, tok: str) -> int:
        i = self.sp.piece_to_id(tok)
        return i if self.sp.id_to_piece(i) == tok else -1

    def id_to_token(self, i: int) -> str:
        return self.sp.id_to_piece(int(i))


class _TrieNode:
    __slots__ = ("next", "token")

    def __init__(self):
        self.next: Dict[int, "_TrieNode"] = {}
        self.token = -1


class RwkvTokenizer:
    """Greedy longest-match over a byte trie.  Vocabulary file: one token per line,
    `<id> <python string or bytes literal> <byte length>`."""

    def __init__(self, vocab_file: Optional[str] = None, tokens: Optional[Dict[int, bytes]] = None):
        self.id2bytes: Dict[int, bytes] = {}
        if vocab_file is not None:
            with open(vocab_file, "r", encoding="utf-8") as f:
                for line in f:
                    line = line.rstrip("\n")
                    if not line:
                        continue
                    sp1, sp2 = line.index(" "), line.rindex(" ")
                    idx = int(line[:sp1])
                    val = ast.literal_eval(line[sp1 + 1:sp2])
                    b = val.encode("utf-8") if isinstance(val, str) else val
                    assert len(b) == int(line[sp2 + 1:]), line
                    self.id2bytes[idx] = b
        if tokens:
            self.id2bytes.update(tokens)
        self.root = _TrieNode()
        for idx, b in self.id2bytes.items():
            n = self.root
            for c in b:
                n = n.next.setdefault(c, _TrieNode())
            n.token = idx
        self.bytes2id = {b: i for i, b in self.id2bytes.items()}

    @property
    def vocab_size(self) -> int:
        return max(self.id2bytes) + 1 if self.id2bytes else 0

    def encode(self, text: str, add_special: bool = False) -> List[int]:
        data = text.encode("utf-8")
        out, i, n = [], 0, len(data)
        while i < n:
            node, best, best_end, j = self.root, -1, i, i
            while j < n and data[j] in node.next:
                node = node.next[data[j]]
                j += 1
                if node.token >= 0:
                    best, best_end = node.token, j
            if best < 0:
                raise ValueError(f"byte {data[i]!r} at offset {i} is not in the vocabulary")
            out.append(best)
            i = best_end
        return out

    def decode(self, ids, skip_special: bool = True) -> str:
        return b"".join(self.id2bytes.get(int(i), b"") for i in ids if int(i) != 0 or not skip_special).decode(
            "utf-8", errors="replace")

    def token_to_id(self, tok: str) -> int:
        return self.bytes2id.get(tok.encode("utf-8"), -1)


class PyIncrementalDecoder:
    """Streaming detokeniser for tokenizers without the native incremental decoder: emits the text
    that became stable (no dangling partial UTF-8 sequence) after each token."""

    def __init__(self, tok, skip_special=True):
        self.tok, self.skip, self.ids, self.sent = tok, skip_special, [], 0

    def push(self, token_id: int) -> str:
        self.ids.append(int(token_id))
        text = self.tok.decode(self.ids, self.skip)
        if text.endswith("�"):
            return ""
        out, self.sent = text[self.sent:], len(text)
        return out


class ClipBpeTokenizer:
    """CLIP's text tokenizer from its original file pair (`vocab.json`, `merges.txt`): lower-cased, whitespace
    collapsed, split by CLIP's pattern, bytes mapped to printable code points, merges applied with the
    end-of-word marker `</w>` on a word's last symbol.  The tokenizer of the first text encoder of the
    diffusion pipelines (xllm/models/dit/ tokenizers of the reference)."""

    def __init__(self, vocab_file: str, merges_file: str):
        import json

        import regex
        with open(vocab_file, encoding="utf-8") as f:
            self.vocab: Dict[str, int] = json.load(f)
        self.inv = {i: t for t, i in self.vocab.items()}
        with open(merges_file, encoding="utf-8") as f:
            lines = [l.rstrip("\n") for l in f if l.strip() and not l.startswith("#version")]
        self.ranks = {tuple(l.split()): i for i, l in enumerate(lines)}
        bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
        cs = bs[:]
        n = 0
        for b in range(256):
            if b not in bs:
                bs.append(b)
                cs.append(256 + n)
                n += 1
        self.byte_enc = {b: chr(c) for b, c in zip(bs, cs)}
        self.byte_dec = {v: k for k, v in self.byte_enc.items()}
        self.pat = regex.compile(r"<\|startoftext\|>|<\|endoftext\|>|'s|'t|'re|'ve|'m|'ll|'d|[\p{L}]+|[\p{N}]|[^\s\p{L}\p{N}]+",
                                 regex.IGNORECASE)
        self.bos_id = self.vocab.get("<|startoftext|>", -1)
        self.eos_id = self.vocab.get("<|endoftext|>", -1)
        self.cache: Dict[str, List[str]] = {}

    @property
    def vocab_size(self) -> int:
        return len(self.vocab)

    def _bpe(self, token: str) -> List[str]:
        if token in self.cache:
            return self.cache[token]
        word = list(token[:-1]) + [token[-1] + "</w>"]
        while len(word) > 1:
            pairs = [(self.ranks.get((a, b), 1 << 30), i) for i, (a, b) in enumerate(zip(word, word[1:]))]
            rank, _ = min(pairs)
            if rank == 1 << 30:
                break
            first, second = next(p for p, r in self.ranks.items() if r == rank)
            out, i = [], 0
            while i < len(word):
                if i + 1 < len(word) and word[i] == first and word[i + 1] == second:
                    out.append(first + second)
                    i += 2
                else:
                    out.append(word[i])
                    i += 1
            word = out
        self.cache[token] = word
        return word

    def encode(self, text: str, add_special: bool = False) -> List[int]:
        text = " ".join(text.split()).strip().lower()
        ids: List[int] = []
        for tok in self.pat.findall(text):
            if tok in ("<|startoftext|>", "<|endoftext|>"):
                ids.append(self.vocab[tok])
                continue
            mapped = "".join(self.byte_enc[b] for b in tok.encode("utf-8"))
            unk = self.eos_id if self.eos_id >= 0 else 0
            ids.extend(self.vocab.get(piece, unk) for piece in self._bpe(mapped))
        if add_special:
            ids = ([self.bos_id] if self.bos_id >= 0 else []) + ids + ([self.eos_id] if self.eos_id >= 0 else [])
        return ids

    def decode(self, ids, skip_special: bool = True) -> str:
        toks = [self.inv.get(int(i), "") for i in ids]
        if skip_special:
            toks = [t for t in toks if t not in ("<|startoftext|>", "<|endoftext|>")]
        words = "".join(toks).split("</w>")
        return " ".join(bytearray(self.byte_dec[c] for c in w if c in self.byte_dec).decode("utf-8", errors="replace")
                        for w in words).strip()

    def token_to_id(self, tok: str) -> int:
        return self.vocab.get(tok, -1)

    def id_to_token(self, i: int) -> str:
        return self.inv.get(int(i), "")
