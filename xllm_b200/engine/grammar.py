"""Constrained decoding: "the output is one JSON object".

Parity: `JsonObjectGrammar` and the token bitmask / filter-mask path of the sampler
(xllm/core/framework/sampling/json_object_grammar.cpp, sampler.cpp).  The grammar is an
incremental character-level validator (a pushdown automaton over JSON's value / object / array /
string / number / literal states) that answers "is this still a prefix of a JSON object?" after
every character.  A token is admissible when all of its characters keep the prefix valid.

Instead of testing the whole vocabulary every step, the filter looks at the `top_n` highest logits
of a constrained row (one device top-k), keeps the admissible ones and masks the rest of the row
to -inf, so the normal device sampler then samples among admissible tokens only.  When none of the
top tokens is admissible the filter falls back to a scan of the vocabulary in logit order.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

_WS = " \t\n\r"
_DIGITS = "0123456789"


class JsonObjectValidator:
    """Feed characters; `feed` returns False (and leaves the state untouched) when the character
    cannot extend a prefix of a single JSON object.  `complete` is True once the object closed."""

    __slots__ = ("stack", "state", "lit", "complete", "num")

    def __init__(self):
        self.stack: List[str] = []     # '{' or '['
        self.state = "start"           # what may come next
        self.lit = ""                  # rest of a literal being matched (rue / alse / ull)
        self.num = ""                  # number sub-state
        self.complete = False

    def copy(self):
        c = JsonObjectValidator()
        c.stack, c.state, c.lit, c.num, c.complete = list(self.stack), self.state, self.lit, self.num, self.complete
        return c

    # -- helpers
    def _after_value(self):
        if not self.stack:
            self.state, self.complete = "end", True
        else:
            self.state = "obj_next" if self.stack[-1] == "{" else "arr_next"

    def _start_value(self, ch) -> bool:
        if ch == "{":
            self.stack.append("{")
            self.state = "obj_first"
        elif ch == "[":
            self.stack.append("[")
            self.state = "arr_first"
        elif ch == '"':
            self.state = "str"
        elif ch in "tfn":
            self.lit = {"t": "rue", "f": "alse", "n": "ull"}[ch]
            self.state = "lit"
        elif ch == "-":
            self.num, self.state = "-", "num"
        elif ch in _DIGITS:
            self.num, self.state = ("0" if ch == "0" else "int"), "num"
        else:
            return False
        return True

    def feed(self, ch: str) -> bool:
        s = self.state
        if s == "end":
            return ch in _WS
        if s == "start":
            if ch in _WS:
                return True
            if ch != "{":
                return False
            return self._start_value(ch)
        if s in ("str", "key"):
            if ch == "\\":
                self.state = s + "_esc"
            elif ch == '"':
                if s == "key":
                    self.state = "colon"
                else:
                    self._after_value()
            elif ch < " ":
                return False
            return True
        if s in ("str_esc", "key_esc"):
            if ch in '"\\/bfnrt':
                self.state = s[:-4]
            elif ch == "u":
                self.state, self.lit = s[:-4] + "_u", "4"
            else:
                return False
            return True
        if s in ("str_u", "key_u"):
            if ch not in "0123456789abcdefABCDEF":
                return False
            n = int(self.lit) - 1
            self.lit = str(n)
            if n == 0:
                self.state = s[:-2]
            return True
        if s == "lit":
            if ch != self.lit[0]:
                return False
            self.lit = self.lit[1:]
            if not self.lit:
                self._after_value()
            return True
        if s == "num":
            n = self.num
            if n == "-":
                if ch == "0":
                    self.num = "0"
                elif ch in _DIGITS:
                    self.num = "int"
                else:
                    return False
                return True
            if n in ("0", "int"):
                if ch in _DIGITS and n == "int":
                    return True
                if ch == ".":
                    self.num = "dot"
                    return True
                if ch in "eE":
                    self.num = "e"
                    return True
            elif n == "dot":
                if ch in _DIGITS:
                    self.num = "frac"
                    return True
                return False
            elif n == "frac":
                if ch in _DIGITS:
                    return True
                if ch in "eE":
                    self.num = "e"
                    return True
            elif n == "e":
                if ch in "+-":
                    self.num = "esign"
                    return True
                if ch in _DIGITS:
                    self.num = "exp"
                    return True
                return False
            elif n == "esign":
                if ch in _DIGITS:
                    self.num = "exp"
                    return True
                return False
            elif n == "exp":
                if ch in _DIGITS:
                    return True
            if n in ("0", "int", "frac", "exp"):   # the number ended: re-read ch as a follower
                self._after_value()
                return self.feed(ch)
            return False
        if ch in _WS:
            return True
        if s == "obj_first":
            if ch == "}":
                self.stack.pop()
                self._after_value()
                return True
            if ch == '"':
                self.state = "key"
                return True
            return False
        if s == "obj_key":
            if ch == '"':
                self.state = "key"
                return True
            return False
        if s == "colon":
            if ch == ":":
                self.state = "value"
                return True
            return False
        if s == "value":
            return self._start_value(ch)
        if s == "arr_first":
            if ch == "]":
                self.stack.pop()
                self._after_value()
                return True
            return self._start_value(ch)
        if s == "obj_next":
            if ch == ",":
                self.state = "obj_key"
                return True
            if ch == "}":
                self.stack.pop()
                self._after_value()
                return True
            return False
        if s == "arr_next":
            if ch == ",":
                self.state = "value"
                return True
            if ch == "]":
                self.stack.pop()
                self._after_value()
                return True
            return False
        return False

    def feed_text(self, text: str) -> bool:
        """All-or-nothing: the state advances only if every character is accepted."""
        trial = self.copy()
        for ch in text:
            if not trial.feed(ch):
                return False
        self.stack, self.state, self.lit, self.num, self.complete = trial.stack, trial.state, trial.lit, trial.num, trial.complete
        return True

    def accepts(self, text: str) -> bool:
        trial = self.copy()
        return all(trial.feed(ch) for ch in text)


class GrammarFilter:
    """Per-request validators + the logits filter applied before sampling."""

    def __init__(self, token_text: Sequence[str], top_n: int = 64, eos_token_id: int = -1):
        self.token_text = token_text
        self.top_n = top_n
        self.eos = eos_token_id
        self.state: Dict[str, JsonObjectValidator] = {}

    def start(self, request_id: str):
        self.state[request_id] = JsonObjectValidator()

    def forget(self, request_id: str):
        self.state.pop(request_id, None)

    def admissible(self, v: JsonObjectValidator, tok: int) -> bool:
        if tok == self.eos:
            return v.complete
        text = self.token_text[tok]
        if v.complete:
            return text != "" and all(c in _WS for c in text) and False   # nothing but EOS after the object
        return text != "" and v.accepts(text)

    def filter_row(self, request_id: str, row_logits: torch.Tensor):
        """Mask `row_logits` ([V]) in place to the admissible tokens."""
        v = self.state[request_id]
        if v.complete and self.eos >= 0:
            keep = [self.eos]
        else:
            top = torch.topk(row_logits, min(self.top_n, row_logits.numel())).indices.tolist()
            keep = [t for t in top if self.admissible(v, t)]
            if not keep:
                order = torch.argsort(row_logits, descending=True).tolist()
                for t in order:
                    if self.admissible(v, t):
                        keep = [t]
                        break
        if keep:
            saved = row_logits[keep].clone()
            row_logits.fill_(float("-inf"))
            row_logits[keep] = saved

    def advance(self, request_id: str, tok: int):
        v = self.state.get(request_id)
        if v is not None and tok != self.eos and 0 <= tok < len(self.token_text):
            v.feed_text(self.token_text[tok])

    def is_complete(self, request_id: str) -> bool:
        v = self.state.get(request_id)
        return v is not None and v.complete
