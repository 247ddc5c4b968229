"""Tokenizer factory: picks the C++ tokenizer for a model directory.

Parity: TokenizerFactory (xllm/core/framework/tokenizer/tokenizer_factory.cpp): `tokenizer.json`
-> byte-level BPE, `*.tiktoken` -> tiktoken vocabulary; chat templates come from
`tokenizer_config.json` (rendered natively for known families, by jinja2 otherwise).
"""
from __future__ import annotations

import json
import os
from typing import List, Optional


class TokenizerWrapper:
    def __init__(self, impl, model_dir: str = "", config: Optional[dict] = None, model_type: str = ""):
        self.impl = impl
        self.model_dir = model_dir
        self.config = config or {}
        self.chat_template_text = self.config.get("chat_template") or ""
        if isinstance(self.chat_template_text, list):  # named templates
            self.chat_template_text = next((t.get("template", "") for t in self.chat_template_text
                                            if t.get("name") == "default"), "")
        from .. import _rt
        self.family = _rt.ChatTemplate.detect_family(model_type, self.chat_template_text)
        self._native = _rt.ChatTemplate(self.family)
        self._rt = _rt

    @property
    def vocab_size(self):
        return self.impl.vocab_size

    def encode(self, text: str, add_special: bool = False) -> List[int]:
        return self.impl.encode(text, add_special)

    def decode(self, ids, skip_special: bool = True) -> str:
        return self.impl.decode(list(ids), skip_special)

    def token_to_id(self, tok: str) -> int:
        return self.impl.token_to_id(tok)

    def incremental_decoder(self, stops=None, skip_special=True):
        if not isinstance(self.impl, self._rt.BpeTokenizer):
            from .tokenizer_extra import PyIncrementalDecoder
            return PyIncrementalDecoder(self.impl, skip_special)
        return self._rt.IncrementalDecoder(self.impl, list(stops or []), skip_special)

    def apply_chat_template(self, messages, tools=None, add_generation_prompt=True, enable_thinking=True,
                            use_jinja: Optional[bool] = None, **kwargs) -> str:
        known = self.family in ("chatml", "llama3", "deepseek", "glm")
        if use_jinja is None:
            use_jinja = bool(self.chat_template_text) and not known
        if use_jinja and self.chat_template_text:
            import jinja2
            env = jinja2.Environment(trim_blocks=True, lstrip_blocks=True)
            env.globals["raise_exception"] = lambda m: (_ for _ in ()).throw(ValueError(m))
            env.filters["tojson"] = lambda v, **kw: json.dumps(v, ensure_ascii=False)
            return env.from_string(self.chat_template_text).render(
                messages=messages, tools=tools, add_generation_prompt=add_generation_prompt,
                enable_thinking=enable_thinking, bos_token=self.config.get("bos_token", ""),
                eos_token=self.config.get("eos_token", ""), **kwargs)
        msgs = []
        for m in messages:
            content = m.get("content") or ""
            if isinstance(content, list):  # OpenAI content parts
                content = "".join(p.get("text", "") for p in content if p.get("type") == "text")
            tc = m.get("tool_calls")
            msgs.append(self._rt.ChatMessage(m.get("role", "user"), content, json.dumps(tc) if tc else "",
                                             m.get("tool_call_id") or ""))
        return self._native.apply(msgs, json.dumps(tools) if tools else "", add_generation_prompt, enable_thinking)


def load_tokenizer(model_dir: str, model_type: str = "") -> Optional[TokenizerWrapper]:
    from .. import _rt
    cfg = {}
    p = os.path.join(model_dir, "tokenizer_config.json")
    if os.path.exists(p):
        with open(p) as f:
            cfg = json.load(f)
    if not model_type:
        c = os.path.join(model_dir, "config.json")
        if os.path.exists(c):
            with open(c) as f:
                model_type = json.load(f).get("model_type", "")
    tj = os.path.join(model_dir, "tokenizer.json")
    spm_file = os.path.join(model_dir, "tokenizer.model")
    if not os.path.exists(spm_file) and os.path.exists(os.path.join(model_dir, "spiece.model")):
        spm_file = os.path.join(model_dir, "spiece.model")           # the name T5-family releases use
    rwkv = [x for x in os.listdir(model_dir) if x.startswith("rwkv_vocab") and x.endswith(".txt")]
    if not os.path.exists(tj) and os.path.exists(spm_file):
        from .tokenizer_extra import SentencePieceTokenizer
        return TokenizerWrapper(SentencePieceTokenizer(spm_file, bool(cfg.get("add_bos_token")),
                                                       bool(cfg.get("add_eos_token"))), model_dir, cfg, model_type)
    if not os.path.exists(tj) and not os.path.exists(spm_file) and os.path.exists(os.path.join(model_dir, "merges.txt")) \
            and os.path.exists(os.path.join(model_dir, "vocab.json")) and (model_type.startswith("clip") or
                                                                          "CLIP" in str(cfg.get("tokenizer_class", ""))):
        from .tokenizer_extra import ClipBpeTokenizer
        return TokenizerWrapper(ClipBpeTokenizer(os.path.join(model_dir, "vocab.json"), os.path.join(model_dir, "merges.txt")),
                                model_dir, cfg, model_type)
    if not os.path.exists(tj) and rwkv:
        from .tokenizer_extra import RwkvTokenizer
        return TokenizerWrapper(RwkvTokenizer(os.path.join(model_dir, rwkv[0])), model_dir, cfg, model_type)
    tok = _rt.BpeTokenizer()
    if os.path.exists(tj):
        tok.load_hf_file(tj)
    else:
        tk = [x for x in os.listdir(model_dir) if x.endswith(".tiktoken")]
        if not tk:
            return None
        specials = []
        for t in (cfg.get("added_tokens_decoder") or {}).items():
            specials.append((t[1]["content"], int(t[0])))
        tok.load_tiktoken_file(os.path.join(model_dir, tk[0]), specials)

    def _tok_id(v):
        if isinstance(v, dict):
            v = v.get("content")
        return tok.token_to_id(v) if isinstance(v, str) else -1

    tok.set_bos_eos(_tok_id(cfg.get("bos_token")) if cfg.get("add_bos_token") else -1, _tok_id(cfg.get("eos_token")))
    return TokenizerWrapper(tok, model_dir, cfg, model_type)
