"""OneRec: an encoder-decoder generative recommender in the T5 layout — a bidirectional encoder over the
user's history, a short causal decoder with cross-attention that emits an item's semantic id (a few tokens)
under a wide beam.

Parity: `onerec` of the reference (xllm/models/rec/onerec.h with rec_model_base.h: d_model / d_kv / d_ff /
num_layers / num_decoder_layers, relative attention buckets, RMS layer norm, tied embedding with the
d_model^-0.5 logit scale; `OneRecXAttention` / prefill-only pipelines of rec_engine.cpp).  The layer
arithmetic is T5's and is checked against HuggingFace's T5ForConditionalGeneration.

Execution model.  The history is encoded once per request (dense bidirectional attention with the learned
relative-position bias).  The decoder never holds more than `num_steps` tokens per beam, so each round
recomputes the beams' few decoder positions instead of keeping a self-attention cache; what is worth keeping
is the cross-attention K / V of every decoder layer, projected once per REQUEST and read by all of its beams
(the beams are extra query rows over shared keys, the same sharing x-attention gives decoder-only models).
Selection runs on the same kernels as the LLM-backbone rec engine (`ops/select.py`).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from ..ops import select


@dataclass
class OneRecArgs:
    vocab_size: int = 8200
    d_model: int = 128
    d_kv: int = 32
    d_ff: int = 256
    num_layers: int = 12                   # encoder
    num_decoder_layers: int = 4
    num_heads: int = 4
    relative_attention_num_buckets: int = 32
    relative_attention_max_distance: int = 128
    layer_norm_epsilon: float = 1e-6
    feed_forward_proj: str = "relu"        # "relu" (wi, wo) | "gated-gelu" (wi_0, wi_1, wo)
    tie_word_embeddings: bool = True
    decoder_start_token_id: int = 0
    pad_token_id: int = 0
    eos_token_id: int = 1

    @staticmethod
    def from_config(cfg: dict) -> "OneRecArgs":
        a = OneRecArgs()
        for k in a.__dataclass_fields__:
            if cfg.get(k) is not None:
                setattr(a, k, type(getattr(a, k))(cfg[k]))
        if cfg.get("num_decoder_layers") is None:
            a.num_decoder_layers = a.num_layers
        return a


def _rms(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def relative_bucket(rel: torch.Tensor, bidirectional: bool, num_buckets: int, max_distance: int) -> torch.Tensor:
    """T5's bucketing of (key position - query position): exact small offsets, logarithmic large ones."""
    out = torch.zeros_like(rel)
    if bidirectional:
        num_buckets //= 2
        out = out + (rel > 0).long() * num_buckets
        rel = rel.abs()
    else:
        rel = -torch.min(rel, torch.zeros_like(rel))
    exact = num_buckets // 2
    small = rel < exact
    large = exact + (torch.log(rel.float().clamp(min=1) / exact) / math.log(max_distance / exact) * (num_buckets - exact)).long()
    large = torch.min(large, torch.full_like(large, num_buckets - 1))
    return out + torch.where(small, rel, large)


class OneRecModel:
    def __init__(self, args: OneRecArgs, dtype=torch.float32, device="cpu"):
        self.args, self.dtype, self.device = args, dtype, torch.device(device)
        a = args
        inner = a.num_heads * a.d_kv
        z = lambda *s: torch.zeros(*s, dtype=dtype, device=self.device)
        p: Dict[str, torch.Tensor] = {"shared.weight": z(a.vocab_size, a.d_model)}
        ff = (("wi_0", (a.d_ff, a.d_model)), ("wi_1", (a.d_ff, a.d_model)), ("wo", (a.d_model, a.d_ff))) \
            if a.feed_forward_proj.startswith("gated") else (("wi", (a.d_ff, a.d_model)), ("wo", (a.d_model, a.d_ff)))
        for stack, n, cross in (("encoder", a.num_layers, False), ("decoder", a.num_decoder_layers, True)):
            for i in range(n):
                b = f"{stack}.block.{i}.layer."
                for nm in "qkvo":
                    p[f"{b}0.SelfAttention.{nm}.weight"] = z(*((a.d_model, inner) if nm == "o" else (inner, a.d_model)))
                p[f"{b}0.layer_norm.weight"] = z(a.d_model)
                j = 1
                if cross:
                    for nm in "qkvo":
                        p[f"{b}1.EncDecAttention.{nm}.weight"] = z(*((a.d_model, inner) if nm == "o" else (inner, a.d_model)))
                    p[f"{b}1.layer_norm.weight"] = z(a.d_model)
                    j = 2
                for nm, shape in ff:
                    p[f"{b}{j}.DenseReluDense.{nm}.weight"] = z(*shape)
                p[f"{b}{j}.layer_norm.weight"] = z(a.d_model)
            p[f"{stack}.block.0.layer.0.SelfAttention.relative_attention_bias.weight"] = z(a.relative_attention_num_buckets, a.num_heads)
            p[f"{stack}.final_layer_norm.weight"] = z(a.d_model)
        if not a.tie_word_embeddings:
            p["lm_head.weight"] = z(a.vocab_size, a.d_model)
        self.p = p

    # ------------------------------------------------------------------------------------------ weights
    def init_random(self, std=0.05, seed=0):
        g = torch.Generator().manual_seed(seed)
        for k, t in self.p.items():
            if k.endswith("layer_norm.weight"):
                t.fill_(1.0)
            else:
                t.copy_((torch.randn(t.shape, generator=g) * std).to(t.dtype))

    def load_weights(self, weights, strict=True):
        seen = set()
        for name, w in weights:
            name = name[len("model."):] if name.startswith("model.") else name
            if name in ("encoder.embed_tokens.weight", "decoder.embed_tokens.weight"):
                continue                                     # aliases of shared.weight
            if name == "lm_head.weight" and self.args.tie_word_embeddings:
                continue
            if name in self.p:
                self.p[name].copy_(w.to(self.dtype))
                seen.add(name)
            elif strict:
                raise KeyError(f"unexpected tensor {name}")
        missing = set(self.p) - seen
        if strict and missing:
            raise KeyError(f"missing tensors: {sorted(missing)[:5]}")
        return seen

    @staticmethod
    def from_pretrained(model_dir: str, dtype=torch.float32, device="cpu") -> "OneRecModel":
        from ..utils.loader import iterate_weights
        with open(os.path.join(model_dir, "config.json")) as f:
            args = OneRecArgs.from_config(json.load(f))
        m = OneRecModel(args, dtype, device)
        m.load_weights(iterate_weights(model_dir))
        return m

    # ------------------------------------------------------------------------------------------ layers
    def _bias(self, stack: str, q_len: int, k_len: int, bidirectional: bool) -> torch.Tensor:
        a = self.args
        ctx = torch.arange(q_len, device=self.device)[:, None]
        mem = torch.arange(k_len, device=self.device)[None, :]
        buckets = relative_bucket(mem - ctx, bidirectional, a.relative_attention_num_buckets, a.relative_attention_max_distance)
        table = self.p[f"{stack}.block.0.layer.0.SelfAttention.relative_attention_bias.weight"]
        return table[buckets].permute(2, 0, 1)                # [heads, q, k]

    def _attn(self, prefix: str, x, kv, bias, mask):
        """x [B, Tq, D] queries, kv [B, Tk, D] (or a precomputed (K, V) pair), additive bias [h, Tq, Tk] and
        mask [B, 1, Tq or 1, Tk]; T5 attention has no 1/sqrt(d) scaling."""
        a, p = self.args, self.p
        B, Tq, _ = x.shape
        q = F.linear(x, p[prefix + "q.weight"]).view(B, Tq, a.num_heads, a.d_kv).transpose(1, 2)
        if isinstance(kv, tuple):
            k, v = kv
        else:
            k, v = self.project_kv(prefix, kv)
        s = torch.matmul(q.float(), k.float().transpose(-1, -2))
        if bias is not None:
            s = s + bias.float()[None]
        if mask is not None:
            s = s + mask
        o = torch.matmul(torch.softmax(s, dim=-1), v.float()).to(x.dtype)
        return F.linear(o.transpose(1, 2).reshape(B, Tq, a.num_heads * a.d_kv), p[prefix + "o.weight"])

    def project_kv(self, prefix: str, kv):
        a, p = self.args, self.p
        B, Tk, _ = kv.shape
        k = F.linear(kv, p[prefix + "k.weight"]).view(B, Tk, a.num_heads, a.d_kv).transpose(1, 2)
        v = F.linear(kv, p[prefix + "v.weight"]).view(B, Tk, a.num_heads, a.d_kv).transpose(1, 2)
        return k, v

    def _ff(self, prefix: str, x):
        p = self.p
        if self.args.feed_forward_proj.startswith("gated"):
            h = F.gelu(F.linear(x, p[prefix + "wi_0.weight"]), approximate="tanh") * F.linear(x, p[prefix + "wi_1.weight"])
        else:
            h = F.relu(F.linear(x, p[prefix + "wi.weight"]))
        return F.linear(h, p[prefix + "wo.weight"])

    # ------------------------------------------------------------------------------------------ stacks
    @torch.no_grad()
    def encode(self, tokens: torch.Tensor, lengths: Optional[torch.Tensor] = None) -> torch.Tensor:
        """tokens [R, L] (right-padded), lengths [R] -> encoder states [R, L, D]."""
        a, p = self.args, self.p
        R, L = tokens.shape
        x = p["shared.weight"][tokens]
        mask = None
        if lengths is not None:
            pad = torch.arange(L, device=self.device)[None, :] >= lengths[:, None]
            mask = torch.zeros(R, 1, 1, L, device=self.device).masked_fill(pad[:, None, None, :], float("-inf"))
        bias = self._bias("encoder", L, L, True)
        for i in range(a.num_layers):
            b = f"encoder.block.{i}.layer."
            h = _rms(x, p[b + "0.layer_norm.weight"], a.layer_norm_epsilon)
            x = x + self._attn(b + "0.SelfAttention.", h, h, bias, mask)
            x = x + self._ff(b + "1.DenseReluDense.", _rms(x, p[b + "1.layer_norm.weight"], a.layer_norm_epsilon))
        return _rms(x, p["encoder.final_layer_norm.weight"], a.layer_norm_epsilon)

    @torch.no_grad()
    def cross_kv(self, enc: torch.Tensor):
        """Per decoder layer the cross-attention (K, V) of the encoder states [R, L, D]: once per request."""
        return [self.project_kv(f"decoder.block.{i}.layer.1.EncDecAttention.", enc) for i in range(self.args.num_decoder_layers)]

    @torch.no_grad()
    def decode(self, dec_tokens: torch.Tensor, cross, enc_mask=None, rows_per_request: int = 1) -> torch.Tensor:
        """dec_tokens [B, t] (B = requests x beams, beams of a request adjacent); `cross` from `cross_kv`
        for the REQUESTS; returns the logits of the last position [B, V]."""
        a, p = self.args, self.p
        B, t = dec_tokens.shape
        x = p["shared.weight"][dec_tokens]
        causal = torch.zeros(t, t, device=self.device).masked_fill(
            torch.ones(t, t, dtype=torch.bool, device=self.device).triu(1), float("-inf"))[None, None]
        bias = self._bias("decoder", t, t, False)
        W = rows_per_request
        for i in range(a.num_decoder_layers):
            b = f"decoder.block.{i}.layer."
            h = _rms(x, p[b + "0.layer_norm.weight"], a.layer_norm_epsilon)
            x = x + self._attn(b + "0.SelfAttention.", h, h, bias, causal)
            k, v = cross[i]                                   # [R, heads, L, d]: shared by the W beams of a request
            if W > 1:
                k, v = k.repeat_interleave(W, 0), v.repeat_interleave(W, 0)
            m = enc_mask.repeat_interleave(W, 0) if (enc_mask is not None and W > 1) else enc_mask
            x = x + self._attn(b + "1.EncDecAttention.", _rms(x, p[b + "1.layer_norm.weight"], a.layer_norm_epsilon), (k, v), None, m)
            x = x + self._ff(b + "2.DenseReluDense.", _rms(x, p[b + "2.layer_norm.weight"], a.layer_norm_epsilon))
        h = _rms(x[:, -1], p["decoder.final_layer_norm.weight"], a.layer_norm_epsilon)
        if a.tie_word_embeddings:
            return F.linear(h * (a.d_model ** -0.5), p["shared.weight"])
        return F.linear(h, p["lm_head.weight"])

    # ------------------------------------------------------------------------------------------ generation
    @torch.no_grad()
    def recommend(self, histories: Sequence[Sequence[int]], beam_width: int = 32, num_steps: int = 3, trie=None,
                  num_return: Optional[int] = None):
        """For every history the `beam_width` most likely items of `num_steps` tokens, best first
        (`engine.rec.RecItem`s); `trie` (an `engine.rec.ItemTrie`) restricts them to a catalogue."""
        from ..engine.rec import RecItem
        a, dev = self.args, self.device
        R, W, V = len(histories), min(int(beam_width), self.args.vocab_size), self.args.vocab_size
        if R == 0:
            return []
        L = max(len(h) for h in histories)
        toks = torch.full((R, L), a.pad_token_id, dtype=torch.long, device=dev)
        lens = torch.tensor([len(h) for h in histories], device=dev)
        for i, h in enumerate(histories):
            toks[i, : len(h)] = torch.tensor(list(h), dtype=torch.long, device=dev)
        enc = self.encode(toks, lens)
        cross = self.cross_kv(enc)
        pad = torch.arange(L, device=dev)[None, :] >= lens[:, None]
        enc_mask = torch.zeros(R, 1, 1, L, device=dev).masked_fill(pad[:, None, None, :], float("-inf"))
        start = torch.full((R, 1), a.decoder_start_token_id, dtype=torch.long, device=dev)

        def candidates(logits, k, mask):
            if mask is None:
                lp, ids = select.topk(logits.float(), k, normalize=True)
            else:
                full = select.log_softmax(logits.float()).masked_fill(~mask, float("-inf"))
                lp, ids = select.topk(full, k)
            lp = lp.float()
            return torch.where(torch.isfinite(lp), lp, torch.full_like(lp, float("-inf"))), ids

        nodes = None
        if trie is not None:
            trie.to(dev)
            nodes = trie.root(R)
        cum, ids = candidates(self.decode(start, cross, enc_mask, 1), W, None if trie is None else trie.mask_of(0, nodes))
        if trie is not None:
            nodes = trie.advance(0, nodes.repeat_interleave(W), ids.reshape(-1).to(torch.long))
        seqs = ids.to(torch.long)[:, :, None]                                      # [R, W, 1]
        k_cand = min(W, V)
        for s in range(1, num_steps):
            dec = torch.cat([start.repeat_interleave(W, 0), seqs.reshape(R * W, -1)], dim=1)
            logits = self.decode(dec, cross, enc_mask, W)
            lp, ids = candidates(logits, k_cand, None if trie is None else trie.mask_of(s, nodes))
            tok, par, cum = select.beam_step(lp.view(R, W, k_cand), ids.view(R, W, k_cand), cum, W)
            par = par.to(torch.long)
            if trie is not None and s + 1 < num_steps:
                nodes = trie.advance(s, nodes.view(R, W).gather(1, par).reshape(-1), tok.reshape(-1).to(torch.long))
            seqs = torch.cat([seqs.gather(1, par[:, :, None].expand(R, W, seqs.shape[2])), tok.to(torch.long)[:, :, None]], dim=2)
        cum_h, seq_h = cum.tolist(), seqs.tolist()
        out = []
        for r in range(R):
            items = [RecItem(seq_h[r][w], cum_h[r][w]) for w in range(W) if cum_h[r][w] != float("-inf")]
            items.sort(key=lambda it: -it.logprob)
            out.append(items[: (num_return or W)])
        return out
