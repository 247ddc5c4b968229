"""Text encoders of the diffusion pipelines: the CLIP text transformer (pooled prompt state) and the T5 encoder
(per-token states).  Parity: xllm/models/dit/encoders/{clip_text_model.h,t5_encoder.h}; both are checked against
HuggingFace's implementations.  The T5 stack is the encoder half of `models/onerec.py`."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch
import torch.nn.functional as F

from ..models.onerec import OneRecArgs, OneRecModel


class ClipTextEncoder:
    """Pre-LN transformer with learned positions and a causal mask; returns (last hidden states after the final
    layer norm [B, T, D], pooled state = the hidden state at each prompt's end-of-text token)."""

    def __init__(self, cfg: dict, dtype=torch.float32, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        D, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
        z = lambda *s: torch.zeros(*s, dtype=dtype, device=self.device)
        p: Dict[str, torch.Tensor] = {"embeddings.token_embedding.weight": z(cfg["vocab_size"], D),
                                      "embeddings.position_embedding.weight": z(cfg["max_position_embeddings"], D),
                                      "final_layer_norm.weight": z(D), "final_layer_norm.bias": z(D)}
        for i in range(L):
            b = f"encoder.layers.{i}."
            for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
                p[b + f"self_attn.{n}.weight"], p[b + f"self_attn.{n}.bias"] = z(D, D), z(D)
            for n in ("layer_norm1", "layer_norm2"):
                p[b + n + ".weight"], p[b + n + ".bias"] = z(D), z(D)
            p[b + "mlp.fc1.weight"], p[b + "mlp.fc1.bias"] = z(I, D), z(I)
            p[b + "mlp.fc2.weight"], p[b + "mlp.fc2.bias"] = z(D, I), z(D)
        self.p = p
        self.heads = cfg["num_attention_heads"]
        self.eps = float(cfg.get("layer_norm_eps", 1e-5))
        self.act = cfg.get("hidden_act", "quick_gelu")
        self.eos = int(cfg.get("eos_token_id", 2))

    @staticmethod
    def from_pretrained(model_dir: str, dtype=torch.float32, device="cpu") -> "ClipTextEncoder":
        from ..utils.loader import iterate_weights
        with open(os.path.join(model_dir, "config.json")) as f:
            cfg = json.load(f)
        cfg = cfg.get("text_config", cfg)
        m = ClipTextEncoder(cfg, dtype, device)
        for name, w in iterate_weights(model_dir):
            name = name[len("text_model."):] if name.startswith("text_model.") else name
            if name in m.p:
                m.p[name].copy_(w.to(dtype))
        return m

    @torch.no_grad()
    def forward(self, ids: torch.Tensor):
        p, H = self.p, self.heads
        B, T = ids.shape
        x = p["embeddings.token_embedding.weight"][ids] + p["embeddings.position_embedding.weight"][:T][None]
        D = x.shape[-1]
        for i in range(self.cfg["num_hidden_layers"]):
            b = f"encoder.layers.{i}."
            h = F.layer_norm(x, (D,), p[b + "layer_norm1.weight"], p[b + "layer_norm1.bias"], self.eps)
            q, k, v = (F.linear(h, p[b + f"self_attn.{n}.weight"], p[b + f"self_attn.{n}.bias"]).view(B, T, H, D // H).transpose(1, 2)
                       for n in ("q_proj", "k_proj", "v_proj"))
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, D)
            x = x + F.linear(o, p[b + "self_attn.out_proj.weight"], p[b + "self_attn.out_proj.bias"])
            h = F.layer_norm(x, (D,), p[b + "layer_norm2.weight"], p[b + "layer_norm2.bias"], self.eps)
            h = F.linear(h, p[b + "mlp.fc1.weight"], p[b + "mlp.fc1.bias"])
            h = h * torch.sigmoid(1.702 * h) if self.act == "quick_gelu" else F.gelu(h)
            x = x + F.linear(h, p[b + "mlp.fc2.weight"], p[b + "mlp.fc2.bias"])
        x = F.layer_norm(x, (D,), p["final_layer_norm.weight"], p["final_layer_norm.bias"], self.eps)
        if self.eos == 2:                    # original checkpoints: the end-of-text token has the largest id
            end = ids.argmax(dim=-1)
        else:
            end = (ids == self.eos).int().argmax(dim=-1)
        return x, x[torch.arange(B, device=x.device), end]

    __call__ = forward


class T5TextEncoder:
    """The encoder stack of a T5 checkpoint (`shared.weight`, `encoder.block.*`)."""

    def __init__(self, model: OneRecModel):
        self.model = model

    @staticmethod
    def from_pretrained(model_dir: str, dtype=torch.float32, device="cpu") -> "T5TextEncoder":
        from ..utils.loader import iterate_weights
        with open(os.path.join(model_dir, "config.json")) as f:
            cfg = json.load(f)
        args = OneRecArgs.from_config(cfg)
        args.num_decoder_layers = 0
        m = OneRecModel(args, dtype, device)
        m.load_weights(((n, w) for n, w in iterate_weights(model_dir) if n in m.p), strict=False)
        return T5TextEncoder(m)

    def forward(self, ids: torch.Tensor, lengths=None) -> torch.Tensor:
        return self.model.encode(ids, lengths)

    __call__ = forward
