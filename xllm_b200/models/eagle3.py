"""EAGLE-3 draft head: one decoder layer that reads the embedding of the next token together with
a fusion of three hidden states of the target model (an early, a middle and a late layer) and
predicts the token after it, over a reduced draft vocabulary.

    g      = fc([h_low | h_mid | h_high])                       3H -> H   (first draft step)
    x      = [input_layernorm(embed(tok)) | hidden_norm(g)]     2H, the attention's input
    h      = g + attn(x);  h = h + mlp(post_attention_layernorm(h))
    logits = lm_head(norm(h))                                   [draft_vocab]
    token  = d + d2t[d]                                         draft id -> target id

Further draft steps feed h back in place of g.  Parity: `Eagle3WorkerImpl`
(xllm/core/runtime/eagle3_worker_impl.cpp:25-110: auxiliary hidden states switched on in the target,
`d2t` turned into the hot-token table) on top of the MTP worker.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from .layers import DenseMLP, Linear, LMHead, MergedColumnLinear, Module, RMSNorm
from ..parallel.state import single


def aux_layer_ids(n_layers: int):
    """The three target layers whose outputs feed the draft head."""
    return (min(2, n_layers - 1), n_layers // 2, max(n_layers - 3, 0))


class Eagle3Draft(Module):
    takes_aux = True

    def __init__(self, args, target, dtype, device, ps=None, draft_vocab: int = 0):
        super().__init__()
        self.args = args
        # The head is one layer: under tensor parallelism every rank runs the WHOLE head on the same
        # (replicated) inputs and so proposes the same drafts; only the token embedding, which it shares
        # with the target, is sharded.  Its KV cache holds all KV heads on every rank (`kv_heads_full`).
        self.target_ps = ps or single()
        self.ps = single()
        H, d = args.hidden_size, args.head_dim
        self.embed = target.embed
        self.rope = target.rope
        self.nq, self.nkv, self.d = args.num_attention_heads, args.num_key_value_heads, d
        self.fc = self.add_module("fc", Linear(3 * H, H, False, dtype, device, self.ps))
        mid = Module()
        self.add_module("midlayer", mid)
        self.input_layernorm = mid.add_module("input_layernorm", RMSNorm(H, args.rms_norm_eps, dtype, device))
        self.hidden_norm = mid.add_module("hidden_norm", RMSNorm(H, args.rms_norm_eps, dtype, device))
        attn = Module()
        mid.add_module("self_attn", attn)
        self.qkv = attn.add_module("qkv_proj", MergedColumnLinear(
            2 * H, [self.nq * d, self.nkv * d, self.nkv * d], ["q_proj", "k_proj", "v_proj"], False, dtype, device, self.ps))
        attn.named_loaders = lambda prefix="", a=attn: ((n.replace("qkv_proj.", ""), f)
                                                        for n, f in Module.named_loaders(a, prefix))
        self.o_proj = attn.add_module("o_proj", Linear(self.nq * d, H, False, dtype, device, self.ps))
        self.post_attention_layernorm = mid.add_module("post_attention_layernorm",
                                                       RMSNorm(H, args.rms_norm_eps, dtype, device))
        self.mlp = mid.add_module("mlp", DenseMLP(H, args.intermediate_size, args.hidden_act, dtype, device, self.ps))
        self.norm = self.add_module("norm", RMSNorm(H, args.rms_norm_eps, dtype, device))
        self.draft_vocab = draft_vocab or args.vocab_size
        self.lm_head = self.add_module("lm_head", LMHead(self.draft_vocab, H, dtype, device, self.ps))
        # draft id -> target id offsets; identity when the head predicts over the full vocabulary
        self.d2t = self.add_param("d2t", torch.zeros(self.draft_vocab, dtype=torch.int64, device=device))
        self.scale = 1.0 / math.sqrt(d)
        self.kv_shape_like = None
        self.kv_heads_full = self.nkv

    def init_random(self, std=0.02, seed=0):
        super().init_random(std, seed)
        self.d2t.zero_()

    def forward(self, tokens, prev, positions, meta, k_cache, v_cache):
        """prev: [T, 3H] fused target states (first step) or [T, H] the head's own output (chained).
        Returns the pre-norm hidden state [T, H] (the input of a chained step); `logits` norms it."""
        g = self.fc(prev) if prev.shape[-1] == 3 * self.args.hidden_size else prev
        e = self.input_layernorm(self.embed(tokens))
        x = torch.cat([e, self.hidden_norm(g)], dim=-1)
        qkv = self.qkv(x)
        q = ops.rope_kv_write(qkv, self.nq, self.nkv, self.d, positions, self.rope.cos_sin, self.rope.rot_dim,
                              slots=meta.slots, k_cache=k_cache, v_cache=v_cache, interleaved=self.rope.interleaved)
        T = q.shape[0]
        out = torch.empty((T, self.nq, self.d), dtype=q.dtype, device=q.device)
        nd = meta.n_decode
        if nd > 0:
            ops.paged_decode_attention(q[:nd], k_cache, v_cache, meta.block_table[:nd], meta.kv_lens[:nd], self.scale,
                                       splits=meta.decode_splits, workspace=meta.decode_workspace, out=out[:nd])
        if meta.n_prefill > 0:
            ops.paged_prefill_attention(q, k_cache, v_cache, meta.block_table[nd:], meta.cu_q[nd:], meta.kv_lens[nd:],
                                        meta.max_q_len, self.scale, causal=True, out=out)
        h = g + self.o_proj(out.view(T, self.nq * self.d))
        return h + self.mlp(self.post_attention_layernorm(h))

    def logits(self, hidden_rows):
        return self.lm_head(self.norm(hidden_rows))

    def to_target_ids(self, draft_ids):
        return draft_ids + self.d2t[draft_ids]

    __call__ = forward
