"""Dense decoder family: Qwen2 / Qwen2.5 / Qwen3 / Llama-style (pre-norm, GQA, SwiGLU).

Parity: `Qwen2DecoderLayerImpl::forward` (xllm/core/layers/qwen2_decoder_layer.cpp:87-109),
`LlmModelImplBase::forward` (xllm/models/llm/llm_model_base.h:85-210), qwen2.h / qwen3.h model
definitions and their `REGISTER_CAUSAL_MODEL` entries.  The residual stream is carried through the
fused add+RMSNorm kernel, exactly one read and one write of the hidden state per norm.
"""
from __future__ import annotations

import torch

from .layers import (Attention, AttentionMetadata, DenseMLP, LMHead, Module, RMSNorm, RotaryEmbedding,
                     VocabEmbedding)
from .registry import register_model
from ..parallel.state import ParallelState, single


class DecoderLayer(Module):
    def __init__(self, args, idx, dtype, device, ps, rope, mlp=None):
        super().__init__()
        self.input_layernorm = self.add_module("input_layernorm", RMSNorm(args.hidden_size, args.rms_norm_eps, dtype, device))
        self.self_attn = self.add_module("self_attn", Attention(args, idx, dtype, device, ps, rope))
        self.post_attention_layernorm = self.add_module(
            "post_attention_layernorm", RMSNorm(args.hidden_size, args.rms_norm_eps, dtype, device))
        self.mlp = self.add_module("mlp", mlp if mlp is not None else
                                   DenseMLP(args.hidden_size, args.intermediate_size, args.hidden_act, dtype, device, ps))

    def forward(self, x, residual, positions, meta, k_cache, v_cache):
        comm = self.self_attn.ps.comm
        if comm is not None and x.is_cuda:
            return self._forward_tp_fused(comm, x, residual, positions, meta, k_cache, v_cache)
        # `residual` holds the running sum; None on the first layer (x is the embedding itself)
        if residual is None:
            residual = x
            h = self.input_layernorm(x)
        else:
            h = self.input_layernorm(x, residual=residual)
        h = self.self_attn(h, positions, meta, k_cache, v_cache)
        h = self.post_attention_layernorm(h, residual=residual)
        h = self.mlp(h)
        return h, residual

    def _forward_tp_fused(self, comm, x, residual, positions, meta, k_cache, v_cache):
        """Tensor-parallel path with the reductions fused into the norms: row-parallel GEMMs leave
        their partial sums in the symmetric buffer, `allreduce_norm` sums them across ranks, adds the
        residual and normalises.  In the two-shot form the residual stream is sharded by token rows
        (each rank keeps and updates only the rows it reduces); in the one-shot form it is replicated."""
        T = x.shape[0]
        eps = self.input_layernorm.eps
        if residual is None:
            residual = comm.new_residual(x)
            h = self.input_layernorm(x)
        else:
            h = comm.allreduce_norm(T, residual, self.input_layernorm.weight, eps)
        self.self_attn(h, positions, meta, k_cache, v_cache)  # partial -> comm.x
        h = comm.allreduce_norm(T, residual, self.post_attention_layernorm.weight, eps)
        h = self.mlp(h)                                       # partial -> comm.x
        return h, residual

    __call__ = forward


class DenseCausalLM(Module):
    """model.embed_tokens -> N x DecoderLayer -> model.norm -> lm_head."""

    fused_tp = True      # False in families whose layers cannot use the fused all-reduce + norm
    supports_prefill_graph = True   # steps with prompt chunks may be captured (padded shapes are safe)

    def __init__(self, args, dtype=torch.bfloat16, device="cpu", ps: ParallelState = None, make_mlp=None,
                 layer_cls=None):
        super().__init__()
        self.args = args
        self.ps = ps or single()
        self.dtype = dtype
        self.device = torch.device(device)
        inner = Module()
        self.add_module("model", inner)
        self.embed = inner.add_module("embed_tokens", VocabEmbedding(args.vocab_size, args.hidden_size, dtype, device, self.ps))
        self.rope = RotaryEmbedding(args.rotary_dim, args.max_position_embeddings, args.rope_theta,
                                    args.rope_scaling, device, args.rope_interleaved)
        layers = Module()
        inner.add_module("layers", layers)
        self.layers = []
        for i in range(args.num_hidden_layers):
            mlp = make_mlp(i) if make_mlp is not None else None
            self.layers.append(layers.add_module(str(i), (layer_cls or DecoderLayer)(args, i, dtype, device, self.ps,
                                                                                      self.rope, mlp)))
        self.norm = inner.add_module("norm", RMSNorm(args.hidden_size, args.rms_norm_eps, dtype, device))
        self.lm_head = LMHead(args.vocab_size, args.hidden_size, dtype, device, self.ps,
                              tied=self.embed if args.tie_word_embeddings else None)
        if not args.tie_word_embeddings:
            self.add_module("lm_head", self.lm_head)

    # KV geometry of one layer on this rank
    @property
    def num_kv_heads_local(self):
        return self.layers[0].self_attn.nkv

    @property
    def head_dim(self):
        return self.args.head_dim

    def forward(self, tokens, positions, meta: AttentionMetadata, kv_caches, embeds=None):
        """tokens/positions: [T] int64.  kv_caches: list of (k_cache, v_cache) per layer.
        `embeds` = (rows, values): input embeddings that replace the token embedding of those rows
        (image tokens of a multimodal prompt).  Returns the final-norm hidden states [T, H]."""
        comm = self.ps.comm if self.fused_tp else None
        if comm is not None and tokens.is_cuda:
            comm.begin_forward(tokens.shape[0])
        x = self.embed(tokens)
        deep = None
        if embeds is not None:
            x = x.clone() if x.data_ptr() == self.embed.weight.data_ptr() else x
            H = x.shape[-1]
            x[embeds[0]] = embeds[1][:, :H].to(x.dtype)
            if embeds[1].shape[-1] > H:                    # "deepstack": further visual features join after the first layers
                deep = embeds[1][:, H:].to(x.dtype).view(embeds[1].shape[0], -1, H)
        residual = None
        aux_ids = getattr(self, "aux_layers", None)        # layers whose outputs a draft head wants to see
        aux = {}
        for i, (layer, (kc, vc)) in enumerate(zip(self.layers, kv_caches)):
            x, residual = layer(x, residual, positions, meta, kc, vc)
            if deep is not None and i < deep.shape[1]:
                x[embeds[0]] += deep[:, i]                  # the branch output joins the residual later: same sum
            if aux_ids and i in aux_ids:
                aux[i] = x + residual                      # the layer's output: the branch joins the residual lazily
        if aux_ids:
            self.last_aux = torch.cat([aux[i] for i in aux_ids], dim=-1)
        if comm is not None and x.is_cuda:
            h = comm.allreduce_norm(x.shape[0], residual, self.norm.weight, self.norm.eps)
            comm.end_forward()
            return h
        return self.norm(x, residual=residual)

    def logits(self, hidden_rows):
        return self.lm_head(hidden_rows)

    # the two halves of `logits`, for callers that can avoid the all-gather (greedy sampling)
    def logits_local(self, hidden_rows):
        return self.lm_head.forward_local(hidden_rows)

    def gather_logits(self, local):
        return self.lm_head.gather(local)

    def greedy_from_local(self, local):
        return self.lm_head.greedy_from_local(local)

    __call__ = forward


@register_model("qwen3", "qwen2", "llama", "mistral", "Qwen3ForCausalLM", "Qwen2ForCausalLM", "LlamaForCausalLM")
def build_dense(args, dtype, device, ps):
    return DenseCausalLM(args, dtype, device, ps)
