"""Decoder families that are variations of the dense / sparse-MoE decoder: GLM-4 (sandwich norms,
interleaved partial rotary, fused gate_up checkpoints), GLM-4.5/4.6 MoE (DeepSeek-V3 style routing on
GQA attention), MiniMax-M2 (whole-vector q/k norm, sigmoid routing, w1/w2/w3 expert names) and MiMo
(Qwen2 layout with MTP layers beside it).

Parity: the reference registers these through `REGISTER_CAUSAL_MODEL` in xllm/models/llm/
(glm4.h, glm4_moe.h, minimax_m2.h, mimo.h and their decoder layers under xllm/core/layers/); the
layer arithmetic follows the published HuggingFace implementations, which the CPU tests use as the
oracle.
"""
from __future__ import annotations

import re

import torch

from .layers import Attention, DenseMLP, Module, RMSNorm
from .qwen import DecoderLayer, DenseCausalLM
from .qwen_moe import SparseMoeBlock
from .registry import register_model


# --------------------------------------------------------------------------------------- GLM-4 dense
class Glm4DecoderLayer(DecoderLayer):
    """x + post_self_attn_norm(attn(input_norm(x))), then the same around the MLP: the branch output is
    normalised before it joins the residual, so the cross-rank sum of a row-parallel GEMM cannot be
    folded into the add+norm that follows; the row-parallel layers all-reduce by themselves."""

    def __init__(self, args, idx, dtype, device, ps, rope, mlp=None):
        Module.__init__(self)
        H, eps = args.hidden_size, args.rms_norm_eps
        self.input_layernorm = self.add_module("input_layernorm", RMSNorm(H, eps, dtype, device))
        self.self_attn = self.add_module("self_attn", Attention(args, idx, dtype, device, ps, rope, fuse_reduce=False))
        self.post_self_attn_layernorm = self.add_module("post_self_attn_layernorm", RMSNorm(H, eps, dtype, device))
        self.post_attention_layernorm = self.add_module("post_attention_layernorm", RMSNorm(H, eps, dtype, device))
        self.mlp = self.add_module("mlp", mlp if mlp is not None else DenseMLP(
            H, args.intermediate_size, args.hidden_act, dtype, device, ps, fuse_reduce=False))
        self.post_mlp_layernorm = self.add_module("post_mlp_layernorm", RMSNorm(H, eps, dtype, device))

    def forward(self, x, residual, positions, meta, k_cache, v_cache):
        if residual is None:
            residual = x.clone()
            h = self.input_layernorm(x)
        else:
            h = self.input_layernorm(x, residual=residual)         # residual += x; h = norm(residual)
        h = self.post_self_attn_layernorm(self.self_attn(h, positions, meta, k_cache, v_cache))
        h = self.post_attention_layernorm(h, residual=residual)
        h = self.post_mlp_layernorm(self.mlp(h))
        return h, residual

    __call__ = forward


class Glm4CausalLM(DenseCausalLM):
    fused_tp = False

    def __init__(self, args, dtype=torch.bfloat16, device="cpu", ps=None):
        super().__init__(args, dtype, device, ps, layer_cls=Glm4DecoderLayer)

    @staticmethod
    def remap_weight(name, w):
        if name.endswith("mlp.gate_up_proj.weight"):               # [2I, H]: gate rows, then up rows
            half = w.shape[0] // 2
            base = name[: -len("gate_up_proj.weight")]
            return [(base + "gate_proj.weight", w[:half]), (base + "up_proj.weight", w[half:])]
        return [(name, w)]


@register_model("glm4", "glm", "Glm4ForCausalLM", "GlmForCausalLM")
def build_glm4(args, dtype, device, ps):
    return Glm4CausalLM(args, dtype, device, ps)


# --------------------------------------------------------------------------------------- GLM-4.5 MoE
def _moe_or_dense(args, dtype, device, ps):
    def make(i):
        if args.is_moe_layer(i):
            return SparseMoeBlock(args, dtype, device, ps)
        return DenseMLP(args.hidden_size, args.intermediate_size, args.hidden_act, dtype, device, ps)
    return make


@register_model("glm4_moe", "Glm4MoeForCausalLM")
def build_glm4_moe(args, dtype, device, ps):
    """GQA attention (optional per-head q/k norm, half of each head rotated) over DeepSeek-V3 style
    MoE layers: sigmoid scores with a selection bias, grouped top-k, shared experts, scaled weights;
    the first `first_k_dense_replace` layers are dense."""
    return DenseCausalLM(args, dtype, device, ps, make_mlp=_moe_or_dense(args, dtype, device, ps))


# --------------------------------------------------------------------------------------- MiniMax-M2
class MiniMaxAttention(Attention):
    """q and k are RMS-normalised over the WHOLE projected vector (all heads together) before the
    rotary embedding.  Under tensor parallelism a rank holds a slice of the heads, so the mean of
    squares is completed with one small all-reduce of [T, 2] sums."""

    def __init__(self, args, layer_idx, dtype, device, ps=None, rope=None):
        a = _with(args, qk_norm=False)
        super().__init__(a, layer_idx, dtype, device, ps, rope)
        tp, rank = self.ps.tp_size, self.ps.tp_rank
        self.nq_total = args.num_attention_heads
        self.q_norm_w = torch.ones(self.nq * self.d, dtype=dtype, device=device)
        self.k_norm_w = torch.ones(self.nkv * self.d, dtype=dtype, device=device)
        kv_rank = rank * min(tp, self.nkv_total) // tp

        def lq(w, t=self.q_norm_w):
            t.copy_(w.narrow(0, rank * t.numel(), t.numel()).to(t.dtype))

        def lk(w, t=self.k_norm_w):
            t.copy_(w.narrow(0, kv_rank * t.numel(), t.numel()).to(t.dtype))

        self.add_param("q_norm.weight", self.q_norm_w, {"q_norm.weight": lq})
        self.add_param("k_norm.weight", self.k_norm_w, {"k_norm.weight": lk})

    def forward(self, x, positions, meta, k_cache, v_cache):
        qkv = self.qkv(x)
        nq, nkv, d = self.nq, self.nkv, self.d
        q, k = qkv[:, : nq * d], qkv[:, nq * d: (nq + nkv) * d]
        ss = torch.stack([q.float().pow(2).sum(-1), k.float().pow(2).sum(-1)], -1)        # [T, 2]
        if self.ps.tp_size > 1:
            # KV heads replicated across ranks would be counted more than once
            rep = max(1, self.ps.tp_size // self.nkv_total)
            ss[:, 1] /= rep
            ss = self.ps.all_reduce(ss)
        inv_q = torch.rsqrt(ss[:, 0:1] / (self.nq_total * d) + self.eps)
        inv_k = torch.rsqrt(ss[:, 1:2] / (self.nkv_total * d) + self.eps)
        qkv = qkv.clone()
        qkv[:, : nq * d] = (q.float() * inv_q).to(qkv.dtype) * self.q_norm_w
        qkv[:, nq * d: (nq + nkv) * d] = (k.float() * inv_k).to(qkv.dtype) * self.k_norm_w
        return self._attend(qkv, positions, meta, k_cache, v_cache)

    __call__ = forward


def _with(args, **kw):
    import dataclasses
    return dataclasses.replace(args, **kw)


class MiniMaxDecoderLayer(DecoderLayer):
    def __init__(self, args, idx, dtype, device, ps, rope, mlp=None):
        Module.__init__(self)
        H, eps = args.hidden_size, args.rms_norm_eps
        self.input_layernorm = self.add_module("input_layernorm", RMSNorm(H, eps, dtype, device))
        self.self_attn = self.add_module("self_attn", MiniMaxAttention(args, idx, dtype, device, ps, rope))
        self.post_attention_layernorm = self.add_module("post_attention_layernorm", RMSNorm(H, eps, dtype, device))
        self.mlp = self.add_module("mlp", mlp)


_MM_EXPERT = re.compile(r"(.*)\.(?:block_sparse_moe|mlp)\.experts\.(\d+)\.(w1|w2|w3)\.weight$")
_MM_NAMES = {"w1": "gate_proj", "w3": "up_proj", "w2": "down_proj"}


class MiniMaxCausalLM(DenseCausalLM):
    def __init__(self, args, dtype=torch.bfloat16, device="cpu", ps=None):
        a = _with(args, moe_intermediate_size=args.moe_intermediate_size or args.intermediate_size,
                  norm_topk_prob=True, scoring_func="sigmoid", router_bias=True, n_shared_experts=0)
        super().__init__(a, dtype, device, ps, layer_cls=MiniMaxDecoderLayer,
                         make_mlp=lambda i: SparseMoeBlock(a, dtype, device, ps))

    @staticmethod
    def remap_weight(name, w):
        m = _MM_EXPERT.match(name)
        if m:
            return [(f"{m.group(1)}.mlp.experts.{m.group(2)}.{_MM_NAMES[m.group(3)]}.weight", w)]
        name = name.replace(".block_sparse_moe.", ".mlp.")
        if name.endswith(".mlp.e_score_correction_bias"):
            name = name[: -len("e_score_correction_bias")] + "gate.e_score_correction_bias"
        return [(name, w)]


@register_model("minimax_m2", "MiniMaxM2ForCausalLM")
def build_minimax_m2(args, dtype, device, ps):
    return MiniMaxCausalLM(args, dtype, device, ps)


# --------------------------------------------------------------------------------------- MiMo
@register_model("mimo", "MiMoForCausalLM")
def build_mimo(args, dtype, device, ps):
    """MiMo-7B: the Qwen2 decoder (q/k/v biases, no q/k norm); its `model.mtp_layers.*` tensors belong
    to the multi-token-prediction drafter and are not part of the target model."""
    return DenseCausalLM(args, dtype, device, ps)
