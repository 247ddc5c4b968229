"""Qwen3-Next / Qwen3.5 style hybrid decoder: three gated-delta-net (linear attention) layers for
every gated full-attention layer, zero-centred RMSNorm weights, sparse MoE with a gated shared expert.

A linear-attention layer keeps, per sequence, a convolution tail [conv_dim, K - 1] and a recurrent
state [value heads, d_k, d_v] (fp32) instead of a KV cache.  The states live in slots owned by the
running requests (`LinearStateCache`); the engine assigns slots and tells the layer which sequences
start from scratch.  Prefix caching is off for this family: skipping cached prompt tokens would skip
the state updates they cause.

    g_t = -exp(A_log) * softplus(a_t + dt_bias),   beta_t = sigmoid(b_t)
    S <- S * exp(g_t);  S <- S + k_t (x) ((v_t - S^T k_t) * beta_t);  o_t = S^T q_t

Parity: xllm/models/llm/qwen3_next.h and the `LinearState` block manager of the reference
(xllm/core/framework/block/); the arithmetic follows the published HuggingFace implementation, which
is the oracle of the CPU test.  The recurrence runs on tensor-library ops (one batched update per
decode step, a token loop per prompt chunk); a fused kernel for it is not built.
"""
from __future__ import annotations

import dataclasses

import torch
import torch.nn.functional as F

from ..ops import gdn as gdn_ops
from .layers import Attention, DenseMLP, Linear, MergedColumnLinear, Module, RMSNorm
from .qwen import DecoderLayer, DenseCausalLM
from .qwen_moe import SparseMoeBlock
from .registry import register_model
from ..parallel.state import single


class LinearStateCache:
    """Convolution tails and recurrent states of every linear-attention layer, one slot per running
    sequence (keyed by the scheduler's sequence id: parallel samples of one request have their own
    state).  The scheduler admits at most `slots` sequences at a time and slots return on finish and
    on preemption, so `slot_of` finds a free slot whenever it needs one."""

    def __init__(self, n_layers, slots, conv_dim, kernel, nv, dk, dv, device, dtype):
        self.conv = torch.zeros(n_layers, slots, conv_dim, kernel - 1, dtype=dtype, device=device)
        self.rec = torch.zeros(n_layers, slots, nv, dk, dv, dtype=torch.float32, device=device)
        self.free = list(range(slots - 1, -1, -1))
        self.owner = {}
        self.n_slots = slots

    def slot_of(self, request_id):
        s = self.owner.get(request_id)
        if s is None:
            if not self.free:
                raise RuntimeError("no free linear-state slot: the scheduler admitted more sequences than the pool holds")
            s = self.owner[request_id] = self.free.pop()
        return s

    def release(self, request_id):
        s = self.owner.pop(request_id, None)
        if s is not None:
            self.free.append(s)


class GatedDeltaNet(Module):
    def __init__(self, args, idx, lin_idx, dtype, device, ps=None):
        super().__init__()
        self.ps = ps or single()
        assert self.ps.tp_size == 1, "linear-attention layers run unsharded"
        e = args.extra
        self.nv, self.nk = e["linear_num_value_heads"], e["linear_num_key_heads"]
        self.dk, self.dv = e["linear_key_head_dim"], e["linear_value_head_dim"]
        self.K = e.get("linear_conv_kernel_dim", 4)
        self.key_dim, self.value_dim = self.nk * self.dk, self.nv * self.dv
        self.conv_dim = 2 * self.key_dim + self.value_dim
        self.lin_idx = lin_idx
        self.eps = args.rms_norm_eps
        H = args.hidden_size
        # Qwen3-Next packs q|k|v|z per key head in one projection (and b|a in another); Qwen3.5 has four
        # plain projections: [all q | all k | all v], z, b, a
        self.split_proj = bool(e.get("split_proj"))
        if self.split_proj:
            self.in_proj_qkv = self.add_module("in_proj_qkv", Linear(H, self.conv_dim, False, dtype, device))
            self.in_proj_z = self.add_module("in_proj_z", Linear(H, self.value_dim, False, dtype, device))
            self.in_proj_b = self.add_module("in_proj_b", Linear(H, self.nv, False, dtype, device))
            self.in_proj_a = self.add_module("in_proj_a", Linear(H, self.nv, False, dtype, device))
        else:
            self.in_proj_qkvz = self.add_module("in_proj_qkvz", Linear(H, 2 * self.key_dim + 2 * self.value_dim, False, dtype, device))
            self.in_proj_ba = self.add_module("in_proj_ba", Linear(H, 2 * self.nv, False, dtype, device))
        self.conv_w = torch.zeros(self.conv_dim, self.K, dtype=dtype, device=device)
        self.add_param("conv1d.weight", self.conv_w, {"conv1d.weight": lambda w, t=self.conv_w: t.copy_(w.reshape(t.shape).to(t.dtype))})
        self.dt_bias = self.add_param("dt_bias", torch.ones(self.nv, dtype=dtype, device=device))
        self.A_log = self.add_param("A_log", torch.zeros(self.nv, dtype=dtype, device=device))
        self.norm_w = self.add_param("norm.weight", torch.ones(self.dv, dtype=dtype, device=device))
        self.out_proj = self.add_module("out_proj", Linear(self.value_dim, H, False, dtype, device))

    def _step(self, S, q, k, v, g, beta):
        """One token for a batch of states: S [B, nv, dk, dv]; q, k [B, nv, dk]; v [B, nv, dv]; g, beta [B, nv]."""
        S = S * g.exp()[:, :, None, None]
        delta = (v - (S * k[..., None]).sum(-2)) * beta[..., None]
        S = S + k[..., None] * delta[:, :, None, :]
        return S, (S * q[..., None]).sum(-2)

    def forward(self, x, meta, state: LinearStateCache):
        T = x.shape[0]
        nk, nv, dk, dv, r = self.nk, self.nv, self.dk, self.dv, self.nv // self.nk
        if self.split_proj:
            mixed = self.in_proj_qkv(x)
            z = self.in_proj_z(x).view(T, nv, dv)
            b, a = self.in_proj_b(x), self.in_proj_a(x)
        else:
            qkvz = self.in_proj_qkvz(x).view(T, nk, 2 * dk + 2 * r * dv)
            ba = self.in_proj_ba(x).view(T, nk, 2 * r)
            q, k, v, z = torch.split(qkvz, [dk, dk, r * dv, r * dv], dim=-1)
            b, a = torch.split(ba, [r, r], dim=-1)
            z = z.reshape(T, nv, dv)
            mixed = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=-1)  # [T, conv_dim]
        beta = torch.sigmoid(b.reshape(T, nv).float())
        g = -self.A_log.float().exp() * F.softplus(a.reshape(T, nv).float() + self.dt_bias.float())
        conv, rec = state.conv[self.lin_idx], state.rec[self.lin_idx]
        slots, fresh, bounds = meta.state_slots, meta.state_fresh, meta.seq_bounds
        out = torch.empty(T, nv, dv, dtype=torch.float32, device=x.device)

        def heads(y):                                      # conv output rows -> normalised, scaled q / k and v per value head
            qh, kh, vh = torch.split(y, [self.key_dim, self.key_dim, self.value_dim], dim=-1)
            qh = qh.reshape(-1, nk, dk).float()
            kh = kh.reshape(-1, nk, dk).float()
            qh = qh * torch.rsqrt((qh * qh).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
            kh = kh * torch.rsqrt((kh * kh).sum(-1, keepdim=True) + 1e-6)
            if r > 1:
                qh, kh = qh.repeat_interleave(r, dim=1), kh.repeat_interleave(r, dim=1)
            return qh, kh, vh.reshape(-1, nv, dv).float()

        nd = meta.n_decode
        if nd > 0:                                         # one token per sequence: a single batched update
            s = slots[:nd]
            tail = conv[s]                                 # [B, conv_dim, K-1]
            full = torch.cat([tail, mixed[:nd, :, None]], dim=-1)                     # [B, conv_dim, K]
            y = F.silu((full.float() * self.conv_w.float()).sum(-1)).to(x.dtype)
            conv[s] = full[:, :, 1:]
            qh, kh, vh = heads(y)
            gdn_ops.decode_step(rec, s, qh, kh, vh, g[:nd], beta[:nd], out=out[:nd])
        for i in range(nd, len(bounds)):                   # prompt chunks
            a0, b0 = bounds[i]
            s = int(slots[i])
            tail = torch.zeros_like(conv[s]) if fresh[i] else conv[s]
            full = torch.cat([tail.T, mixed[a0:b0]], dim=0)                           # [K-1+n, conv_dim]
            win = full.unfold(0, self.K, 1)                                           # [n, conv_dim, K]
            y = F.silu((win.float() * self.conv_w.float()).sum(-1)).to(x.dtype)
            conv[s] = full[-(self.K - 1):].T
            qh, kh, vh = heads(y)
            # the whole chunk in one kernel on CUDA (the state stays in registers across the tokens)
            gdn_ops.prefill(rec, s, bool(fresh[i]), qh, kh, vh, g[a0:b0], beta[a0:b0], out=out[a0:b0])
        # gated RMSNorm over each value head, then the output projection
        o = out * torch.rsqrt(out.pow(2).mean(-1, keepdim=True) + self.eps)
        o = (self.norm_w * o.to(x.dtype)) * F.silu(z.float())
        return self.out_proj(o.to(x.dtype).reshape(T, nv * dv))

    __call__ = forward


class GatedAttention(Attention):
    """Full attention whose q projection also emits a per-element output gate:
    o_proj(attn(q, k, v) * sigmoid(gate)); q/k norms are zero-centred (weight + 1)."""

    def __init__(self, args, idx, dtype, device, ps=None, rope=None):
        super().__init__(args, idx, dtype, device, ps, rope)
        H, tp = args.hidden_size, self.ps.tp_size
        kv_shards = min(tp, self.nkv_total)
        self.qkv = self.add_module("qkv_proj", MergedColumnLinear(
            H, [args.num_attention_heads * self.d * 2, self.nkv_total * self.d, self.nkv_total * self.d],
            ["q_proj", "k_proj", "v_proj"], args.attention_bias, dtype, device, self.ps, shard_counts=[tp, kv_shards, kv_shards]))
        self.norm_offset = 1.0

    def forward(self, x, positions, meta, k_cache, v_cache):
        T, nq, d = x.shape[0], self.nq, self.d
        qkv = self.qkv(x)
        qg = qkv[:, : nq * d * 2].view(T, nq, 2 * d)
        gate = qg[..., d:].reshape(T, nq * d)
        packed = torch.cat([qg[..., :d].reshape(T, nq * d), qkv[:, nq * d * 2:]], dim=-1)
        return self._attend(packed, positions, meta, k_cache, v_cache, gate=gate)

    __call__ = forward


class NextDecoderLayer(DecoderLayer):
    def __init__(self, args, idx, dtype, device, ps, rope, mlp=None):
        Module.__init__(self)
        H, eps = args.hidden_size, args.rms_norm_eps
        self.linear = args.extra["layer_types"][idx] == "linear_attention"
        self.input_layernorm = self.add_module("input_layernorm", RMSNorm(H, eps, dtype, device, gemma=True))
        if self.linear:
            lin_idx = sum(t == "linear_attention" for t in args.extra["layer_types"][:idx])
            self.mixer = self.add_module("linear_attn", GatedDeltaNet(args, idx, lin_idx, dtype, device, ps))
        else:
            self.mixer = self.add_module("self_attn", GatedAttention(args, idx, dtype, device, ps, rope))
        self.self_attn = self.mixer
        self.post_attention_layernorm = self.add_module("post_attention_layernorm", RMSNorm(H, eps, dtype, device, gemma=True))
        self.mlp = self.add_module("mlp", mlp)
        self.state = None

    def forward(self, x, residual, positions, meta, k_cache, v_cache):
        if residual is None:
            residual = x.clone()
            h = self.input_layernorm(x)
        else:
            h = self.input_layernorm(x, residual=residual)
        h = self.mixer(h, meta, self.state) if self.linear else self.mixer(h, positions, meta, k_cache, v_cache)
        h = self.post_attention_layernorm(h, residual=residual)
        return self.mlp(h), residual

    __call__ = forward


class Qwen3NextCausalLM(DenseCausalLM):
    fused_tp = False
    needs_state = True
    supports_graph = False

    def __init__(self, args, dtype=torch.bfloat16, device="cpu", ps=None):
        e = dict(args.extra)
        n = args.num_hidden_layers
        if not e.get("layer_types"):
            iv = int(e.get("full_attention_interval", 4))
            e["layer_types"] = ["full_attention" if (i + 1) % iv == 0 else "linear_attention" for i in range(n)]
        e["shared_expert_gate"] = True
        e["split_proj"] = args.model_type.lower().startswith("qwen3_5")
        a = dataclasses.replace(args, extra=e, qk_norm=True,
                                n_shared_experts=1 if args.shared_expert_intermediate_size else 0)

        def make_mlp(i):
            if a.is_moe_layer(i):
                return SparseMoeBlock(a, dtype, device, ps)
            return DenseMLP(a.hidden_size, a.intermediate_size, a.hidden_act, dtype, device, ps, fuse_reduce=False)

        super().__init__(a, dtype, device, ps, make_mlp=make_mlp, layer_cls=NextDecoderLayer)
        self.norm.gemma = True
        for layer in self.layers:
            if not layer.linear:
                layer.mixer.q_norm.gemma = layer.mixer.k_norm.gemma = True
        self.state = None

    @property
    def num_kv_heads_local(self):
        return next(l.mixer.nkv for l in self.layers if not l.linear)

    def alloc_state(self, slots):
        lin = [l for l in self.layers if l.linear]
        m = lin[0].mixer
        self.state = LinearStateCache(len(lin), slots, m.conv_dim, m.K, m.nv, m.dk, m.dv, self.device, self.dtype)
        for l in lin:
            l.state = self.state
        return self.state

    def init_random(self, std=0.02, seed=0):
        super().init_random(std, seed)
        for name, t in self.named_params():          # zero-centred norm weights; decay parameters in a sane range
            if name.endswith("layernorm.weight") or name.endswith("model.norm.weight") or name.endswith("_norm.weight"):
                t.zero_()
            elif name.endswith("linear_attn.norm.weight") or name.endswith("dt_bias"):
                t.fill_(1.0)

    @staticmethod
    def remap_weight(name, w):
        # checkpoints written from the vision-language wrapper nest the decoder under one or more `language_model.`
        while name.startswith("model.language_model."):
            name = "model." + name[len("model.language_model."):]
        name = name.replace(".mlp.shared_expert.", ".mlp.shared_experts.")
        if name.endswith(".mlp.shared_expert_gate.weight"):
            name = name.replace(".mlp.shared_expert_gate.", ".mlp.shared_gate.")
        return [(name, w)]


@register_model("qwen3_next", "qwen3_5_text", "qwen3_5_moe_text", "Qwen3NextForCausalLM", "Qwen3_5ForCausalLM",
                "Qwen3_5MoeForCausalLM")
def build_qwen3_next(args, dtype, device, ps):
    return Qwen3NextCausalLM(args, dtype, device, ps)


class Qwen3_5ForConditionalGeneration(Qwen3NextCausalLM):
    """Qwen3.5 with its vision tower (the Qwen3-VL tower without deepstack mergers); the decoder's full
    attention layers take the interleaved 3-axis rotary table, the linear layers need no positions."""
    mrope_interleaved = True

    def __init__(self, args, dtype=torch.bfloat16, device="cpu", ps=None):
        super().__init__(args, dtype, device, ps)
        from .qwen_vl import VisionTowerV3
        self.visual = self.add_module("visual", VisionTowerV3(args.vision_config or {}, dtype, device))
        half = self.args.rotary_dim // 2
        self.mrope_section = list(args.mrope_section) or [half - 2 * (half // 3), half // 3, half // 3]

    def encode_images(self, pixel_values, grid_thw):
        return self.visual(pixel_values.to(self.device), grid_thw)

    @staticmethod
    def remap_weight(name, w):
        out = []
        for n, t in Qwen3NextCausalLM.remap_weight(name, w):
            out.append((n[len("model."):] if n.startswith("model.visual.") else n, t))
        return out


@register_model("qwen3_5", "qwen3_5_moe", "Qwen3_5ForConditionalGeneration", "Qwen3_5MoeForConditionalGeneration")
def build_qwen3_5_vl(args, dtype, device, ps):
    if not args.vision_config:
        return Qwen3NextCausalLM(args, dtype, device, ps)
    return Qwen3_5ForConditionalGeneration(args, dtype, device, ps)
