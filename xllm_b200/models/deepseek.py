"""DeepSeek-V2 / V3 family: multi-head latent attention (MLA) + sigmoid grouped-routing MoE with
shared experts, and the multi-token-prediction (MTP) draft layer.

Parity: the reference has DeepSeek only for non-CUDA back ends (xllm/models/llm/deepseek_v2.h,
deepseek_v3.h; MLA blueprint xllm/core/layers/dcu/deepseek_v2_attention.cpp:242-433;
deepseek_mtp.h).  MLA has two forms here.

Materialised (default): the latent c_kv is expanded through kv_b_proj into per-head K (nope | rope)
and V, heads are padded to 256 and laid out [rope | nope | pad] so that the fused rope/KV-write
kernel and the paged attention kernels of the dense models are reused unchanged (dot products do
not depend on the order of head dimensions as long as Q and K agree).  Its price is KV-cache size.

Latent (`ModelArgs.mla_latent_cache`): the paged cache holds one row of kv_lora_rank + rope
values per token, shared by all heads ([normed c_kv | rotated k_pe], 576 values for DeepSeek-V3
against 128 heads x 512 in the other form).  Queries are absorbed into the latent space
(q_nope W_UK), attention is multi-query over the latent rows, and the result is expanded through
W_UV.  This form runs on batched matrix products of the tensor library (a gather of the context
rows, two batched GEMMs and a masked softmax per group of rows); a fused tcgen05 decode kernel over
the latent cache is not built.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from .layers import AttentionMetadata, DenseMLP, LMHead, Linear, Module, RMSNorm, RotaryEmbedding, VocabEmbedding
from .qwen import DecoderLayer, DenseCausalLM
from .qwen_moe import SparseMoeBlock
from .registry import register_model
from ..parallel.state import single

PAD_D = 256


def _yarn_mscale(scale, mscale):
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


class MLAAttention(Module):
    def __init__(self, args, layer_idx, dtype, device, ps=None, rope=None):
        super().__init__()
        self.ps = ps or single()
        tp = self.ps.tp_size
        a = args
        self.nh = a.num_attention_heads // tp
        self.nope, self.rope_d, self.vd = a.qk_nope_head_dim, a.qk_rope_head_dim, a.v_head_dim
        self.qk_d = self.nope + self.rope_d
        H = a.hidden_size
        self.q_lora = a.q_lora_rank
        qn = "fp8_block" if getattr(a, "fp8_execution", False) else None
        if self.q_lora:
            self.q_a_proj = self.add_module("q_a_proj", Linear(H, self.q_lora, False, dtype, device, self.ps, quant=qn))
            self.q_a_layernorm = self.add_module("q_a_layernorm", RMSNorm(self.q_lora, a.rms_norm_eps, dtype, device))
            self.q_b_proj = self.add_module("q_b_proj", Linear(self.q_lora, a.num_attention_heads * self.qk_d, False, dtype,
                                                               device, self.ps, parallel="column", quant=qn))
        else:
            self.q_proj = self.add_module("q_proj", Linear(H, a.num_attention_heads * self.qk_d, False, dtype, device,
                                                           self.ps, parallel="column", quant=qn))
        self.kv_a_proj = self.add_module("kv_a_proj_with_mqa", Linear(H, a.kv_lora_rank + self.rope_d, False, dtype, device,
                                                                      self.ps, quant=qn))
        self.kv_a_layernorm = self.add_module("kv_a_layernorm", RMSNorm(a.kv_lora_rank, a.rms_norm_eps, dtype, device))
        self.kv_b_proj = self.add_module("kv_b_proj", Linear(a.kv_lora_rank, a.num_attention_heads * (self.nope + self.vd), False,
                                                             dtype, device, self.ps, parallel="column"))
        self.o_proj = self.add_module("o_proj", Linear(a.num_attention_heads * self.vd, H, False, dtype, device, self.ps,
                                                       parallel="row", quant=qn))
        self.kv_lora = a.kv_lora_rank
        self.rope = rope
        self.scale = 1.0 / math.sqrt(self.qk_d)
        rs = a.rope_scaling or {}
        if rs.get("mscale_all_dim"):
            m = _yarn_mscale(float(rs.get("factor", 1.0)), float(rs["mscale_all_dim"]))
            self.scale *= m * m
        # on this rank the cache sees `nh` KV heads of PAD_D
        self.nq = self.nkv = self.nh
        self.d = PAD_D
        self.latent = bool(getattr(args, "mla_latent_cache", False))
        if self.latent:
            self.nkv, self.d = 1, self.kv_lora + self.rope_d

    # ------------------------------------------------------------------ latent-cache form
    def _rope(self, v, positions):
        """Rotary embedding on adjacent pairs of the last dimension; v [T, heads, rope_d]."""
        half = self.rope_d // 2
        cs = self.rope.cos_sin[positions.long()].float()
        cos, sin = cs[:, None, :half], cs[:, None, half:]
        vf = v.float()
        x1, x2 = vf[..., 0::2], vf[..., 1::2]
        return torch.stack([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).flatten(-2).to(v.dtype)

    def _forward_latent(self, x, positions, meta: AttentionMetadata, cache):
        """Absorbed form over the latent cache: q_abs = q_nope . W_UK, attention against rows
        [c_kv | k_pe] (one shared "head" of 576), out = (P . c_kv) . W_UV.  The cache write, both rotary
        embeddings and the attention are kernels of ops.mla; nothing is read back to the host."""
        from ..ops import mla as mla_ops
        T, nh, L, r = x.shape[0], self.nh, self.kv_lora, self.rope_d
        if self.q_lora:
            q = self.q_b_proj(self.q_a_layernorm(self.q_a_proj(x)))
        else:
            q = self.q_proj(x)
        q = q.view(T, nh, self.qk_d)
        kv_a = self.kv_a_proj(x)
        w = self.kv_b_proj.weight.view(nh, self.nope + self.vd, L)
        w_uk, w_uv = w[:, :self.nope], w[:, self.nope:]        # [nh, nope, L], [nh, vd, L]
        q_cat = torch.empty((T, nh, L + r), dtype=x.dtype, device=x.device)
        q_cat[..., :L] = torch.einsum("thn,hnl->thl", q[..., :self.nope], w_uk)
        mla_ops.cache_write(kv_a, self.kv_a_layernorm.weight, self.kv_a_layernorm.eps, self.rope.cos_sin, positions,
                            meta.slots, cache, q[..., self.nope:], q_cat)
        o_lat = torch.empty((T, nh, L), dtype=x.dtype, device=x.device)
        nd = meta.n_decode
        if nd > 0:                                            # one query token per sequence
            mla_ops.decode(q_cat[:nd], cache, meta.block_table, self.scale, seq_lens=meta.kv_lens[:nd], out=o_lat[:nd],
                           latent=L)
        if meta.n_prefill > 0 and T > nd:
            # every token of a prompt chunk is a query row that sees the cache up to its own position
            tok = torch.arange(nd, T, device=x.device, dtype=torch.int32)
            seq = torch.bucketize(tok, meta.cu_q[nd + 1:].contiguous(), right=True).clamp_(max=meta.n_prefill - 1)
            mla_ops.decode(q_cat[nd:], cache, meta.block_table, self.scale, positions=positions[nd:],
                           bt_rows=(seq + nd).to(torch.int32), out=o_lat[nd:], latent=L)
        out = torch.einsum("thl,hvl->thv", o_lat, w_uv)
        return self.o_proj(out.reshape(T, nh * self.vd))

    def forward(self, x, positions, meta: AttentionMetadata, k_cache, v_cache):
        if self.latent:
            return self._forward_latent(x, positions, meta, k_cache)
        T = x.shape[0]
        nh = self.nh
        if self.q_lora:
            q = self.q_b_proj(self.q_a_layernorm(self.q_a_proj(x)))
        else:
            q = self.q_proj(x)
        q = q.view(T, nh, self.qk_d)
        kv_a = self.kv_a_proj(x)
        c_kv, k_pe = kv_a[:, :self.kv_lora], kv_a[:, self.kv_lora:]
        kv = self.kv_b_proj(self.kv_a_layernorm(c_kv.contiguous())).view(T, nh, self.nope + self.vd)
        # packed [q | k | v] with heads of PAD_D laid out [rope | nope | 0]
        packed = torch.zeros(T, 3 * nh, PAD_D, dtype=x.dtype, device=x.device)
        packed[:, :nh, :self.rope_d] = q[..., self.nope:]
        packed[:, :nh, self.rope_d:self.qk_d] = q[..., :self.nope]
        packed[:, nh:2 * nh, :self.rope_d] = k_pe[:, None, :]
        packed[:, nh:2 * nh, self.rope_d:self.qk_d] = kv[..., :self.nope]
        packed[:, 2 * nh:, :self.vd] = kv[..., self.nope:]
        qr = ops.rope_kv_write(packed.view(T, -1), nh, nh, PAD_D, positions, self.rope.cos_sin, self.rope_d,
                               slots=meta.slots, k_cache=k_cache, v_cache=v_cache, interleaved=True)
        out = torch.empty((T, nh, PAD_D), dtype=x.dtype, device=x.device)
        nd = meta.n_decode
        if nd > 0:
            ops.paged_decode_attention(qr[:nd], k_cache, v_cache, meta.block_table[:nd], meta.kv_lens[:nd], self.scale,
                                       splits=meta.decode_splits, workspace=meta.decode_workspace, out=out[:nd])
        if meta.n_prefill > 0:
            ops.paged_prefill_attention(qr, k_cache, v_cache, meta.block_table[nd:], meta.cu_q[nd:], meta.kv_lens[nd:],
                                        meta.max_q_len, self.scale, causal=True, out=out)
        return self.o_proj(out[:, :, :self.vd].reshape(T, nh * self.vd))

    __call__ = forward


class DeepseekDecoderLayer(DecoderLayer):
    def __init__(self, args, idx, dtype, device, ps, rope, mlp):
        Module.__init__(self)
        self.input_layernorm = self.add_module("input_layernorm", RMSNorm(args.hidden_size, args.rms_norm_eps, dtype, device))
        self.self_attn = self.add_module("self_attn", MLAAttention(args, idx, dtype, device, ps, rope))
        self.post_attention_layernorm = self.add_module(
            "post_attention_layernorm", RMSNorm(args.hidden_size, args.rms_norm_eps, dtype, device))
        self.mlp = self.add_module("mlp", mlp)


class DeepseekCausalLM(DenseCausalLM):
    supports_prefill_graph = False
    def __init__(self, args, dtype=torch.bfloat16, device="cpu", ps=None):
        Module.__init__(self)
        self.args = args
        self.ps = ps or single()
        self.dtype = dtype
        self.device = torch.device(device)
        inner = Module()
        self.add_module("model", inner)
        self.embed = inner.add_module("embed_tokens", VocabEmbedding(args.vocab_size, args.hidden_size, dtype, device, self.ps))
        self.rope = RotaryEmbedding(args.qk_rope_head_dim, args.max_position_embeddings, args.rope_theta,
                                    args.rope_scaling, device, True)
        layers = Module()
        inner.add_module("layers", layers)
        self.layers = []
        for i in range(args.num_hidden_layers):
            if args.is_moe_layer(i):
                mlp = SparseMoeBlock(args, dtype, device, self.ps)
            else:
                mlp = DenseMLP(args.hidden_size, args.intermediate_size, args.hidden_act, dtype, device, self.ps,
                               quant="fp8_block" if getattr(args, "fp8_execution", False) else None)
            self.layers.append(layers.add_module(str(i), DeepseekDecoderLayer(args, i, dtype, device, self.ps, self.rope, mlp)))
        self.norm = inner.add_module("norm", RMSNorm(args.hidden_size, args.rms_norm_eps, dtype, device))
        self.lm_head = LMHead(args.vocab_size, args.hidden_size, dtype, device, self.ps,
                              tied=self.embed if args.tie_word_embeddings else None)
        if not args.tie_word_embeddings:
            self.add_module("lm_head", self.lm_head)

    @property
    def num_kv_heads_local(self):
        return self.layers[0].self_attn.nkv

    @property
    def head_dim(self):
        return self.layers[0].self_attn.d

    @property
    def kv_planes(self):
        """2 = separate K and V caches; 1 = one latent cache per layer (the V handle aliases it)."""
        return 1 if self.layers[0].self_attn.latent else 2

    @property
    def supports_graph(self):
        """The latent-cache kernels exist for DeepSeek's widths (512 + 64); other widths run the
        tensor-op form, which reads lengths on the host and therefore cannot be captured."""
        att = self.layers[0].self_attn
        return not att.latent or (self.args.kv_lora_rank == 512 and self.args.qk_rope_head_dim == 64)


class MTPDraft(Module):
    """One multi-token-prediction layer (DeepSeek-V3 `num_nextn_predict_layers`): the draft for
    position t+2 is computed from the target's hidden state at t and the embedding of token t+1:
    h' = layer(eh_proj([enorm(embed(tok)), hnorm(h)])) ; logits = shared_head(norm(h')).
    Parity: xllm/models/llm/deepseek_mtp.h, runtime/mtp_worker_impl.cpp:1245-1850."""

    def __init__(self, args, target: DeepseekCausalLM, dtype, device, ps=None, layer_cls=None):
        super().__init__()
        self.args = args
        self.ps = ps or single()
        self.embed = target.embed          # shared with the target model
        self.lm_head = target.lm_head
        H = args.hidden_size
        self.enorm = self.add_module("enorm", RMSNorm(H, args.rms_norm_eps, dtype, device))
        self.hnorm = self.add_module("hnorm", RMSNorm(H, args.rms_norm_eps, dtype, device))
        self.eh_proj = self.add_module("eh_proj", Linear(2 * H, H, False, dtype, device, self.ps))
        mlp = SparseMoeBlock(args, dtype, device, self.ps) if args.num_experts > 0 else \
            DenseMLP(H, args.intermediate_size, args.hidden_act, dtype, device, self.ps)
        if layer_cls is None:
            self.layer = self.add_module("layer", DeepseekDecoderLayer(args, 0, dtype, device, self.ps, target.rope, mlp))
        else:
            self.layer = self.add_module("layer", layer_cls(args, 0, dtype, device, self.ps, target.rope, mlp))
        self.norm = self.add_module("shared_head.norm", RMSNorm(H, args.rms_norm_eps, dtype, device))

    def forward(self, tokens, prev_hidden, positions, meta, k_cache, v_cache):
        comm = self.ps.comm
        if comm is not None and tokens.is_cuda:
            comm.begin_forward(tokens.shape[0])
        e = self.enorm(self.embed(tokens))
        h = self.hnorm(prev_hidden)
        x = self.eh_proj(torch.cat([e, h], dim=-1))
        y, residual = self.layer(x, None, positions, meta, k_cache, v_cache)
        if comm is not None and x.is_cuda:
            h = comm.allreduce_norm(x.shape[0], residual, self.norm.weight, self.norm.eps)
            comm.end_forward()
            return h
        return self.norm(y, residual=residual)

    def logits(self, hidden_rows):
        return self.lm_head(hidden_rows)


# DeepSeek-V3.2 is not registered: its sparse attention (the DSA indexer) is not implemented, and running
# such a checkpoint with dense attention would silently compute something else.
@register_model("deepseek_v2", "deepseek_v3", "kimi_k2", "DeepseekV2ForCausalLM", "DeepseekV3ForCausalLM")
def build_deepseek(args, dtype, device, ps):
    return DeepseekCausalLM(args, dtype, device, ps)
