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


def _pairs_from_halves(w: torch.Tensor, start: int, width: int, period: int) -> torch.Tensor:
    """Reorders output rows of a projection so that a rotary embedding over (x[i], x[i + width/2])
    pairs becomes one over adjacent pairs: in every block of `period` rows, the `width` rows from
    `start` on are permuted new[2i] = old[i], new[2i+1] = old[i + width/2].  Dot products between
    vectors permuted the same way do not change."""
    half = width // 2
    perm = torch.empty(width, dtype=torch.long)
    perm[0::2] = torch.arange(half)
    perm[1::2] = torch.arange(half) + half
    out = w.clone()
    for b in range(0, w.shape[0], period):
        out[b + start: b + start + width] = w[b + start: b + start + width][perm]
    return out


class DsaIndexer(Module):
    """The lightweight indexer of DeepSeek sparse attention (DSA): per token one index key of
    `index_head_dim` values (cached), per query `index_n_heads` index queries; the score of context
    token t for query s is sum_h w[s,h] * relu(q[s,h] . k[t]) * d^-0.5, and attention only sees the
    `index_topk` best-scored tokens.  Parity: xllm/models/llm/deepseek_v32.h, glm5.h (the indexer of
    the reference's NPU layers) and HuggingFace's GlmMoeDsaIndexer, which the tests compare against."""

    def __init__(self, args, dtype, device, rope):
        super().__init__()
        a = args
        self.nh, self.d, self.rope_d, self.topk = a.index_n_heads, a.index_head_dim, a.qk_rope_head_dim, a.index_topk
        self.rope = rope
        self.interleave = bool(a.indexer_rope_interleave)
        self.wq_b = self.add_module("wq_b", Linear(a.q_lora_rank, self.nh * self.d, False, dtype, device, None))
        self.wk = self.add_module("wk", Linear(a.hidden_size, self.d, False, dtype, device, None))
        self.k_norm_w = self.add_param("k_norm.weight", torch.ones(self.d, dtype=dtype, device=device))
        self.k_norm_b = self.add_param("k_norm.bias", torch.zeros(self.d, dtype=dtype, device=device))
        self.weights_proj = self.add_module("weights_proj", Linear(a.hidden_size, self.nh, False, dtype, device, None))
        self.cache = None            # [n_slots, d]: index keys of every cached token (alloc_cache)

    def alloc_cache(self, n_slots, dtype, device):
        self.cache = torch.zeros(n_slots, self.d, dtype=dtype, device=device)

    def _rope(self, v, positions):
        """v [T, heads, rope_d]"""
        half = self.rope_d // 2
        cs = self.rope.cos_sin[positions.long()].float()
        cos, sin = cs[:, None, :half], cs[:, None, half:]
        vf = v.float()
        if self.interleave:
            x1, x2 = vf[..., 0::2], vf[..., 1::2]
            return torch.stack([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).flatten(-2)
        x1, x2 = vf[..., :half], vf[..., half:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)

    def forward(self, x, q_resid, positions, meta: AttentionMetadata):
        """Writes this step's index keys into the cache and returns (sel [T, k] int64 context positions,
        padded with 0, n_sel [T] int32): the tokens every query row attends to.  k = min(index_topk,
        longest context of the step)."""
        T = x.shape[0]
        q = self.wq_b(q_resid).view(T, self.nh, self.d).float()
        q = torch.cat([self._rope(q[..., :self.rope_d], positions), q[..., self.rope_d:]], dim=-1)
        k = torch.nn.functional.layer_norm(self.wk(x).float(), (self.d,), self.k_norm_w.float(), self.k_norm_b.float(), 1e-6)
        k = torch.cat([self._rope(k[:, None, :self.rope_d], positions)[:, 0], k[:, self.rope_d:]], dim=-1)
        ok = meta.slots >= 0
        self.cache.index_copy_(0, meta.slots[ok].long(), k[ok].to(self.cache.dtype))
        w = self.weights_proj(x).float() * (self.nh ** -0.5) * (self.d ** -0.5)        # [T, nh]
        bt = meta.block_table.long()
        P = self._page
        kmax = min(self.topk, int(meta.max_kv_len) if meta.max_kv_len else int(meta.kv_lens.max()))
        sel = torch.zeros(T, kmax, dtype=torch.long, device=x.device)
        n_sel = torch.zeros(T, dtype=torch.int32, device=x.device)
        cu = meta.cu_q.tolist()
        lens = meta.kv_lens.tolist()
        for s_idx in range(meta.n_seqs):
            r0, r1, L = cu[s_idx], cu[s_idx + 1], lens[s_idx]
            if r1 <= r0 or L <= 0:
                continue
            pos_all = torch.arange(L, device=x.device)
            slots = bt[s_idx, pos_all // P] * P + pos_all % P
            keys = self.cache[slots].float()                                              # [L, d]
            sc = torch.einsum("shd,td->sht", q[r0:r1], keys)
            sc = (torch.relu(sc) * w[r0:r1, :, None]).sum(1)                              # [rows, L]
            qpos = positions[r0:r1].long()
            sc = sc.masked_fill(pos_all[None, :] > qpos[:, None], float("-inf"))
            kk = min(kmax, L)
            if sc.is_cuda:
                from ..ops import select
                top_v, top_i = select.topk(sc.contiguous(), kk)          # radix selection kernel
                top_i = top_i.long()
            else:
                top = sc.topk(kk, dim=-1)
                top_v, top_i = top.values, top.indices
            valid = torch.isfinite(top_v)
            sel[r0:r1, :kk] = torch.where(valid, top_i, torch.zeros_like(top_i))
            n_sel[r0:r1] = valid.sum(-1).to(torch.int32)
            # selected-but-masked entries (rows whose context is shorter than kk) sort last: compact is implied
            # because topk returns finite scores first
        return sel, n_sel

    __call__ = forward
    _page = 16


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
        self.split_half = bool(getattr(args, "mla_rope_split_half", False))
        self.indexer = None
        if getattr(args, "index_topk", 0) > 0:
            assert self.latent and self.q_lora and tp == 1, "DSA runs on the latent cache, with q_lora, without TP"
            self.indexer = self.add_module("indexer", DsaIndexer(args, dtype, device, rope))

    def named_loaders(self, prefix=""):
        """Checkpoints whose rotary embedding pairs (x[i], x[i + d/2]) get the rope rows of their q and
        k_pe projections reordered at load, so that the adjacent-pair kernels compute the same dot products."""
        for n, f in super().named_loaders(prefix):
            if self.split_half and n.endswith(("q_b_proj.weight", "q_proj.weight")):
                yield n, (lambda w, f=f: f(_pairs_from_halves(w, self.nope, self.rope_d, self.qk_d)))
            elif self.split_half and n.endswith("kv_a_proj_with_mqa.weight"):
                yield n, (lambda w, f=f: f(_pairs_from_halves(w, self.kv_lora, self.rope_d, self.kv_lora + self.rope_d)))
            else:
                yield n, f

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
        q_resid = None
        if self.q_lora:
            q_resid = self.q_a_layernorm(self.q_a_proj(x))
            q = self.q_b_proj(q_resid)
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
        if self.indexer is not None:
            self.indexer._page = cache.shape[-2]
            sel, n_sel = self.indexer(x, q_resid, positions, meta)
            self._sparse_attend(q_cat, cache, meta, positions, sel, n_sel, o_lat)
            out = torch.einsum("thl,hvl->thv", o_lat, w_uv)
            return self.o_proj(out.reshape(T, nh * self.vd))
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

    def _sparse_attend(self, q_cat, cache, meta, positions, sel, n_sel, o_lat):
        """Attention of every query row over ITS selected context tokens: their latent rows are gathered
        into scratch pages (one run of pages per row) and the MLA kernel runs over those, with the
        number of selected tokens as the row's length.  Rows are processed in groups that keep the
        scratch under 256 MB."""
        from ..ops import mla as mla_ops
        T, k = sel.shape
        W = cache.shape[-1]
        page = cache.shape[-2]
        kpad = (k + page - 1) // page * page
        rows_cache = cache.view(-1, W)
        tok = torch.arange(T, device=q_cat.device)
        seq = torch.bucketize(tok, meta.cu_q[1:].contiguous().long(), right=True).clamp_(max=meta.n_seqs - 1)
        bt = meta.block_table.long()
        slots = bt[seq[:, None], sel // page] * page + sel % page                     # [T, k] cache slots
        group = max(1, (256 << 20) // (kpad * W * cache.element_size()))
        for a in range(0, T, group):
            b = min(T, a + group)
            n = b - a
            scratch = torch.zeros(n * kpad // page, page, W, dtype=cache.dtype, device=cache.device)
            scratch.view(n, kpad, W)[:, :k] = rows_cache[slots[a:b]]
            bt_s = torch.arange(n * kpad // page, dtype=torch.int32, device=cache.device).view(n, kpad // page)
            mla_ops.decode(q_cat[a:b], scratch, bt_s, self.scale, seq_lens=n_sel[a:b].contiguous(), out=o_lat[a:b],
                           latent=self.kv_lora)

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
        tensor-op form, which reads lengths on the host and therefore cannot be captured.  The DSA
        indexer sizes its selection from the step's lengths on the host: eager as well."""
        att = self.layers[0].self_attn
        if att.indexer is not None:
            return False
        return not att.latent or (self.args.kv_lora_rank == 512 and self.args.qk_rope_head_dim == 64)

    @property
    def needs_index_cache(self):
        return self.layers[0].self_attn.indexer is not None

    def alloc_index_cache(self, num_blocks: int, block_size: int):
        """Index keys of the DSA indexer: one [slots, index_head_dim] tensor per layer beside the KV cache."""
        for layer in self.layers:
            layer.self_attn.indexer.alloc_cache(num_blocks * block_size, self.dtype, self.device)


# How each family spells its multi-token-prediction layer: module names, order of the two halves of the
# projection input, where the layer lives in the checkpoint.
MTP_KINDS = {
    # DeepSeek-V3 / GLM-4.5 / GLM-5: an extra decoder layer after the last one (deepseek_mtp.h, mtp_model_base.h)
    "deepseek": dict(enorm="enorm", hnorm="hnorm", proj="eh_proj", order="eh", final="shared_head.norm",
                     prefix=lambda a: f"model.layers.{a.num_hidden_layers}.", layer_prefix="", mask_first=False),
    # MiMo: `model.mtp_layers.N.*`, input = [hidden | token] (mimo_mtp.h)
    "mimo": dict(enorm="token_layernorm", hnorm="hidden_layernorm", proj="input_proj", order="he", final="final_layernorm",
                 prefix=lambda a: "model.mtp_layers.0.", layer_prefix="", mask_first=True),
    # Qwen3.5 / Qwen3-Next: `mtp.*` with the layer under `mtp.layers.0.` (qwen3_5_mtp_base.h)
    "qwen3_5": dict(enorm="pre_fc_norm_embedding", hnorm="pre_fc_norm_hidden", proj="fc", order="eh", final="norm",
                    prefix=lambda a: "mtp.", layer_prefix="layers.0.", mask_first=False),
}


def mtp_kind_of(args) -> str:
    mt = args.model_type.lower()
    if mt.startswith("mimo"):
        return "mimo"
    if mt.startswith("qwen3_5") or mt.startswith("qwen3_next"):
        return "qwen3_5"
    return "deepseek"


class MTPDraft(Module):
    """One multi-token-prediction layer: the draft for position t+2 is computed from the target's
    hidden state at t and the embedding of token t+1:
    h' = layer(proj([norm_e(embed(tok)), norm_h(h)])) ; logits = lm_head(final_norm(h')),
    with the embedding and the lm_head shared with the target.  `kind` selects the family's spelling
    (MTP_KINDS); the layer itself is the family's decoder layer.
    Parity: xllm/models/llm/deepseek_mtp.h, mimo_mtp.h, qwen3_5_mtp.h, runtime/mtp_worker_impl.cpp:1245-1850."""

    def __init__(self, args, target, dtype, device, ps=None, layer_cls=None, kind: str = None):
        super().__init__()
        self.args = args
        self.ps = ps or single()
        self.kind = kind or mtp_kind_of(args)
        k = self.spec = MTP_KINDS[self.kind]
        self.embed = target.embed          # shared with the target model
        self.lm_head = target.lm_head
        H = args.hidden_size
        gemma = self.kind == "qwen3_5"     # zero-centred norm weights
        self.enorm = self.add_module(k["enorm"], RMSNorm(H, args.rms_norm_eps, dtype, device, gemma=gemma))
        self.hnorm = self.add_module(k["hnorm"], RMSNorm(H, args.rms_norm_eps, dtype, device, gemma=gemma))
        self.eh_proj = self.add_module(k["proj"], Linear(2 * H, H, False, dtype, device, self.ps))
        rope = target.rope
        if self.kind == "deepseek" and layer_cls is None and args.kv_lora_rank:
            mlp = SparseMoeBlock(args, dtype, device, self.ps) if args.num_experts > 0 else \
                DenseMLP(H, args.intermediate_size, args.hidden_act, dtype, device, self.ps)
            self.layer = self.add_module("layer", DeepseekDecoderLayer(args, 0, dtype, device, self.ps, rope, mlp))
        elif self.kind == "qwen3_5" and layer_cls is None:
            from .qwen3_next import NextDecoderLayer
            a = target.args                 # the target's completed arguments (layer types, projections)
            full = next(i for i, t in enumerate(a.extra["layer_types"]) if t != "linear_attention")
            mlp = SparseMoeBlock(a, dtype, device, self.ps) if a.num_experts > 0 else \
                DenseMLP(H, a.intermediate_size, a.hidden_act, dtype, device, self.ps, fuse_reduce=False)
            self.layer = self.add_module("layer", NextDecoderLayer(a, full, dtype, device, self.ps, rope, mlp))
            self.layer.mixer.q_norm.gemma = self.layer.mixer.k_norm.gemma = True
        else:
            mlp = SparseMoeBlock(args, dtype, device, self.ps) if args.num_experts > 0 else \
                DenseMLP(H, args.intermediate_size, args.hidden_act, dtype, device, self.ps)
            cls = layer_cls or DecoderLayer
            self.layer = self.add_module("layer", cls(args, 0, dtype, device, self.ps, rope, mlp))
        self.norm = self.add_module(k["final"], RMSNorm(H, args.rms_norm_eps, dtype, device, gemma=gemma))

    def checkpoint_name(self, name: str) -> str:
        """Name of parameter `name` of this module in the family's checkpoint."""
        k = self.spec
        prefix = k["prefix"](self.args)
        if name.startswith("layer."):
            return prefix + k["layer_prefix"] + name[len("layer."):]
        return prefix + name

    def load_from_checkpoint(self, weights, strict: bool = True) -> int:
        """Picks the MTP tensors out of a checkpoint's (name, tensor) stream; the shared embedding and
        head copies some checkpoints carry beside them are skipped.  Returns the number of tensors used."""
        k = self.spec
        prefix = k["prefix"](self.args)
        top = {k["enorm"], k["hnorm"], k["proj"], k["final"].split(".")[0]}
        mapped = []
        for name, w in weights:
            if not name.startswith(prefix):
                continue
            n = name[len(prefix):]
            head = n.split(".")[0]
            if head in ("embed_tokens",) or n.startswith("shared_head.head"):
                continue
            if head in top:
                mapped.append((n, w))
            elif k["layer_prefix"] and n.startswith(k["layer_prefix"]):
                mapped.append(("layer." + n[len(k["layer_prefix"]):], w))
            elif not k["layer_prefix"]:
                mapped.append(("layer." + n, w))
        if mapped:
            self.load_weights(mapped, strict=strict)
        return len(mapped)

    def forward(self, tokens, prev_hidden, positions, meta, k_cache, v_cache):
        comm = self.ps.comm
        if comm is not None and tokens.is_cuda:
            comm.begin_forward(tokens.shape[0])
        emb = self.embed(tokens)
        if self.spec["mask_first"]:          # the embedding at position 0 has no predecessor state
            emb = emb.masked_fill((positions == 0)[:, None], 0)
        e = self.enorm(emb)
        h = self.hnorm(prev_hidden)
        x = self.eh_proj(torch.cat([e, h] if self.spec["order"] == "eh" else [h, e], dim=-1))
        y, residual = self.layer(x, None, positions, meta, k_cache, v_cache)
        if comm is not None and x.is_cuda and self.kind == "deepseek":
            h = comm.allreduce_norm(x.shape[0], residual, self.norm.weight, self.norm.eps)
            comm.end_forward()
            return h
        if comm is not None and x.is_cuda:
            comm.end_forward()
        return self.norm(y, residual=residual)

    def logits(self, hidden_rows):
        return self.lm_head(hidden_rows)


# DeepSeek-V3.2 and GLM-5 (`glm_moe_dsa`) are this decoder with the DSA indexer in every attention layer
# (ModelArgs.index_topk > 0); JoyAI-LLM-Flash is the DeepSeek-V2 decoder under another name
# (xllm/models/llm/deepseek_v32.h, glm5.h, joyai_llm_flash.h).
@register_model("deepseek_v2", "deepseek_v3", "kimi_k2", "DeepseekV2ForCausalLM", "DeepseekV3ForCausalLM",
                "deepseek_v32", "DeepseekV32ForCausalLM", "glm_moe_dsa", "GlmMoeDsaForCausalLM",
                "joyai_llm_flash", "JoyAILLMFlashForCausalLM")
def build_deepseek(args, dtype, device, ps):
    return DeepseekCausalLM(args, dtype, device, ps)
