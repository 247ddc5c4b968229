"""Sparse-MoE decoders: Qwen3-MoE (softmax top-k routing, no shared expert) and the generic
MoE block reused by DeepSeek-style models (sigmoid grouped routing, shared experts).

Parity: Qwen3MoeDecoderLayer (xllm/core/layers/qwen3_moe_decoder_layer.cpp:141-160), FusedMoE
(layers/cuda/fused_moe.cpp:96-124) and models/llm/qwen3_moe.h.  Expert parallelism places
E / ep experts on each EP rank; with ep_size == 1 every rank holds all experts with the expert
intermediate dimension sharded across the TP group.  Either way a rank produces a partial sum over
"its" part of the experts and the partials are reduced by the same fused all-reduce(+norm) that the
dense layers use — the reference reduces with two NCCL all-reduces (moe_tp then moe_ep).
"""
from __future__ import annotations

import os

import torch

from .. import ops
from ..ops import moe as moe_ops
from .layers import DenseMLP, Linear, Module
from .qwen import DenseCausalLM
from .registry import register_model
from ..parallel.state import single


class SparseMoeBlock(Module):
    def __init__(self, args, dtype, device, ps=None):
        super().__init__()
        self.ps = ps or single()
        self.args = args
        E, H, I = args.num_experts, args.hidden_size, args.moe_intermediate_size
        ep = self.ps.ep_size if self.ps.ep_size > 1 else 1
        tp = self.ps.tp_size
        self.ep = ep
        if ep > 1:
            self.e_local = E // ep
            self.e_begin = self.ps.ep_rank * self.e_local
            self.i_local, i_rank, i_parts = I, 0, 1
        else:
            self.e_local, self.e_begin = E, 0
            self.i_local, i_rank, i_parts = I // tp, self.ps.tp_rank, tp
        self.top_k = args.num_experts_per_tok
        self.gate = self.add_module("gate", Linear(H, E, False, dtype, device, self.ps))  # replicated router
        il = self.i_local
        # block-scaled fp8 experts: e4m3 weights + 128 x 128 scales, grouped block-scaled GEMMs
        self.fp8 = bool(getattr(args, "fp8_execution", False)) and il % 128 == 0 and H % 128 == 0
        if self.fp8:
            from .layers import FP8, _to_fp8_blocks
            self.w_gate_up = torch.zeros(self.e_local, 2 * il, H, dtype=FP8, device=device)
            self.w_down = torch.zeros(self.e_local, H, il, dtype=FP8, device=device)
            self.s_gate_up = torch.ones(self.e_local, 2 * il // 128, H // 128, dtype=torch.float32, device=device)
            self.s_down = torch.ones(self.e_local, H // 128, il // 128, dtype=torch.float32, device=device)
            self._params["experts.gate_up"] = self.w_gate_up
            self._params["experts.down"] = self.w_down
            self._params["experts.gate_up_scale"] = self.s_gate_up
            self._params["experts.down_scale"] = self.s_down

            def put(wt, st, e, r0, rows, w, dim):
                """rows [r0, r0 + rows) of expert e from checkpoint tensor w (sharded along `dim`)."""
                w = w.narrow(dim, i_rank * il, il)
                if w.dtype == FP8:
                    wt[e, r0:r0 + rows].copy_(w)
                else:
                    q, sc = _to_fp8_blocks(w)
                    wt[e, r0:r0 + rows].copy_(q)
                    st[e, r0 // 128: r0 // 128 + sc.shape[0]].copy_(sc)

            def put_s(st, e, r0, sc, dim):
                sc = sc.float().narrow(dim, i_rank * il // 128, il // 128)
                st[e, r0 // 128: r0 // 128 + sc.shape[0]].copy_(sc)

            for e in range(self.e_local):
                ge = e + self.e_begin
                L_ = self._loaders
                L_[f"experts.{ge}.gate_proj.weight"] = lambda w, e=e: put(self.w_gate_up, self.s_gate_up, e, 0, il, w, 0)
                L_[f"experts.{ge}.up_proj.weight"] = lambda w, e=e: put(self.w_gate_up, self.s_gate_up, e, il, il, w, 0)
                L_[f"experts.{ge}.down_proj.weight"] = lambda w, e=e: put(self.w_down, self.s_down, e, 0, H, w, 1)
                L_[f"experts.{ge}.gate_proj.weight_scale_inv"] = lambda sc, e=e: put_s(self.s_gate_up, e, 0, sc, 0)
                L_[f"experts.{ge}.up_proj.weight_scale_inv"] = lambda sc, e=e: put_s(self.s_gate_up, e, il, sc, 0)
                L_[f"experts.{ge}.down_proj.weight_scale_inv"] = lambda sc, e=e: put_s(self.s_down, e, 0, sc, 1)
        else:
            self.w_gate_up = torch.empty(self.e_local, 2 * self.i_local, H, dtype=dtype, device=device)
            self.w_down = torch.empty(self.e_local, H, self.i_local, dtype=dtype, device=device)
            self._params["experts.gate_up"] = self.w_gate_up
            self._params["experts.down"] = self.w_down
        # On the device, without expert parallelism, every expert's gate|up rows are stored in groups of
        # 128 = [64 gate | 64 up of the same features]: the grouped GEMM's epilogue then applies SiLU(gate) * up
        # itself (ops/moe.py).  Expert-parallel layers keep the plain layout (their weights move between ranks).
        self.interleaved = (not self.fp8 and ep == 1 and il % 64 == 0 and dtype == torch.bfloat16
                            and torch.device(device).type == "cuda" and os.environ.get("XLLM_FUSED_ACT", "1") != "0")
        if self.interleaved:
            self.w_gate_up._xllm_interleaved = True
        for e in range(self.e_local if not self.fp8 else 0):
            ge = e + self.e_begin

            def half(e, p):
                """Rows of expert e that hold gate (p = 0) or up (p = 1), as a [il // 64, 64, H] or [il, H] view."""
                if self.interleaved:
                    return self.w_gate_up[e].view(2 * il // 128, 2, 64, H)[:, p]
                return self.w_gate_up[e, p * il:(p + 1) * il]

            def lg(w, e=e):
                half(e, 0).copy_(w.narrow(0, i_rank * il, il).to(dtype).view(half(e, 0).shape))

            def lu(w, e=e):
                half(e, 1).copy_(w.narrow(0, i_rank * il, il).to(dtype).view(half(e, 1).shape))

            def ld(w, e=e):
                self.w_down[e].copy_(w.narrow(1, i_rank * il, il).to(dtype))

            self._loaders[f"experts.{ge}.gate_proj.weight"] = lg
            self._loaders[f"experts.{ge}.up_proj.weight"] = lu
            self._loaders[f"experts.{ge}.down_proj.weight"] = ld
        self.bias = None
        if args.router_bias:
            self.bias = torch.zeros(E, dtype=torch.float32, device=device)
            self.add_param("gate.e_score_correction_bias", self.bias)
        self.shared = None
        if args.n_shared_experts > 0:
            si = args.shared_expert_intermediate_size or args.moe_intermediate_size * args.n_shared_experts
            self.shared = self.add_module("shared_experts", DenseMLP(
                H, si, args.hidden_act, dtype, device, self.ps, reduce=False,
                quant="fp8_block" if getattr(args, "fp8_execution", False) else None))
        self.shared_gate = None
        if self.shared is not None and args.extra.get("shared_expert_gate"):
            self.shared_gate = self.add_module("shared_gate", Linear(H, 1, False, dtype, device, self.ps))
        self._ws = None

    def forward(self, x):
        a = self.args
        T = x.shape[0]
        logits = self.gate(x)
        shared_out = None
        if self.shared is not None:
            # the shared expert is TP-sharded like a dense MLP: its partial joins the routed partial.
            # With EP every rank would add the full shared output, so only the rank that owns
            # expert 0 contributes it.
            hs = self.shared.hidden(x)
            if self.shared.down.fp8 is not None:
                from .layers import _fp8_linear
                shared_out = _fp8_linear(hs, self.shared.down.fp8.q, self.shared.down.fp8.scale)
            else:
                shared_out = ops.linear(hs, self.shared.down.weight)
            if self.shared_gate is not None:               # Qwen2-MoE / Qwen3-Next: sigmoid-gated shared expert
                shared_out = shared_out * torch.sigmoid(self.shared_gate(x).float()).to(shared_out.dtype)
            if self.ep > 1 and self.e_begin != 0 and self.shared.ps.tp_size == 1 and self.ps.dp_size == 1:
                shared_out = None
        if self.ep > 1 and self.ps.dp_size > 1:
            return self._forward_dp(x, logits, shared_out)
        comm = self.ps.comm
        out = comm.partial_buffer(T) if (comm is not None and x.is_cuda) else None
        if self._use_a2a(x, comm):
            return self._forward_a2a(x, logits, shared_out, comm, out)
        if x.is_cuda and (self._ws is None or self._ws.max_tokens < T):
            self._ws = moe_ops.MoeWorkspace(max(T, 256), self.top_k, a.num_experts, self.e_local, a.hidden_size,
                                            self.i_local, x.device, x.dtype)
        y = moe_ops.fused_moe(x, logits, self.w_gate_up, self.w_down, self.top_k, a.scoring_func, self.bias,
                              a.n_group, a.topk_group, a.norm_topk_prob, a.routed_scaling_factor, self.e_begin,
                              a.num_experts, shared_out, self._ws, out,
                              w_scales=(self.s_gate_up, self.s_down) if self.fp8 else None,
                              interleaved=self.interleaved)
        if out is None and self.ps.tp_size > 1:
            y = self.ps.all_reduce(y)
        return y

    # ---- expert load balancing (parallel/eplb_gpu.py): with a store attached the layer counts the tokens
    # every expert receives and its weights can move between the ranks
    expert_store = None

    def _load(self):
        return self.expert_store.load if self.expert_store is not None else None

    def enable_eplb(self):
        """Collective over the expert-parallel group: moves this layer's expert weights into a
        double-buffered symmetric store.  Returns the store (`rebalance()` re-places the experts)."""
        from ..parallel.eplb_gpu import ExpertStore
        ps = self.ps
        group = ps.moe_ep_group if ps.dp_size > 1 or ps.moe_ep_group is not None else ps.tp_group
        rank = ps.ep_rank if ps.ep_size > 1 else ps.tp_rank
        self.expert_store = ExpertStore(self, group or ps.world_group, rank, self.ep)
        return self.expert_store

    # ---- expert parallelism by all-to-all (parallel/ep.py): every rank routes the token rows it owns
    # in the sequence-sharded residual stream, tokens visit the owners of their experts and come
    # back; the rows land in this rank's part of the partial buffer (zeros elsewhere), so the fused
    # all-reduce + norm that follows assembles the full activation without summing duplicates.
    def _use_a2a(self, x, comm) -> bool:
        import os
        return (self.ep > 1 and not self.fp8 and x.is_cuda and comm is not None and self.ep == self.ps.tp_size
                and os.environ.get("XLLM_EP_MODE", "a2a") == "a2a"
                and (getattr(self.ps, "ep_comm", None) is not None or not torch.cuda.is_current_stream_capturing()))

    def _forward_a2a(self, x, logits, shared_out, comm, out):
        a = self.args
        T = x.shape[0]
        ep = getattr(self.ps, "ep_comm", None)
        if ep is None:
            from ..parallel.ep import EpComm
            ep = EpComm(self.ps.tp_group, self.ps.tp_rank, self.ps.tp_size, x.device, a.num_experts, a.hidden_size,
                        self.top_k, max_local_tokens=comm.max_tokens // self.ps.tp_size + 1)
            self.ps.ep_comm = ep
        b, e, _ = comm.shard(T)
        out.zero_()
        if shared_out is not None:
            out.copy_(shared_out)            # TP-sharded shared expert: a partial sum over all rows
        if e > b:
            ep.moe(x[b:e], logits[b:e], self.w_gate_up, self.w_down, a.scoring_func, self.bias, a.n_group, a.topk_group,
                   a.norm_topk_prob, a.routed_scaling_factor, None, out=self._a2a_rows(e - b, x), load=self._load())
            out[b:e] += self._rows[: e - b]
        else:
            ep.moe(x[:0], logits[:0], self.w_gate_up, self.w_down, a.scoring_func, self.bias, a.n_group, a.topk_group,
                   a.norm_topk_prob, a.routed_scaling_factor, None, out=x[:0])   # idle ranks still join the exchange
        return out

    # ---- data-parallel attention: every rank holds DIFFERENT tokens (its own requests) and the
    # experts are spread over all ranks.  On CUDA the tokens go through the all-to-all kernels; the
    # library path (CPU, or XLLM_EP_MODE=gather) is the reference's scheme: all-gather the tokens of
    # all DP ranks (ragged: padded to the longest), run the local experts over everything,
    # all-reduce, keep the own rows (xllm/core/framework/parallel_state/dp_utils.h:55-104).
    def _forward_dp(self, x, logits, shared_out):
        import os

        import torch.distributed as dist
        a = self.args
        ps = self.ps
        group = ps.moe_ep_group or ps.world_group
        T = x.shape[0]
        if x.is_cuda and os.environ.get("XLLM_EP_MODE", "a2a") == "a2a" and \
                (getattr(ps, "ep_comm", None) is not None or not torch.cuda.is_current_stream_capturing()):
            ep = getattr(ps, "ep_comm", None)
            if ep is None:
                from ..parallel.ep import EpComm
                ep = EpComm(group, ps.ep_rank, ps.ep_size, x.device, a.num_experts, a.hidden_size, self.top_k,
                            max_local_tokens=int(getattr(ps, "max_tokens_per_batch", 8192)))
                ps.ep_comm = ep
            return ep.moe(x, logits, self.w_gate_up, self.w_down, a.scoring_func, self.bias, a.n_group, a.topk_group,
                          a.norm_topk_prob, a.routed_scaling_factor, shared_out, load=self._load())
        W = ps.ep_size
        counts = torch.zeros(W, dtype=torch.int64, device=x.device)
        counts[ps.ep_rank] = T
        dist.all_reduce(counts, group=group)
        cl = counts.tolist()
        mx = max(max(cl), 1)
        pad_x = torch.zeros(mx, x.shape[1], dtype=x.dtype, device=x.device)
        pad_l = torch.zeros(mx, logits.shape[1], dtype=logits.dtype, device=x.device)
        pad_x[:T], pad_l[:T] = x, logits
        gx = [torch.empty_like(pad_x) for _ in range(W)]
        gl = [torch.empty_like(pad_l) for _ in range(W)]
        dist.all_gather(gx, pad_x, group=group)
        dist.all_gather(gl, pad_l, group=group)
        ax = torch.cat([g[:n] for g, n in zip(gx, cl)])
        al = torch.cat([g[:n] for g, n in zip(gl, cl)])
        y = moe_ops.fused_moe(ax, al, self.w_gate_up, self.w_down, self.top_k, a.scoring_func, self.bias, a.n_group,
                              a.topk_group, a.norm_topk_prob, a.routed_scaling_factor, self.e_begin, a.num_experts)
        y = y.float() if not y.is_cuda else y
        dist.all_reduce(y, group=group)
        off = sum(cl[: ps.ep_rank])
        mine = y[off:off + T].to(x.dtype)
        return mine + shared_out if shared_out is not None else mine

    def _a2a_rows(self, n, x):
        if getattr(self, "_rows", None) is None or self._rows.shape[0] < n:
            self._rows = torch.empty(max(n, 64), x.shape[1], dtype=x.dtype, device=x.device)
        return self._rows[:n]

    __call__ = forward


def _make_mlp(args, dtype, device, ps):
    def make(i):
        if args.is_moe_layer(i):
            return SparseMoeBlock(args, dtype, device, ps)
        return DenseMLP(args.hidden_size, args.intermediate_size, args.hidden_act, dtype, device, ps)
    return make


@register_model("qwen3_moe", "qwen2_moe", "Qwen3MoeForCausalLM", "Qwen2MoeForCausalLM")
def build_qwen_moe(args, dtype, device, ps):
    m = DenseCausalLM(args, dtype, device, ps, make_mlp=_make_mlp(args, dtype, device, ps))
    return m
