"""Fused mixture-of-experts layer: route -> permute -> grouped GEMM (gate|up) -> SiLU·mul ->
grouped GEMM (down) -> weighted finalize.

On CUDA every stage is a kernel of this library (`csrc/kernels/moe.cu` + the grouped mode of the
tcgen05 GEMM); the reference calls FlashInfer's CUTLASS MoE runner for the same job
(xllm/core/kernels/cuda/moe/fused_moe.cpp:23-123, layers/cuda/fused_moe.cpp:96-124).
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import F, I, L, P, check, ptr, stream

_lib.register_signature("xllm_moe_route", [P, I, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P])
_lib.register_signature("xllm_moe_offsets", [P, P, P, P, I, I, I, P])
_lib.register_signature("xllm_moe_permute", [P, P, P, P, P, P, I, I, I, P])
_lib.register_signature("xllm_moe_finalize", [P, P, P, P, P, I, I, I, P])
_lib.register_signature("xllm_gemm_bf16_grouped", [P, P, P, P, I, I, I, I, L, L, P])
_lib.register_signature("xllm_gemm_bf16_grouped_act_mul", [P, P, P, P, I, I, I, I, L, L, I, P])


def route_reference(logits, top_k, scoring="softmax", bias=None, n_group=1, topk_group=1, renorm=True, scale=1.0):
    """Returns (ids [T,K] int64, weights [T,K] fp32)."""
    x = logits.float()
    scores = torch.softmax(x, -1) if scoring == "softmax" else torch.sigmoid(x)
    sel = scores + bias.float() if bias is not None else scores
    if n_group > 1 and topk_group < n_group:
        T, E = sel.shape
        g = sel.view(T, n_group, E // n_group)
        gs = g.topk(2, dim=-1).values.sum(-1) if bias is not None else g.max(-1).values
        keep = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, gs.topk(topk_group, dim=-1).indices, True)
        sel = sel.masked_fill(~keep[:, :, None].expand_as(g).reshape(T, E), float("-inf"))
    ids = sel.topk(top_k, dim=-1).indices
    w = scores.gather(1, ids)
    if renorm:
        w = w / w.sum(-1, keepdim=True)
    return ids, w * scale


def fused_moe_reference(x, logits, w_gate_up, w_down, top_k, scoring="softmax", bias=None, n_group=1, topk_group=1,
                        renorm=True, scale=1.0, expert_begin=0, shared_out=None, act="silu"):
    ids, w = route_reference(logits, top_k, scoring, bias, n_group, topk_group, renorm, scale)
    out = torch.zeros_like(x, dtype=torch.float32)
    if shared_out is not None:
        out += shared_out.float()
    E_local = w_gate_up.shape[0]
    for e in range(E_local):
        ge = e + expert_begin
        tok, kk = torch.nonzero(ids == ge, as_tuple=True)
        if tok.numel() == 0:
            continue
        h = (x[tok].float() @ w_gate_up[e].float().T).to(x.dtype).float()
        d = h.shape[-1] // 2
        a = (torch.nn.functional.silu(h[:, :d]) * h[:, d:]).to(x.dtype).float()
        y = (a @ w_down[e].float().T).to(x.dtype).float()
        out.index_add_(0, tok, y * w[tok, kk, None])
    return out.to(x.dtype)


class MoeWorkspace:
    """Static-size buffers of one MoE layer shape (sized for max_tokens; reusable across layers)."""

    def __init__(self, max_tokens, top_k, n_experts, n_local, hidden, inter, device, dtype=torch.bfloat16):
        self.rows = (max_tokens * top_k + n_local * 127 + 127) // 128 * 128
        self.max_tiles = self.rows // 128
        i32 = dict(dtype=torch.int32, device=device)
        self.counts = torch.zeros(n_experts, **i32)
        self.offsets = torch.zeros(n_experts, **i32)
        self.tile_expert = torch.full((self.max_tiles,), -1, **i32)
        self.meta = torch.zeros(4, **i32)
        self.topk_ids = torch.zeros(max_tokens * top_k, **i32)
        self.slot = torch.zeros(max_tokens * top_k, **i32)
        self.rows_of = torch.zeros(max_tokens * top_k, **i32)
        self.topk_w = torch.zeros(max_tokens * top_k, dtype=torch.float32, device=device)
        self.xp = torch.zeros(self.rows, hidden, dtype=dtype, device=device)
        self.h = torch.zeros(self.rows, 2 * inter, dtype=dtype, device=device)
        self.a = torch.zeros(self.rows, inter, dtype=dtype, device=device)
        self.y = torch.zeros(self.rows, hidden, dtype=dtype, device=device)
        self.max_tokens = max_tokens


def fused_moe(x, logits, w_gate_up, w_down, top_k, scoring="softmax", bias=None, n_group=1, topk_group=1,
              renorm=True, scale=1.0, expert_begin=0, n_experts=None, shared_out=None, ws: MoeWorkspace = None,
              out=None, w_scales=None, interleaved=False):
    """x [T,H], logits [T,E]; w_gate_up [E_local, 2I, H], w_down [E_local, H, I] -> [T,H].
    `interleaved`: every expert's gate|up rows are stored in groups of 128 = [64 gate | the 64 up rows of the
    same features] (`ops.gemm_tcgen05.interleave_gate_up`); the first grouped GEMM then applies SiLU(gate) * up
    in its epilogue and the [rows, 2I] intermediate is never written.
    `w_scales` = (s_gate_up [E_local, 2I/128, H/128], s_down [E_local, H/128, I/128]): the weights are e4m3
    with 128 x 128 block scales and both grouped GEMMs run block-scaled in fp8 (the rows are quantised
    per token in groups of 128 before each of them)."""
    if not x.is_cuda:
        if interleaved:
            from .gemm_tcgen05 import deinterleave_gate_up
            w_gate_up = torch.cat(deinterleave_gate_up(w_gate_up), dim=-2)
        if w_scales is not None:
            from . import fp8
            w_gate_up = torch.stack([fp8.dequant_block128_ref(w_gate_up[e], w_scales[0][e], x.dtype) for e in range(w_gate_up.shape[0])])
            w_down = torch.stack([fp8.dequant_block128_ref(w_down[e], w_scales[1][e], x.dtype) for e in range(w_down.shape[0])])
        return fused_moe_reference(x, logits, w_gate_up, w_down, top_k, scoring, bias, n_group, topk_group, renorm,
                                   scale, expert_begin, shared_out)
    from . import _count, act_and_mul
    lib = _lib.load()
    T, H = x.shape
    E = logits.shape[1]
    E_local, I2, _ = w_gate_up.shape
    inter = I2 // 2
    if ws is None or ws.max_tokens < T:
        ws = MoeWorkspace(T, top_k, E, E_local, H, inter, x.device, x.dtype)
    s = stream()
    lf = logits.dtype == torch.float32
    if not lf and logits.dtype != torch.bfloat16:
        logits, lf = logits.float(), True
    check(lib.xllm_moe_route(ptr(logits), int(lf), ptr(bias), ptr(ws.topk_ids), ptr(ws.topk_w), ptr(ws.counts),
                             ptr(ws.slot), T, E, top_k, n_group, topk_group, 0 if scoring == "softmax" else 1,
                             int(renorm), float(scale), expert_begin, expert_begin + E_local, s), "moe_route")
    check(lib.xllm_moe_offsets(ptr(ws.counts), ptr(ws.offsets), ptr(ws.tile_expert), ptr(ws.meta), E, ws.max_tiles,
                               expert_begin, s), "moe_offsets")
    check(lib.xllm_moe_permute(ptr(ws.xp), ptr(ws.rows_of), ptr(x), ptr(ws.topk_ids), ptr(ws.slot), ptr(ws.offsets),
                               T, top_k, H, s), "moe_permute")
    if w_scales is not None:
        from . import fp8
        xq, xs = fp8.quant_group128(ws.xp)
        fp8.block_scaled_mm_grouped(xq, xs, w_gate_up, w_scales[0], ws.tile_expert, ws.h)
        act_and_mul(ws.h, "silu", out=ws.a)
        aq, as_ = fp8.quant_group128(ws.a)
        fp8.block_scaled_mm_grouped(aq, as_, w_down, w_scales[1], ws.tile_expert, ws.y)
    else:
        if interleaved:
            check(lib.xllm_gemm_bf16_grouped_act_mul(ptr(ws.xp), ptr(w_gate_up), ptr(ws.a), ptr(ws.tile_expert), ws.rows,
                                                     I2, H, E_local, H, inter, 1, s), "moe_gemm1_act")
        else:
            check(lib.xllm_gemm_bf16_grouped(ptr(ws.xp), ptr(w_gate_up), ptr(ws.h), ptr(ws.tile_expert), ws.rows, I2, H,
                                             E_local, H, I2, s), "moe_gemm1")
            act_and_mul(ws.h, "silu", out=ws.a)
        check(lib.xllm_gemm_bf16_grouped(ptr(ws.a), ptr(w_down), ptr(ws.y), ptr(ws.tile_expert), ws.rows, H, inter,
                                         E_local, inter, H, s), "moe_gemm2")
    if out is None:
        out = torch.empty_like(x)
    check(lib.xllm_moe_finalize(ptr(out), ptr(ws.y), ptr(ws.rows_of), ptr(ws.topk_w), ptr(shared_out), T, top_k, H, s),
          "moe_finalize")
    _count(6)
    return out
