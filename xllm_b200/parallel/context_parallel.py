"""Context parallelism: shard a long sequence over ranks for prefill (CP) and shard the KV cache of
running sequences over ranks for decode (DCP / kv_split).

Parity: the reference's model-side CP (tokens sharded after the embedding in load-balanced
"previous / next half" pairs, KV all-gathered per layer, outputs restored before the LM head:
xllm/core/framework/parallel_state/parallel_args.h:167-183, collective_communicator.cpp:332-348) and
DCP (every rank attends to its KV shard; outputs and log-sum-exps are all-gathered and merged:
xllm/core/layers/mlu/dcp_attention_merge.cpp:26-75) — both NPU/MLU-only there.

What is here: the sharding maps, the merge of partial attention states (the same math as the
split-KV merge kernel `xllm_attn_merge`), and reference-level CP / DCP attention over
torch.distributed groups, used by the tests and as the oracle for device kernels.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def zigzag_shards(n_tokens: int, cp: int) -> List[torch.Tensor]:
    """Token indices per rank: the sequence is cut into 2*cp chunks and rank r takes chunks r and
    2*cp-1-r, so that causal attention work is balanced (early chunks are cheap, late ones dear)."""
    bounds = [round(i * n_tokens / (2 * cp)) for i in range(2 * cp + 1)]
    chunks = [torch.arange(bounds[i], bounds[i + 1]) for i in range(2 * cp)]
    return [torch.cat([chunks[r], chunks[2 * cp - 1 - r]]) for r in range(cp)]


def restore_order(parts: List[torch.Tensor], shards: List[torch.Tensor]) -> torch.Tensor:
    """Inverse of the sharding: rows of `parts[r]` go back to positions `shards[r]`."""
    n = sum(len(s) for s in shards)
    out = torch.empty((n,) + tuple(parts[0].shape[1:]), dtype=parts[0].dtype, device=parts[0].device)
    for p, s in zip(parts, shards):
        out[s.to(out.device)] = p
    return out


def attention_with_lse(q, k, v, scale: float, q_pos=None, k_pos=None, causal=True) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [Tq, H, D], k/v [Tk, Hkv, D]; positions give the absolute token index of every row (for the
    causal mask of sharded sequences).  Returns (out [Tq, H, D] fp32, lse [Tq, H] fp32, natural log)."""
    H, Hkv = q.shape[1], k.shape[1]
    kk = k.float().repeat_interleave(H // Hkv, dim=1)
    vv = v.float().repeat_interleave(H // Hkv, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kk) * scale
    if causal:
        qp = q_pos if q_pos is not None else torch.arange(q.shape[0], device=q.device)
        kp = k_pos if k_pos is not None else torch.arange(k.shape[0], device=q.device)
        s = s.masked_fill((kp[None, :] > qp[:, None])[None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                                  # [H, Tq]
    p = torch.exp(s - lse[..., None])
    p = torch.nan_to_num(p, nan=0.0)                                   # rows with nothing visible
    out = torch.einsum("hqk,khd->qhd", p, vv)
    return out, lse.transpose(0, 1)


def merge_states(outs: List[torch.Tensor], lses: List[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Combine attention computed over disjoint KV subsets: out = sum_i softmax_i-weight * out_i."""
    L = torch.stack(lses)                                              # [n, Tq, H]
    m = L.max(dim=0).values
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w = torch.exp(L - m)                                               # -inf -> 0
    denom = w.sum(0)
    out = (torch.stack(outs) * w[..., None]).sum(0) / denom.clamp_min(1e-38)[..., None]
    return out, m + torch.log(denom.clamp_min(1e-38))


def dcp_decode_attention(q, k_shard, v_shard, k_pos_shard, scale: float, group=None):
    """Decode with the KV of every sequence split over the ranks of `group`: q [B=1.., H, D] is
    replicated, each rank holds k/v rows `k_pos_shard`; partial states are all-gathered and merged."""
    o, lse = attention_with_lse(q, k_shard, v_shard, scale, causal=False)
    if group is None or dist.get_world_size(group) == 1:
        return o
    n = dist.get_world_size(group)
    os_, ls_ = [torch.empty_like(o) for _ in range(n)], [torch.empty_like(lse) for _ in range(n)]
    dist.all_gather(os_, o.contiguous(), group=group)
    dist.all_gather(ls_, lse.contiguous(), group=group)
    return merge_states(os_, ls_)[0]


def cp_prefill_attention(q_local, k_local, v_local, pos_local, scale: float, group=None):
    """Causal prefill with the sequence zig-zag sharded over `group`: K/V (and their positions) are
    all-gathered, every rank attends with its own queries."""
    if group is None or dist.get_world_size(group) == 1:
        return attention_with_lse(q_local, k_local, v_local, scale, pos_local, pos_local)[0]
    n = dist.get_world_size(group)
    sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(n)]
    dist.all_gather(sizes, torch.tensor([k_local.shape[0]], dtype=torch.int64), group=group)
    mx = int(max(s.item() for s in sizes))

    def gather(x):
        pad = torch.zeros((mx,) + tuple(x.shape[1:]), dtype=x.dtype)
        pad[: x.shape[0]] = x
        bufs = [torch.empty_like(pad) for _ in range(n)]
        dist.all_gather(bufs, pad, group=group)
        return torch.cat([b[: int(s.item())] for b, s in zip(bufs, sizes)])

    return attention_with_lse(q_local, gather(k_local), gather(v_local), scale, pos_local, gather(pos_local))[0]
