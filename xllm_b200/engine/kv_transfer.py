"""PD disaggregation data plane: push KV blocks of a finished prefill to the decode GPU.

Parity: KVCacheTransfer push mode with per-layer synchronisation
(xllm/core/framework/kv_cache_transfer/kv_cache_transfer.h:63-165, llm_worker_impl.cpp:280-305),
which the reference implements with Mooncake on non-CUDA back ends only.  Here the prefill side
writes straight into the decode side's KV cache over NVLink with `xllm_kv_push` (plain peer stores,
16 bytes per thread) one layer at a time, so layer l can be pushed while layer l+1 computes, and
publishes a per-layer flag; the decode side waits on the flag with a bounded device-side wait.
KV heads are re-sliced when the two sides use different TP degrees (`head ranges`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

from ..ops import _lib
from ..ops._lib import I, L, P, check, ptr, stream
import ctypes

_lib.register_signature("xllm_kv_push", [P, P, P, I, L, L, L, I, I, I, P, ctypes.c_uint32, P, P])
_lib.register_signature("xllm_kv_wait", [P, ctypes.c_uint32, P, ctypes.c_longlong, P])
_lib.register_signature("xllm_kv_wait_many", [P, I, ctypes.c_uint32, P, ctypes.c_longlong, P])


def plan_head_slices(src_tp: int, src_rank: int, dst_tp: int, n_kv_heads: int) -> List[Tuple[int, int, int, int]]:
    """Which destination ranks need which of this source rank's KV heads.

    Returns (dst_rank, src_head0, dst_head0, n_heads) tuples — the reshard plan for P and D
    instances with different TP degrees (the reference's ReshardPlanner, reshard_planner.cpp)."""
    def owned(tp, r):
        per = max(1, n_kv_heads // tp)
        first = (r * n_kv_heads // tp) if tp <= n_kv_heads else (r * n_kv_heads // tp)
        return first, per
    s0, sn = owned(src_tp, src_rank)
    out = []
    for d in range(dst_tp):
        d0, dn = owned(dst_tp, d)
        lo, hi = max(s0, d0), min(s0 + sn, d0 + dn)
        if hi > lo:
            out.append((d, lo - s0, lo - d0, hi - lo))
    return out


@dataclass
class PushTarget:
    """Peer-mapped base pointers of the destination KV cache: ptrs[layer][0|1] (K, V)."""
    layer_ptrs: List[Tuple[int, int]]
    block_bytes: int
    flag_ptr: int          # uint32[n_layers] on the receiver
    head0: int = 0


class KVPusher:
    def __init__(self, kv_caches, block_size: int, device):
        self.kv = kv_caches
        k0 = kv_caches[0][0]
        self.nkv, self.page, self.d = k0.shape[1], k0.shape[2], k0.shape[3]
        self.head_bytes = self.page * self.d * k0.element_size()
        self.block_bytes = self.nkv * self.head_bytes
        self.arrive = torch.zeros(1, dtype=torch.int32, device=device)
        self.device = device

    def push_layer(self, layer: int, pairs: torch.Tensor, target: PushTarget, epoch: int, src_head0=0, n_heads=None):
        """pairs: int32 [n, 2] device tensor (source block, destination block)."""
        n_heads = n_heads or self.nkv
        lib = _lib.load()
        for which in (0, 1):
            last = which == 1
            check(lib.xllm_kv_push(ptr(self.kv[layer][which]), target.layer_ptrs[layer][which], ptr(pairs), pairs.shape[0],
                                   self.block_bytes, target.block_bytes, self.head_bytes, src_head0, target.head0, n_heads,
                                   target.flag_ptr + 4 * layer if last else None, epoch, ptr(self.arrive), stream()),
                  "kv_push")

    def push_all(self, pairs, target, epoch):
        for l in range(len(self.kv)):
            self.push_layer(l, pairs, target, epoch)


def wait_layer(flags: torch.Tensor, layer: int, epoch: int, status: torch.Tensor, budget_cycles: int = 2_000_000_000):
    """Device-side bounded wait for layer `layer` of transfer `epoch`; status[0] = 1 on expiry."""
    check(_lib.load().xllm_kv_wait(flags.data_ptr() + 4 * layer, epoch, ptr(status), budget_cycles, stream()), "kv_wait")
