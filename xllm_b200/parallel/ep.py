"""Expert-parallel MoE with a true all-to-all over NVLink peer memory.

`EpComm` owns one symmetric allocation per rank (count matrix, receive buffer for token rows,
buffer of expert outputs) and runs the dispatch / combine kernels of `csrc/kernels/ep_a2a.cu`
around the grouped tcgen05 GEMMs.  Every rank routes only ITS tokens (data-parallel attention
ranks, or the token shard a tensor-parallel rank owns after the reduce-scatter), so a token crosses
NVLink once on the way to each of its experts and once on the way back; the reference's CUDA path
replicates all tokens on all ranks and all-reduces the outputs twice
(xllm/core/layers/cuda/fused_moe.cpp:96-118).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..ops import _lib
from ..ops._lib import F, I, L, P, check, ptr, stream

_EP = [P, P, L, L, L, L, P, P, I, I, I, I, I]
_lib.register_signature("xllm_ep_barrier", _EP + [P])
_lib.register_signature("xllm_ep_publish_counts", _EP + [P, P])
_lib.register_signature("xllm_ep_layout", _EP + [P, P, P, I, P])
_lib.register_signature("xllm_ep_dispatch", _EP + [P, P, P, P, P, I, I, P])
_lib.register_signature("xllm_ep_combine", _EP + [P, P, P, P, I, I, P])
_lib.register_signature("xllm_ep_counts_layout", _EP + [P, P, P, P, I, P])
_lib.register_signature("xllm_ep_dispatch_sync", _EP + [P, P, P, P, P, I, I, P])
_lib.register_signature("xllm_ep_combine_sync", _EP + [P, P, P, P, I, I, P])
_lib.register_signature("xllm_act_and_mul_rows", [P, P, L, P, I, L, I, P])
_lib.register_signature("xllm_ep_set_wait_budget", [ctypes.c_longlong], ctypes.c_longlong)


class EpComm:
    def __init__(self, group, rank: int, world: int, device, n_experts: int, hidden: int, top_k: int,
                 max_local_tokens: int, capacity_rows: int = 0):
        import torch.distributed._symmetric_memory as symm_mem

        self.rank, self.world, self.E, self.H, self.K = rank, world, n_experts, hidden, top_k
        self.e_local = n_experts // world
        self.device = device
        self.max_local_tokens = max_local_tokens
        # worst case every token of every rank picks experts of one rank
        cap = capacity_rows or (max_local_tokens * world * top_k + self.e_local * 127)
        self.cap = (cap + 127) // 128 * 128
        self.max_tiles = self.cap // 128
        al = lambda n: (n + 255) & ~255
        self.cnt_off = 0
        self.recvx_off = al(world * n_experts * 4)
        self.recvy_off = al(self.recvx_off + self.cap * hidden * 2)
        total = al(self.recvy_off + self.cap * hidden * 2)
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.peer_ptrs = self.hdl.buffer_ptrs_dev
        self.signal_ptrs = self.hdl.signal_pad_ptrs_dev
        self.sig_off = self.hdl.signal_pad_size // 8 + 64     # clear of the TP communicator's slots
        i32 = dict(dtype=torch.int32, device=device)
        self.state = torch.zeros(4, **i32)
        self.err = torch.zeros(1, **i32)
        self.counts = torch.zeros(n_experts, **i32)
        self.send_off = torch.zeros(n_experts, **i32)
        self.tile_expert = torch.full((self.max_tiles,), -1, **i32)
        self.meta = torch.zeros(4, **i32)
        n = max_local_tokens * top_k
        self.topk_ids = torch.zeros(n, **i32)
        self.slot = torch.zeros(n, **i32)
        self.where = torch.zeros(n, **i32)
        self.topk_w = torch.zeros(n, dtype=torch.float32, device=device)
        self.recv_x = self.buf[self.recvx_off:self.recvx_off + self.cap * hidden * 2].view(torch.bfloat16).view(self.cap, hidden)
        self.recv_y = self.buf[self.recvy_off:self.recvy_off + self.cap * hidden * 2].view(torch.bfloat16).view(self.cap, hidden)
        self.h = None
        self.a = None
        self.hdl.barrier()

    def _common(self):
        return (self.peer_ptrs, self.signal_ptrs, self.cnt_off, self.recvx_off, self.recvy_off, self.sig_off,
                ptr(self.state), ptr(self.err), self.rank, self.world, self.E, self.H, self.cap)

    def barrier(self):
        check(_lib.load().xllm_ep_barrier(*self._common(), stream()), "ep_barrier")

    def moe(self, x, logits, w_gate_up, w_down, scoring="softmax", bias=None, n_group=1, topk_group=1, renorm=True,
            scale=1.0, shared_out=None, out=None, load=None):
        """x [T, H] = this rank's tokens, logits [T, E]; w_gate_up [E_local, 2I, H] and w_down
        [E_local, H, I] = this rank's experts.  Returns the MoE output of this rank's tokens."""
        from ..ops import _count
        lib = _lib.load()
        T = x.shape[0]
        assert T <= self.max_local_tokens and x.shape[1] == self.H
        I2 = w_gate_up.shape[1]
        inter = I2 // 2
        if self.h is None or self.h.shape[1] != I2:
            self.h = torch.zeros(self.cap, I2, dtype=x.dtype, device=x.device)
            self.a = torch.zeros(self.cap, inter, dtype=x.dtype, device=x.device)
        s = stream()
        c = self._common()
        lf = logits.dtype == torch.float32
        if not lf and logits.dtype != torch.bfloat16:
            logits, lf = logits.float(), True
        # routing over ALL experts: counts per global expert and the slot of every (token, k) pair
        check(lib.xllm_moe_route(ptr(logits), int(lf), ptr(bias), ptr(self.topk_ids), ptr(self.topk_w), ptr(self.counts),
                                 ptr(self.slot), T, self.E, self.K, n_group, topk_group, 0 if scoring == "softmax" else 1,
                                 int(renorm), float(scale), 0, self.E, s), "moe_route")
        if load is not None:                      # expert load statistics: this rank's tokens per (physical) expert
            load += self.counts
        # counts to every peer + layout of the receive buffers (exchange 1)
        check(lib.xllm_ep_counts_layout(*c, ptr(self.counts), ptr(self.send_off), ptr(self.tile_expert), ptr(self.meta),
                                        self.max_tiles, s), "ep_counts_layout")
        # rows to their experts' owners; the kernel ends when every rank's rows have landed (exchange 2)
        check(lib.xllm_ep_dispatch_sync(*c, ptr(x), ptr(self.topk_ids), ptr(self.slot), ptr(self.send_off),
                                        ptr(self.where), T, self.K, s), "ep_dispatch")
        check(lib.xllm_gemm_bf16_grouped(ptr(self.recv_x), ptr(w_gate_up), ptr(self.h), ptr(self.tile_expert), self.cap,
                                         I2, self.H, self.e_local, self.H, I2, s), "ep_gemm1")
        # the activation only touches the rows that arrived (meta[0], known on the device)
        check(lib.xllm_act_and_mul_rows(ptr(self.a), ptr(self.h), self.cap, ptr(self.meta), inter, I2, 0, s), "ep_act")
        check(lib.xllm_gemm_bf16_grouped(ptr(self.a), ptr(w_down), ptr(self.recv_y), ptr(self.tile_expert), self.cap,
                                         self.H, inter, self.e_local, inter, self.H, s), "ep_gemm2")
        if out is None:
            out = torch.empty_like(x)
        # waits for every rank's expert outputs (exchange 3), then gathers and weights this rank's rows.
        # No closing barrier: nobody can overwrite a buffer before the next layer's exchanges, which
        # every rank only enters after this combine.
        check(lib.xllm_ep_combine_sync(*c, ptr(out), ptr(self.where), ptr(self.topk_w), ptr(shared_out), T, self.K, s),
              "ep_combine")
        _count(7)
        return out

    def error_status(self) -> int:
        v = int(self.err.item())
        if v:
            self.err.zero_()
        return v
