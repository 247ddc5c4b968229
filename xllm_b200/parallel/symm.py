"""Symmetric-memory communicator for the fused tensor-parallel kernels.

One symmetric arena per TP group (allocated and exchanged through
``torch.distributed._symmetric_memory``: cuMem VMM allocations mapped into every peer, an NVSwitch
multicast mapping when the fabric offers one, and a signal pad per rank).  The arena holds, at the
same offsets on every rank,

* ``x``   [max_tokens, hidden] — where a row-parallel GEMM writes its partial result,
* ``out`` [max_tokens, hidden] — where the reduced (+ residual + RMSNorm) rows of all ranks land.

``allreduce_norm`` launches `xllm_tp_allreduce_norm` (csrc/kernels/comm.cu) on the current stream:
an ordinary kernel, so it is captured by CUDA graphs and needs no side stream (the reference's
Python path made the same move for small messages, xllm/python/distributed/collectives.py:258-312;
its C++ path uses NCCL, layers/common/linear.cpp:1938-1940).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..ops import _lib
from ..ops._lib import I, L, P, check, ptr, stream

F = _lib.F
_lib.register_signature("xllm_tp_allreduce_norm", [P, P, _lib.U64, L, L, L, P, P, P, P, I, I, I, I, I, F, I, P])


class TpComm:
    def __init__(self, ps, max_tokens: int, hidden: int, use_multimem: Optional[bool] = None):
        import torch.distributed._symmetric_memory as symm_mem

        self.ps = ps
        self.world = ps.tp_size
        self.rank = ps.tp_rank
        self.hidden = hidden
        self.max_tokens = (max_tokens + self.world - 1) // self.world * self.world
        self.device = ps.device
        row_bytes = hidden * 2
        self.x_off = 0
        self.out_off = self.max_tokens * row_bytes
        total = 2 * self.max_tokens * row_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self.hdl = symm_mem.rendezvous(self.buf, ps.tp_group)
        self.peer_ptrs = self.hdl.buffer_ptrs_dev
        self.signal_ptrs = self.hdl.signal_pad_ptrs_dev
        mc = int(self.hdl.multicast_ptr or 0)
        if use_multimem is None:
            use_multimem = os.environ.get("XLLM_TP_MULTIMEM", "1") == "1"
        self.mc_base = mc if use_multimem else 0
        # flag slots live in the upper half of the signal pad (the lower half is left to torch's own
        # barrier helpers)
        self.sig_off = self.hdl.signal_pad_size // 8
        self.state = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.x = self.buf[: self.max_tokens * row_bytes].view(torch.bfloat16).view(self.max_tokens, hidden)
        self.out = self.buf[self.out_off:].view(torch.bfloat16).view(self.max_tokens, hidden)
        self.hdl.barrier()

    # rows of the token dimension owned by this rank for a step of T tokens
    def shard(self, T: int):
        S = (T + self.world - 1) // self.world
        b = min(self.rank * S, T)
        return b, min(b + S, T), S

    def partial_buffer(self, T: int) -> torch.Tensor:
        assert T <= self.max_tokens
        return self.x[:T]

    def _launch(self, T, residual, weight, eps, mode):
        S = (T + self.world - 1) // self.world
        n_ctas = max(1, min(S, 148))
        check(_lib.load().xllm_tp_allreduce_norm(self.peer_ptrs, self.signal_ptrs, self.mc_base, self.x_off,
                                                 self.out_off, self.sig_off, ptr(self.state), ptr(residual),
                                                 ptr(weight), ptr(self.err), T, self.hidden, self.rank,
                                                 self.world, mode, eps, n_ctas, stream()), "tp_allreduce_norm")
        from ..ops import _count
        _count()
        return self.out[:T]

    def allreduce_norm(self, T: int, residual_shard: torch.Tensor, weight: torch.Tensor, eps: float):
        """x[:T] (partials of all ranks) -> out[:T] = rmsnorm(sum + residual) * w on every rank;
        `residual_shard` ([ceil(T/world), H], this rank's rows) is updated in place."""
        return self._launch(T, residual_shard, weight, eps, 1)

    def allreduce(self, T: int):
        """x[:T] (partials of all ranks) -> out[:T] = sum, on every rank."""
        return self._launch(T, None, None, 0.0, 0)

    def error_status(self) -> int:
        v = int(self.err.item())
        if v:
            self.err.zero_()
        return v


def attach(ps, max_tokens: int, hidden: int, **kw) -> Optional[TpComm]:
    """Create the communicator for `ps` when it is a multi-rank CUDA TP group."""
    if ps is None or ps.tp_size <= 1 or ps.device.type != "cuda":
        return None
    if os.environ.get("XLLM_TP_COMM", "fused") != "fused":
        return None
    ps.comm = TpComm(ps, max_tokens, hidden, **kw)
    return ps.comm
