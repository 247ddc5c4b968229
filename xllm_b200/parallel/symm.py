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

import ctypes
import os
from typing import Optional

import torch

from ..ops import _lib
from ..ops._lib import I, L, P, check, ptr, stream

F = _lib.F
_lib.register_signature("xllm_tp_allreduce_norm", [P, P, _lib.U64, L, L, L, P, P, P, P, I, I, I, I, I, F, I, P])
_lib.register_signature("xllm_tp_inbox_norm", [P, P, _lib.U64, L, L, L, L, ctypes.c_uint32, P, P, P, P, I, I, I, I, I, F,
                                               I, P])
_lib.register_signature("xllm_gemm_bf16_push", [P, P, P, P, L, L, I, I, I, L, L, I, I, I, I, P])


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
        self.counter_idx = self.sig_off + 32   # arrival counter of the push-mode GEMM (flags use [0, world))
        self._pushed = None                     # (T, expected arrivals) of a push-mode GEMM awaiting its reduction
        self.push_min_tokens = int(os.environ.get("XLLM_TP_PUSH_MIN_TOKENS", "512"))
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
        # two 256-thread CTAs fit on an SM (127 registers per thread), and every CTA works on one row at
        # a time, so 296 co-resident CTAs double the rows in flight
        n_ctas = max(1, min(S, 296))
        if self._pushed is not None:
            pT, expected = self._pushed
            self._pushed = None
            assert pT == T, "the reduction must follow the pushed GEMM of the same token count"
            check(_lib.load().xllm_tp_inbox_norm(self.peer_ptrs, self.signal_ptrs, self.mc_base, self.x_off,
                                                 self.out_off, self.sig_off, self.counter_idx, expected,
                                                 ptr(self.state), ptr(residual), ptr(weight), ptr(self.err), T,
                                                 self.hidden, self.rank, self.world, mode, float(eps), n_ctas,
                                                 stream()), "tp_inbox_norm")
            from ..ops import _count
            _count()
            return self.out[:T]
        check(_lib.load().xllm_tp_allreduce_norm(self.peer_ptrs, self.signal_ptrs, self.mc_base, self.x_off,
                                                 self.out_off, self.sig_off, ptr(self.state), ptr(residual),
                                                 ptr(weight), ptr(self.err), T, self.hidden, self.rank,
                                                 self.world, mode, eps, n_ctas, stream()), "tp_allreduce_norm")
        from ..ops import _count
        _count()
        return self.out[:T]

    # ---- fused row-parallel GEMM -> reduce-scatter -> (+residual, RMSNorm) -> all-gather
    def gemm_rs_norm(self, x_local: torch.Tensor, weight: torch.Tensor, residual_shard, norm_weight, eps: float,
                     tile_n: int = 0):
        """out[:T] = rmsnorm(sum_ranks(x_local @ weight^T) + residual) * w on every rank.

        Two launches: the tcgen05 GEMM whose epilogue pushes each finished tile into the owner
        rank's inbox over NVLink while the next tile's MMAs run (`xllm_gemm_bf16_push`), and the
        owner-side kernel that waits for its arrival counter, reduces, normalises and broadcasts
        (`xllm_tp_inbox_norm`).  The reference does this as cuBLAS + NCCL all-reduce + a norm kernel
        (layers/common/linear.cpp:1938-1940); its sequence-parallel NPU path has the fused
        matmul+reduce-scatter shape (common/flash_comm1_context.*).  With `norm_weight=None` the
        result is the plain sum."""
        T = x_local.shape[0]
        self.push_gemm(x_local, weight, tile_n)
        if norm_weight is None:
            return self.allreduce(T)
        return self.allreduce_norm(T, residual_shard, norm_weight, eps)

    def push_gemm(self, x_local: torch.Tensor, weight: torch.Tensor, tile_n: int = 0):
        """Launch the row-parallel GEMM in push mode; the next `allreduce` / `allreduce_norm` call
        (same T) completes the operation from the inbox instead of running its opening barrier."""
        T, K = x_local.shape
        N = weight.shape[0]
        assert N == self.hidden and T <= self.max_tokens and self._pushed is None
        assert x_local.stride(1) == 1 and weight.stride(1) == 1
        S = (T + self.world - 1) // self.world
        if tile_n == 0:
            tile_n = 256 if T > 512 else 128
        n_tiles = (N + tile_n - 1) // tile_n
        b, e, _ = self.shard(T)
        check(_lib.load().xllm_gemm_bf16_push(ptr(x_local), ptr(weight), self.peer_ptrs, self.signal_ptrs, self.x_off,
                                              self.counter_idx, T, N, K, x_local.stride(0), weight.stride(0), S,
                                              self.rank, self.world, tile_n, stream()), "gemm_bf16_push")
        from ..ops import _count
        _count()
        self._pushed = (T, (e - b) * n_tiles * self.world)
        return self.x[:T]  # placeholder with the right shape; the data lives in the owners' inboxes

    def push_supported(self, x, weight, bias) -> bool:
        """Whether a row-parallel linear of this shape should take the push path."""
        return (bias is None and x.dim() == 2 and x.shape[0] >= self.push_min_tokens and x.dtype == torch.bfloat16
                and weight.dtype == torch.bfloat16 and x.stride(1) == 1 and weight.stride(1) == 1
                and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
                and not torch.cuda.is_current_stream_capturing())

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
