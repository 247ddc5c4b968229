"""Symmetric-memory communicator for the fused tensor-parallel kernels.

One symmetric arena per TP group (allocated and exchanged through
``torch.distributed._symmetric_memory``: cuMem VMM allocations mapped into every peer, an NVSwitch
multicast mapping when the fabric offers one, and a signal pad per rank).  The arena holds, at the
same offsets on every rank,

* ``x``   [max_tokens, hidden] — where a row-parallel GEMM writes its partial result,
* ``x1``  [oneshot_tokens, hidden] — the second partial buffer of the one-shot form (consecutive
  one-shot reductions alternate between ``x`` and ``x1``, which is what lets them drop the closing
  barrier),
* ``out`` [max_tokens, hidden] — where the reduced (+ residual + RMSNorm) rows of all ranks land in
  the two-shot form,
* a pair area for the vocabulary-sharded arg-max and, on demand, a gather area for full logits rows.

A forward pass brackets its reductions with ``begin_forward(T)`` / ``end_forward()``.  Steps of up to
``oneshot_tokens`` tokens use the one-shot kernel (`xllm_tp_oneshot_norm`: every rank reduces all rows
with ``multimem.ld_reduce``, the residual stream is replicated, one flag exchange per call); longer
steps use the sequence-sharded two-shot kernel or the GEMM's push epilogue.

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
_lib.register_signature("xllm_tp_oneshot_norm", [P, P, _lib.U64, L, L, P, P, P, P, P, P, I, I, I, I, F, I, P])
_lib.register_signature("xllm_tp_argmax", [P, L, P, P, L, L, P, P, P, I, I, I, I, I, I, P])
_lib.register_signature("xllm_tp_gather_cols", [P, L, P, P, _lib.U64, L, L, L, P, P, I, I, I, I, P])
_lib.register_signature("xllm_comm_set_wait_budget", [ctypes.c_longlong], ctypes.c_longlong)

MAX_SAMPLE_ROWS = 1024     # rows of the arg-max pair area


class TpComm:
    def __init__(self, ps, max_tokens: int, hidden: int, use_multimem: Optional[bool] = None,
                 vocab_shard: int = 0, max_sample_rows: int = 0):
        import torch.distributed._symmetric_memory as symm_mem

        self.ps = ps
        self.world = ps.tp_size
        self.rank = ps.tp_rank
        self.hidden = hidden
        self.max_tokens = (max_tokens + self.world - 1) // self.world * self.world
        self.device = ps.device
        row_bytes = hidden * 2
        al = lambda n: (n + 255) & ~255
        # One-shot or two-shot?  One-shot has one flag exchange (~10 us) but every rank pulls the whole
        # message through the switch, so each GPU serves `world` readers; two-shot has two exchanges and
        # moves (1 + 1/world) messages per GPU.  They cost the same at about
        # 10 us x 600 GB/s / (world - 1 - 1/world) bytes: 12 MB at 2 ranks, 2.2 MB at 4, 0.9 MB at 8.
        even = 6e6 / max(self.world - 1.0 - 1.0 / self.world, 0.25)
        auto = max(16, int(even / row_bytes))
        self.oneshot_tokens = min(self.max_tokens, int(os.environ.get("XLLM_TP_ONESHOT_TOKENS", str(auto))))
        self.x_off = 0
        self.x1_off = al(self.max_tokens * row_bytes)
        self.out_off = al(self.x1_off + self.oneshot_tokens * row_bytes)
        self.pair_off = al(self.out_off + self.max_tokens * row_bytes)
        self.gather_off = al(self.pair_off + 2 * self.world * MAX_SAMPLE_ROWS * 8)
        # full logits rows for sampling that needs the whole distribution (optional)
        self.vocab_shard = (int(vocab_shard) + 7) // 8 * 8
        self.gather_rows = int(max_sample_rows) if vocab_shard else 0
        self.gather_stride = self.vocab_shard * self.world
        total = self.gather_off + self.gather_rows * self.gather_stride * 2
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self.hdl = symm_mem.rendezvous(self.buf, ps.tp_group)
        self.peer_ptrs = self.hdl.buffer_ptrs_dev
        self.signal_ptrs = self.hdl.signal_pad_ptrs_dev
        mc = int(self.hdl.multicast_ptr or 0)
        if use_multimem is None:
            use_multimem = os.environ.get("XLLM_TP_MULTIMEM", "1") == "1"
        self.mc_base = mc if use_multimem else 0
        if not self.mc_base:
            # without in-switch reduction a one-shot call reads `world` copies of the message
            self.oneshot_tokens = min(self.oneshot_tokens, int(os.environ.get("XLLM_TP_ONESHOT_TOKENS_P2P", "64")))
        # flag slots live in the upper half of the signal pad (the lower half is left to torch's own
        # barrier helpers); every kernel family has its own 32-slot group and its own epoch words
        self.sig_off = self.hdl.signal_pad_size // 8
        self.counter_idx = self.sig_off + 32   # arrival counter of the push-mode GEMM (flags use [0, world))
        self.sig_oneshot = self.sig_off + 64
        self.sig_argmax = self.sig_off + 96
        self.sig_gather = self.sig_off + 128
        self._pushed = None                     # (T, expected arrivals) of a push-mode GEMM awaiting its reduction
        self.push_min_tokens = int(os.environ.get("XLLM_TP_PUSH_MIN_TOKENS", "512"))
        self.state = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.state_oneshot = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.state_argmax = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.state_gather = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        bf = lambda off, rows: self.buf[off: off + rows * row_bytes].view(torch.bfloat16).view(rows, hidden)
        self.x = bf(self.x_off, self.max_tokens)
        self.x1 = bf(self.x1_off, self.oneshot_tokens)
        self.out = bf(self.out_off, self.max_tokens)
        self.gathered = None
        if self.gather_rows:
            self.gathered = self.buf[self.gather_off:].view(torch.bfloat16).view(self.gather_rows, self.gather_stride)
        # one-shot bookkeeping: which partial buffer the next row-parallel GEMM writes
        self.oneshot = False
        self._parity = 0
        self._calls = 0
        self._scratch = torch.empty((1, hidden), dtype=torch.bfloat16, device=self.device)
        self.hdl.barrier()

    # ---- forward bracket
    def begin_forward(self, T: int) -> bool:
        """Choose the reduction form for a step of T tokens; returns True for the one-shot form (the
        residual stream is then replicated: [T, H] on every rank)."""
        assert self._pushed is None
        self.oneshot = 0 < T <= self.oneshot_tokens
        self._parity = 0
        self._calls = 0
        return self.oneshot

    def end_forward(self):
        """Close a forward: one-shot calls must come in pairs so that the next forward may start on
        buffer 0 again; an odd count is completed with a one-row call on the other buffer."""
        if self.oneshot and (self._calls & 1):
            self._oneshot(1, None, None, None, 0.0, out=self._scratch)
        self.oneshot = False

    # rows of the token dimension owned by this rank for a step of T tokens
    def shard(self, T: int):
        S = (T + self.world - 1) // self.world
        b = min(self.rank * S, T)
        return b, min(b + S, T), S

    def partial_buffer(self, T: int) -> torch.Tensor:
        """Where the next row-parallel GEMM (or any producer of a partial sum) writes its [T, H]."""
        assert T <= self.max_tokens
        if self.oneshot:
            return (self.x1 if self._parity else self.x)[:T]
        return self.x[:T]

    def _mc(self, T):
        """Multicast address for a reduction of T rows, or 0 for plain peer loads.  With two ranks a
        peer load fetches one remote copy, which measures faster than `multimem.ld_reduce` from 128
        rows on (41 us against 59 us at 2048 x 4096); with more ranks the in-switch reduction wins
        because a rank would otherwise fetch world - 1 copies."""
        return 0 if (self.world == 2 and T >= 128) else self.mc_base

    def _oneshot(self, T, residual_in, residual_out, weight, eps, out=None):
        if out is None:
            out = torch.empty((T, self.hidden), dtype=torch.bfloat16, device=self.device)
        x_off = self.x1_off if self._parity else self.x_off
        check(_lib.load().xllm_tp_oneshot_norm(self.peer_ptrs, self.signal_ptrs, self._mc(T), x_off, self.sig_oneshot,
                                               ptr(self.state_oneshot), ptr(residual_in), ptr(residual_out),
                                               ptr(weight), ptr(out), ptr(self.err), T, self.hidden, self.rank,
                                               self.world, float(eps), 296, stream()), "tp_oneshot_norm")
        from ..ops import _count
        _count()
        self._parity ^= 1
        self._calls += 1
        return out

    def _launch(self, T, residual, weight, eps, mode):
        if self.oneshot:
            return self._oneshot(T, residual, residual, weight, eps)
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
        check(_lib.load().xllm_tp_allreduce_norm(self.peer_ptrs, self.signal_ptrs, self._mc(T), self.x_off,
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
        return (not self.oneshot and bias is None and x.dim() == 2 and x.shape[0] >= self.push_min_tokens and x.dtype == torch.bfloat16
                and weight.dtype == torch.bfloat16 and x.stride(1) == 1 and weight.stride(1) == 1
                and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
                and not torch.cuda.is_current_stream_capturing())

    def allreduce_norm(self, T: int, residual_shard: torch.Tensor, weight: torch.Tensor, eps: float):
        """x[:T] (partials of all ranks) -> out[:T] = rmsnorm(sum + residual) * w on every rank;
        `residual_shard` is updated in place: this rank's rows ([ceil(T/world), H]) in the two-shot form,
        the whole replicated [T, H] stream in the one-shot form."""
        return self._launch(T, residual_shard, weight, eps, 1)

    def new_residual(self, x: torch.Tensor) -> torch.Tensor:
        """The residual stream that starts as `x` ([T, H], complete on every rank): the tensor itself in
        the one-shot form, this rank's rows (zero padded to the shard size) in the two-shot form."""
        if self.oneshot:
            return x
        b, e, S = self.shard(x.shape[0])
        r = torch.zeros((S, x.shape[1]), dtype=x.dtype, device=x.device)
        r[: e - b].copy_(x[b:e])
        return r

    # ---- sampling over vocabulary shards
    def argmax(self, local_logits: torch.Tensor, valid_cols: int, vocab_start: int, out: Optional[torch.Tensor] = None):
        """Greedy token ids of every row from the local logits shards of all ranks (identical on every
        rank); 8 bytes per row and peer cross the link instead of the logits."""
        B = local_logits.shape[0]
        assert B <= MAX_SAMPLE_ROWS and local_logits.dtype == torch.bfloat16 and local_logits.stride(1) == 1
        if out is None:
            out = torch.empty(B, dtype=torch.int64, device=self.device)
        check(_lib.load().xllm_tp_argmax(ptr(local_logits), local_logits.stride(0), self.peer_ptrs, self.signal_ptrs,
                                         self.pair_off, self.sig_argmax, ptr(self.state_argmax), ptr(out),
                                         ptr(self.err), B, int(valid_cols), int(vocab_start), MAX_SAMPLE_ROWS,
                                         self.rank, self.world, stream()), "tp_argmax")
        from ..ops import _count
        _count()
        return out

    def gather_logits(self, local_logits: torch.Tensor) -> Optional[torch.Tensor]:
        """All-gather the vocabulary shards into full rows [B, world * shard] inside the symmetric
        buffer (peer stores / `multimem.st` from one kernel); None when no gather area was reserved or
        the shapes do not fit it."""
        B, Vs = local_logits.shape
        if (self.gathered is None or B > self.gather_rows or Vs != self.vocab_shard
                or local_logits.dtype != torch.bfloat16 or local_logits.stride(1) != 1
                or local_logits.stride(0) % 8 or (local_logits.data_ptr() & 15)):
            return None
        check(_lib.load().xllm_tp_gather_cols(ptr(local_logits), local_logits.stride(0), self.peer_ptrs,
                                              self.signal_ptrs, self.mc_base, self.gather_off, self.gather_stride,
                                              self.sig_gather, ptr(self.state_gather), ptr(self.err), B, Vs, self.rank,
                                              self.world, stream()), "tp_gather_cols")
        from ..ops import _count
        _count()
        return self.gathered[:B]

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
