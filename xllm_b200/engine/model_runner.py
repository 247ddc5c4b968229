"""Worker-side execution of scheduled batches: staging, forward, sampling, CUDA graphs.

Capability parity with the reference's WorkerImpl / LLMWorkerImpl::step_internal
(xllm/core/runtime/worker_impl.cpp:1532-1627, llm_worker_impl.cpp:269-457) and its
CudaGraphExecutorImpl (cuda_graph_executor_impl.cpp:106-127 buckets, 902-1073 capture,
1075-1158 replay):

* every per-step input is packed by the C++ batch builder into one pinned buffer and reaches the
  device with a single H2D copy; staging buffers alternate so that a step can be prepared while the
  previous one is still running (schedule overlap);
* decode-only batches replay a CUDA graph per padded batch-size bucket, and steps that carry
  prompt chunks replay a graph per (decode bucket, prompt-token bucket): the whole step - embedding,
  layers, the fused tensor-parallel reductions, lm_head and the sampler - is one graph launch.  The
  graph reads its inputs from a persistent device buffer with the same packed layout, so refreshing
  the graph inputs is one device-to-device copy; padding rows are inert (kv_len 0, slot -1) and
  padding sequences have no query rows;
* sampling runs on the device inside the graph (arg-max or the full sampler with per-row random
  streams; over vocabulary shards with tensor parallelism) and the sampled ids stay on the device,
  so the next step can consume them as placeholders without a host round trip.  Batches that need
  the host between logits and sampling (penalties, grammar masks, top_logprobs) use a graph that
  stops at the logits.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import os

import numpy as np
import torch

from .. import ops
from ..models.layers import AttentionMetadata


def default_buckets(max_batch: int) -> List[int]:
    """1, 2, 4, 8, then multiples of 8 up to 64, then multiples of 16 (the reference pads to
    1, 2, 4, 8, 16·k: cuda_graph_executor_impl.cpp:106-127)."""
    out = [b for b in (1, 2, 4, 8) if b <= max_batch]
    b = 16
    while b <= max_batch:
        out.append(b)
        b += 8 if b < 64 else 16
    if out and out[-1] < max_batch:
        out.append(max_batch)
    return out or [max_batch]


@dataclass
class StepOutput:
    batch_id: int
    n_samples: int
    ids: torch.Tensor                     # device int64 [>= n_samples]
    logprobs: Optional[torch.Tensor]      # device fp32 or None
    ids_host: Optional[torch.Tensor]      # pinned, valid after `event`
    logprobs_host: Optional[torch.Tensor]
    event: Optional[torch.cuda.Event]
    top: Optional[tuple] = None           # (ids int32 [n, k], logprobs fp32 [n, k]) device tensors

    def wait(self):
        if self.event is not None:
            self.event.synchronize()
        ids = self.ids_host[:self.n_samples].numpy()
        lp = self.logprobs_host[:self.n_samples].numpy() if self.logprobs_host is not None else None
        return ids, lp

    def top_host(self):
        """(ids, logprobs) numpy arrays [n_samples, k] of the alternatives, or None."""
        if self.top is None:
            return None
        return self.top[0].cpu().numpy(), self.top[1].cpu().numpy()


class _Staging:
    def __init__(self, nbytes, device, pinned):
        self.host = torch.empty(nbytes, dtype=torch.uint8, pin_memory=pinned)
        self.dev = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.ids_host = None
        self.lp_host = None


def _view(buf, off, n, dtype):
    esz = torch.empty((), dtype=dtype).element_size()
    return buf[off:off + n * esz].view(dtype)


class ModelRunner:
    def __init__(self, model, block_size: int, num_blocks: int, max_seqs: int, max_tokens: int,
                 max_model_len: int, device, dtype, enable_graph: bool = True,
                 graph_buckets: Optional[List[int]] = None, n_staging: int = 2,
                 prefill_graph_tokens: Optional[List[int]] = None, prefill_graph_seqs: int = 4,
                 kv_allocator=None):
        from .. import _rt
        self._rt = _rt
        self.model = model
        self.args = model.args
        self.device = torch.device(device)
        self.dtype = dtype
        self.block_size = block_size
        self.num_blocks = num_blocks
        self.max_seqs = max_seqs
        self.max_tokens = max(max_tokens, max_seqs)
        self.max_model_len = max_model_len
        self.cuda = self.device.type == "cuda"
        self.enable_graph = enable_graph and self.cuda
        self.bt_cols = (max_model_len + block_size - 1) // block_size
        self.kv_allocator = kv_allocator     # (n_bytes) -> uint8 tensor, e.g. a slice of peer-mapped memory
        self.kv_caches = self._alloc_kv()
        # a padded mixed step has up to `prefill_graph_seqs` prompt-chunk sequences besides a full decode bucket
        extra = max(1, int(prefill_graph_seqs))
        cap = self._capacity(self.max_tokens + extra, self.max_seqs + extra, self.max_seqs + extra, self.bt_cols)
        self.staging = [_Staging(cap, self.device, self.cuda) for _ in range(n_staging)]
        for s in self.staging:
            s.ids_host = torch.empty(self.max_seqs, dtype=torch.int64, pin_memory=self.cuda)
            s.lp_host = torch.empty(self.max_seqs, dtype=torch.float32, pin_memory=self.cuda)
        self._turn = 0
        self.prev_ids: Optional[torch.Tensor] = None  # sampled ids of the previous step (device)
        self.overlap = False  # set by the engine: inputs may hold placeholders for prev_ids
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.graph_replays = 0
        self.graph_launches = 0      # kernel launches re-issued by graph replays
        self.logits_hook = None
        self.mm_hook = None          # multimodal requests: (batch) -> None | (embeds, rope_table, rope_rows)
        self.meta_hook = None        # (batch, meta) -> None: per-sequence state slots of linear-attention models
        self.keep_hidden = False     # speculative decoding with a draft layer needs the step's hidden states
        self.last_hidden = self.last_meta = self.last_positions = None
        self.graph_launches_per_replay: Dict[tuple, int] = {}
        # CUDA graphs: key = (decode rows, prompt-chunk sequences, prompt-chunk token rows, sample mode)
        self.buckets = graph_buckets or default_buckets(max_seqs)
        if prefill_graph_tokens is None:
            prefill_graph_tokens = [t for t in (128, 256, 512, 1024, 2048) if t <= self.max_tokens]
        self.prefill_buckets = sorted(prefill_graph_tokens) if self.enable_graph else []
        self.prefill_graph_seqs = max(1, int(prefill_graph_seqs))
        self.graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self.graph_in: Dict[tuple, torch.Tensor] = {}
        self.graph_out: Dict[tuple, tuple] = {}
        self.graph_off: Dict[tuple, list] = {}
        self.graph_pool = None
        nkv = self.model.num_kv_heads_local
        nq = self.args.num_attention_heads // self.model.ps.tp_size
        self._nq, self._nkv = nq, nkv
        self._ws: Dict[int, Optional[torch.Tensor]] = {}

    # ------------------------------------------------------------------ memory
    def _alloc_kv(self):
        m = self.model
        L = self.args.num_hidden_layers
        planes = int(getattr(m, "kv_planes", 2))
        shape = (L, planes, self.num_blocks, m.num_kv_heads_local, self.block_size, m.head_dim)
        if self.kv_allocator is not None:
            n = 1
            for d in shape:
                n *= d
            raw = self.kv_allocator(n * torch.empty((), dtype=self.dtype).element_size())
            kv = raw.view(self.dtype).view(shape)
            kv.zero_()
        else:
            kv = torch.zeros(shape, dtype=self.dtype, device=self.device)
        self.kv_tensor = kv
        return [(kv[i, 0], kv[i, planes - 1]) for i in range(L)]

    @staticmethod
    def kv_bytes_per_block(args, nkv_local, block_size, dtype, head_dim=None, planes=2):
        esz = torch.empty((), dtype=dtype).element_size()
        return args.num_hidden_layers * planes * nkv_local * block_size * (head_dim or args.head_dim) * esz

    @staticmethod
    def _capacity(T, S, NS, bt):
        al = lambda x: (x + 15) & ~15
        return (al(T * 8) * 2 + al(NS * 8) * 2 + al(T * 4) + al(S * 4) + al((S + 1) * 4) + al(S * 4)
                + al(NS * 4) * 4 + al(S * bt * 4) + 256)

    # ------------------------------------------------------------------ helpers
    def _decode_splits(self, B):
        return ops.decode_splits(B, self._nkv, self._nq // self._nkv)

    def _workspace(self, B, splits):
        key = (B, splits)
        if key not in self._ws:
            self._ws[key] = ops.decode_workspace(B, self._nq, self.model.head_dim, splits, self.device)
        return self._ws[key]

    def _meta_from(self, buf, off, n_decode, n_prefill, max_q_len, max_kv_len, bt_stride, padded=False):
        T, S = off[12], off[13]
        splits = self._decode_splits(n_decode) if n_decode > 0 and self.cuda else 1
        return AttentionMetadata(
            n_decode=n_decode, n_prefill=n_prefill,
            slots=_view(buf, off[3], T, torch.int32),
            block_table=_view(buf, off[10], S * bt_stride, torch.int32).view(S, bt_stride),
            kv_lens=_view(buf, off[4], S, torch.int32),
            cu_q=_view(buf, off[5], S + 1, torch.int32),
            max_q_len=max_q_len, max_kv_len=max_kv_len, decode_splits=splits,
            decode_workspace=self._workspace(n_decode, splits) if splits > 1 else None, padded=padded)

    def _bucket(self, n):
        for b in self.buckets:
            if b >= n:
                return b
        return None

    # ------------------------------------------------------------------ sampling
    def sample_mode(self, batch) -> str:
        """'greedy' / 'sample': the sampler runs right behind lm_head (inside the graph when there is
        one); 'logits': the step stops at the logits because the host takes part in sampling."""
        if batch.any_penalty or self.logits_hook is not None or batch.max_top_logprobs > 0:
            return "logits"
        if batch.all_greedy and not batch.any_logprobs:
            return "greedy"
        return "sample"

    def _device_sample(self, logits, src, off, NS, mode, want_lp=True):
        """Sampled ids (and log-probabilities) of NS rows from this rank's logits shard; the sampling
        parameters come from the packed buffer `src`.  Every rank returns the same ids."""
        m = self.model
        tp = m.ps.tp_size
        comm = m.ps.comm if logits.is_cuda else None
        head = m.lm_head
        if mode == "greedy":
            if tp == 1:
                return ops.sample(logits[:, :head.vocab] if logits.shape[1] != head.vocab else logits, None, None, None)
            if comm is not None and logits.dtype == torch.bfloat16 and NS <= 1024:
                valid = max(0, min(head.shard, head.vocab - head.start))
                return comm.argmax(logits, valid, head.start), None
            return m.greedy_from_local(logits), None
        if tp > 1:
            full = comm.gather_logits(logits) if comm is not None else None
            if full is None:
                full = m.gather_logits(logits)
            logits = full
        if logits.shape[1] != head.vocab:
            logits = logits[:, :head.vocab]
        return ops.sample(logits, _view(src, off[8], NS, torch.float32), _view(src, off[7], NS, torch.int32),
                          _view(src, off[9], NS, torch.float32), seeds=_view(src, off[15], NS, torch.int64),
                          offsets=_view(src, off[16], NS, torch.int32), want_logprob=want_lp)

    # ------------------------------------------------------------------ graph capture
    def graph_key(self, batch, mode, mm=None):
        """Which captured graph runs this batch, or None for the eager path."""
        if not self.enable_graph or mm is not None or batch.max_blocks > self.bt_cols or self.meta_hook is not None \
                or self.keep_hidden:
            return None
        nd, npf = batch.n_decode, batch.n_prefill
        if npf == 0:
            Bp = self._bucket(nd)
            return None if Bp is None else (Bp, 0, 0, mode)
        if npf > self.prefill_graph_seqs or not getattr(self.model, "supports_prefill_graph", True) \
                or os.environ.get("XLLM_PREFILL_GRAPH", "1") == "0":
            return None
        ptok = batch.n_tokens - nd
        Tq = next((t for t in self.prefill_buckets if t >= ptok), None)
        Bp = 0 if nd == 0 else self._bucket(nd)
        if Tq is None or Bp is None or Bp + Tq > self.max_tokens:
            return None
        return (Bp, self.prefill_graph_seqs, Tq, mode)

    def capture_graph(self, key):
        """Capture one whole step (forward + lm_head + sampler) for the padded shape `key`."""
        from ..ops import gemm_tcgen05
        if isinstance(key, int):
            key = (key, 0, 0, "greedy")
        Bp, P, Tq, mode = key
        gemm_tcgen05.prepare()   # per-device scratch must exist before a capture starts
        T, S = Bp + Tq, Bp + P
        NS = S
        off = list(self._rt.packed_layout(T, S, NS, self.bt_cols))
        gin = torch.zeros(off[11], dtype=torch.uint8, device=self.device)
        _view(gin, off[3], T, torch.int32).fill_(-1)   # slots: no KV write during warm-up
        cu = _view(gin, off[5], S + 1, torch.int32)
        cu[: Bp + 1].copy_(torch.arange(Bp + 1, dtype=torch.int32))
        cu[Bp + 1:].fill_(Bp)                           # prompt-chunk sequences without rows
        _view(gin, off[9], NS, torch.float32).fill_(1.0)
        meta = self._meta_from(gin, off, Bp, P, Tq if P else 1, 0, self.bt_cols, padded=P > 0)
        tokens = _view(gin, off[0], T, torch.int64)
        positions = _view(gin, off[1], T, torch.int64)
        rows = _view(gin, off[2], NS, torch.int64)

        def run():
            h = self.model.forward(tokens, positions, meta, self.kv_caches)
            if P > 0:
                h = ops.gather_rows(h, rows)
            logits = self.model.logits_local(h)   # this rank's vocabulary shard
            if mode == "logits":
                return logits, None, None
            ids, lp = self._device_sample(logits, gin, off, NS, mode)
            return logits, ids, lp

        from ..utils.platform import graph_capture
        with graph_capture():                  # no other thread of the process launches on the device meanwhile
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                for _ in range(2):
                    run()
            torch.cuda.current_stream().wait_stream(s)
            g = torch.cuda.CUDAGraph()
            before = ops.launches()
            with torch.cuda.graph(g, pool=self.graph_pool):
                out = run()
        self.graph_launches_per_replay[key] = ops.launches() - before
        if self.graph_pool is None:
            self.graph_pool = g.pool()
        self.graphs[key] = g
        self.graph_in[key] = gin
        self.graph_out[key] = out
        self.graph_off[key] = off
        return g

    def warmup(self, buckets: Optional[List[int]] = None, modes=("greedy",), prefill_tokens: Optional[List[int]] = None):
        """Capture graphs up front, largest first so that smaller ones reuse its pool (the reference
        warms up every bucket at start-up too: scheduler/profile/graph_warmup.cpp).  `buckets`:
        decode batch sizes; `prefill_tokens`: prompt-chunk token buckets to capture with each of them."""
        if not self.enable_graph:
            return
        for mode in modes:
            for b in sorted(buckets or self.buckets, reverse=True):
                if (b, 0, 0, mode) not in self.graphs:
                    self.capture_graph((b, 0, 0, mode))
                for tq in (prefill_tokens or []):
                    key = (b, self.prefill_graph_seqs, tq, mode)
                    if key not in self.graphs and b + tq <= self.max_tokens:
                        self.capture_graph(key)

    # ------------------------------------------------------------------ one step
    @torch.no_grad()
    def execute(self, batch, want_host=True) -> StepOutput:
        st = self.staging[self._turn % len(self.staging)]
        self._turn += 1
        nd, npf = batch.n_decode, batch.n_prefill
        mm = self.mm_hook(batch) if self.mm_hook is not None else None
        mode = self.sample_mode(batch)
        key = self.graph_key(batch, mode, mm)
        n_real = batch.n_samples
        if key is not None:
            Bp, P, Tq, _ = key
            off = batch.fill_packed(st.host.data_ptr(), st.host.numel(), self.bt_cols, Bp, Tq, P)
            bt_stride = self.bt_cols
        else:
            bt_stride = max(8, (batch.max_blocks + 7) // 8 * 8)
            off = batch.fill_packed(st.host.data_ptr(), st.host.numel(), bt_stride, 0)
        nbytes = off[11]
        if self.cuda:
            st.dev[:nbytes].copy_(st.host[:nbytes], non_blocking=True)
            self.h2d_bytes += nbytes
            buf = st.dev
        else:
            buf = st.host
        T, S, NS = off[12], off[13], off[14]

        ids = lp = None
        if key is not None:
            if key not in self.graphs:
                self.capture_graph(key)
            gin = self.graph_in[key]
            gin[:nbytes].copy_(buf[:nbytes])
            if self.overlap and self.prev_ids is not None:
                ops.resolve_placeholders(_view(gin, off[0], T, torch.int64), self.prev_ids)
            self.graphs[key].replay()
            self.graph_replays += 1
            self.graph_launches += self.graph_launches_per_replay[key]
            logits, ids, lp = self.graph_out[key]
            src = gin
        else:
            tokens = _view(buf, off[0], T, torch.int64)
            positions = _view(buf, off[1], T, torch.int64)
            if self.overlap and self.prev_ids is not None:
                ops.resolve_placeholders(tokens, self.prev_ids)
            meta = self._meta_from(buf, off, nd, npf, batch.max_q_len, batch.max_kv_len, bt_stride)
            if self.meta_hook is not None:
                self.meta_hook(batch, meta)
            if mm is not None:
                embeds, meta.rope_table, meta.rope_rows = mm
                hidden = self.model.forward(tokens, positions, meta, self.kv_caches, embeds=embeds)
            else:
                hidden = self.model.forward(tokens, positions, meta, self.kv_caches)
            if self.keep_hidden:
                self.last_hidden, self.last_meta, self.last_positions = hidden, meta, positions
            rows = _view(buf, off[2], NS, torch.int64)
            h = hidden if (NS == T and npf == 0) else ops.gather_rows(hidden, rows)
            logits = self.model.logits_local(h)
            src = buf
            if mode != "logits":
                ids, lp = self._device_sample(logits, src, off, NS, mode, want_lp=batch.any_logprobs)

        top = None
        if mode == "logits":
            # the host takes part: penalties over the sequences' token histories, grammar masks,
            # alternatives for top_logprobs; all of them need whole rows of the vocabulary
            if self.model.ps.tp_size > 1:
                logits = self.model.gather_logits(logits)
            if logits.shape[1] != self.model.lm_head.vocab:
                logits = logits[:, :self.model.lm_head.vocab]
            if batch.any_penalty:
                self._apply_penalties(batch, logits)
            if self.logits_hook is not None:
                self.logits_hook(batch, logits)   # e.g. grammar masks of constrained requests
            if batch.max_top_logprobs > 0 and n_real > 0:
                # alternatives under the temperature-scaled distribution the sample is drawn from
                # (the reference takes them from the processed logits too: sampler.cpp:155-169)
                t = _view(src, off[8], NS, torch.float32)[:n_real]
                scaled = logits[:n_real].float() / torch.where(t > 0, t, torch.ones_like(t)).unsqueeze(1)
                top = ops.top_logprobs(scaled, int(batch.max_top_logprobs))
            if batch.all_greedy and not batch.any_logprobs:
                ids, lp = ops.sample(logits, None, None, None)
            else:
                ids, lp = ops.sample(logits, _view(src, off[8], NS, torch.float32), _view(src, off[7], NS, torch.int32),
                                     _view(src, off[9], NS, torch.float32),
                                     seeds=_view(src, off[15], NS, torch.int64),
                                     offsets=_view(src, off[16], NS, torch.int32), want_logprob=batch.any_logprobs)
        if not batch.any_logprobs:
            lp = None
        self.prev_ids = ids
        out = StepOutput(batch.batch_id, n_real, ids, lp, None, None, None, top)
        if want_host:
            if self.cuda:
                st.ids_host[:n_real].copy_(ids[:n_real], non_blocking=True)
                self.d2h_bytes += n_real * 8
                if lp is not None:
                    st.lp_host[:n_real].copy_(lp[:n_real], non_blocking=True)
                    self.d2h_bytes += n_real * 4
                ev = torch.cuda.Event()
                ev.record()
                out.event = ev
                out.ids_host = st.ids_host
                out.logprobs_host = st.lp_host if lp is not None else None
            else:
                out.ids_host = ids
                out.logprobs_host = lp
        return out

    def _apply_penalties(self, batch, logits):
        pen = batch.penalty_tokens()
        if pen is None:
            return
        ids, counts = pen
        dev = logits.device
        n = ids.shape[0]
        # one staging tensor, one copy: [ids | counts] as int32 and the three penalty vectors as fp32
        host_i = torch.from_numpy(np.concatenate([ids.reshape(-1), counts.reshape(-1)]))
        host_f = torch.from_numpy(np.concatenate([batch.frequency_penalty, batch.presence_penalty,
                                                  batch.repetition_penalty]).astype(np.float32))
        if self.cuda:
            host_i, host_f = host_i.pin_memory(), host_f.pin_memory()
        di, df = host_i.to(dev, non_blocking=True), host_f.to(dev, non_blocking=True)
        w = ids.shape[1]
        ops.apply_penalties(logits[:n], di[: n * w].view(n, w), di[n * w:].view(n, w), df[:n], df[n:2 * n], df[2 * n:])
