"""Worker-side execution of scheduled batches: staging, forward, sampling, CUDA graphs.

Capability parity with the reference's WorkerImpl / LLMWorkerImpl::step_internal
(xllm/core/runtime/worker_impl.cpp:1532-1627, llm_worker_impl.cpp:269-457) and its
CudaGraphExecutorImpl (cuda_graph_executor_impl.cpp:106-127 buckets, 902-1073 capture,
1075-1158 replay):

* every per-step input is packed by the C++ batch builder into one pinned buffer and reaches the
  device with a single H2D copy; staging buffers alternate so that a step can be prepared while the
  previous one is still running (schedule overlap);
* decode-only batches replay a CUDA graph per padded batch-size bucket.  The graph reads its
  inputs from a persistent device buffer with the same packed layout, so refreshing the graph
  inputs is one device-to-device copy; padding rows are inert (kv_len 0, slot -1);
* sampling runs on the device right after the forward pass and the sampled ids stay on the
  device, so the next step can consume them as placeholders without a host round trip.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

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

    def wait(self):
        if self.event is not None:
            self.event.synchronize()
        ids = self.ids_host[:self.n_samples].numpy()
        lp = self.logprobs_host[:self.n_samples].numpy() if self.logprobs_host is not None else None
        return ids, lp


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
                 graph_buckets: Optional[List[int]] = None, n_staging: int = 2):
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
        self.kv_caches = self._alloc_kv()
        cap = self._capacity(self.max_tokens, self.max_seqs, self.max_seqs, self.bt_cols)
        self.staging = [_Staging(cap, self.device, self.cuda) for _ in range(n_staging)]
        for s in self.staging:
            s.ids_host = torch.empty(self.max_seqs, dtype=torch.int64, pin_memory=self.cuda)
            s.lp_host = torch.empty(self.max_seqs, dtype=torch.float32, pin_memory=self.cuda)
        self._turn = 0
        self.prev_ids: Optional[torch.Tensor] = None  # sampled ids of the previous step (device)
        self.overlap = False  # set by the engine: inputs may hold placeholders for prev_ids
        self.sample_offset = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.graph_replays = 0
        self.logits_hook = None
        self.mm_hook = None          # multimodal requests: (batch) -> None | (embeds, rope_table, rope_rows)
        self.meta_hook = None        # (batch, meta) -> None: per-sequence state slots of linear-attention models
        self.keep_hidden = False     # speculative decoding with a draft layer needs the step's hidden states
        self.last_hidden = self.last_meta = self.last_positions = None
        self.graph_launches_per_replay: Dict[int, int] = {}
        # CUDA graphs
        self.buckets = graph_buckets or default_buckets(max_seqs)
        self.graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.graph_in: Dict[int, torch.Tensor] = {}
        self.graph_logits: Dict[int, torch.Tensor] = {}
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
        return (al(T * 8) * 2 + al(NS * 8) + al(T * 4) + al(S * 4) + al((S + 1) * 4) + al(S * 4)
                + al(NS * 4) * 3 + al(S * bt * 4) + 256)

    # ------------------------------------------------------------------ helpers
    def _decode_splits(self, B):
        return ops.decode_splits(B, self._nkv, self._nq // self._nkv)

    def _workspace(self, B, splits):
        key = (B, splits)
        if key not in self._ws:
            self._ws[key] = ops.decode_workspace(B, self._nq, self.model.head_dim, splits, self.device)
        return self._ws[key]

    def _meta_from(self, buf, off, n_decode, n_prefill, max_q_len, max_kv_len, bt_stride):
        T, S = off[12], off[13]
        splits = self._decode_splits(n_decode) if n_decode > 0 and self.cuda else 1
        return AttentionMetadata(
            n_decode=n_decode, n_prefill=n_prefill,
            slots=_view(buf, off[3], T, torch.int32),
            block_table=_view(buf, off[10], S * bt_stride, torch.int32).view(S, bt_stride),
            kv_lens=_view(buf, off[4], S, torch.int32),
            cu_q=_view(buf, off[5], S + 1, torch.int32),
            max_q_len=max_q_len, max_kv_len=max_kv_len, decode_splits=splits,
            decode_workspace=self._workspace(n_decode, splits) if splits > 1 else None)

    def _bucket(self, n):
        for b in self.buckets:
            if b >= n:
                return b
        return None

    # ------------------------------------------------------------------ graph capture
    def _graph_offsets(self, Bp):
        al = lambda x: (x + 15) & ~15
        off = [0] * 15
        o = 0
        off[0] = o; o = al(o + Bp * 8)
        off[1] = o; o = al(o + Bp * 8)
        off[2] = o; o = al(o + Bp * 8)
        off[3] = o; o = al(o + Bp * 4)
        off[4] = o; o = al(o + Bp * 4)
        off[5] = o; o = al(o + (Bp + 1) * 4)
        off[6] = o; o = al(o + Bp * 4)
        off[7] = o; o = al(o + Bp * 4)
        off[8] = o; o = al(o + Bp * 4)
        off[9] = o; o = al(o + Bp * 4)
        off[10] = o; o = al(o + Bp * self.bt_cols * 4)
        off[11] = o; off[12] = Bp; off[13] = Bp; off[14] = Bp
        return off

    def capture_graph(self, Bp):
        """Capture forward + lm_head for a padded decode batch of Bp rows."""
        from ..ops import gemm_tcgen05
        gemm_tcgen05.prepare()   # per-device scratch must exist before a capture starts
        off = self._graph_offsets(Bp)
        gin = torch.zeros(off[11], dtype=torch.uint8, device=self.device)
        _view(gin, off[3], Bp, torch.int32).fill_(-1)   # slots: no KV write during warm-up
        meta = self._meta_from(gin, off, Bp, 0, 1, 0, self.bt_cols)
        tokens = _view(gin, off[0], Bp, torch.int64)
        positions = _view(gin, off[1], Bp, torch.int64)

        def run():
            h = self.model.forward(tokens, positions, meta, self.kv_caches)
            return self.model.logits_local(h)   # this rank's vocabulary shard; gathered (or not) after the graph

        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                run()
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        before = ops.launches()
        with torch.cuda.graph(g, pool=self.graph_pool):
            logits = run()
        self.graph_launches_per_replay[Bp] = ops.launches() - before
        if self.graph_pool is None:
            self.graph_pool = g.pool()
        self.graphs[Bp] = g
        self.graph_in[Bp] = gin
        self.graph_logits[Bp] = logits
        return g

    def warmup(self, buckets: Optional[List[int]] = None):
        """Capture the decode graphs up front, largest first so that smaller ones reuse its pool
        (the reference warms up every bucket at start-up too: scheduler/profile/graph_warmup.cpp)."""
        if not self.enable_graph:
            return
        for b in sorted(buckets or self.buckets, reverse=True):
            if b not in self.graphs:
                self.capture_graph(b)

    # ------------------------------------------------------------------ one step
    @torch.no_grad()
    def execute(self, batch, want_host=True) -> StepOutput:
        st = self.staging[self._turn % len(self.staging)]
        self._turn += 1
        nd, npf = batch.n_decode, batch.n_prefill
        mm = self.mm_hook(batch) if self.mm_hook is not None else None
        use_graph = self.enable_graph and npf == 0 and self._bucket(nd) is not None \
            and batch.max_blocks <= self.bt_cols and mm is None
        Bp = self._bucket(nd) if use_graph else 0
        bt_stride = self.bt_cols if use_graph else max(8, (batch.max_blocks + 7) // 8 * 8)
        off = batch.fill_packed(st.host.data_ptr(), st.host.numel(), bt_stride, Bp)
        nbytes = off[11]
        if self.cuda:
            st.dev[:nbytes].copy_(st.host[:nbytes], non_blocking=True)
            self.h2d_bytes += nbytes
            buf = st.dev
        else:
            buf = st.host
        T, S, NS = off[12], off[13], off[14]
        n_real = batch.n_samples

        if use_graph:
            if Bp not in self.graphs:
                self.capture_graph(Bp)
            gin = self.graph_in[Bp]
            gin[:nbytes].copy_(buf[:nbytes])
            if self.overlap and self.prev_ids is not None:
                ops.resolve_placeholders(_view(gin, off[0], Bp, torch.int64), self.prev_ids)
            self.graphs[Bp].replay()
            self.graph_replays += 1
            logits = self.graph_logits[Bp]
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

        temperature = _view(src, off[8], NS, torch.float32)
        top_k = _view(src, off[7], NS, torch.int32)
        top_p = _view(src, off[9], NS, torch.float32)
        want_lp = batch.any_logprobs
        sharded = self.model.ps.tp_size > 1
        greedy_sharded = (sharded and batch.all_greedy and not want_lp and not batch.any_penalty
                          and self.logits_hook is None)
        if sharded and not greedy_sharded:
            logits = self.model.gather_logits(logits)
        if batch.any_penalty:
            self._apply_penalties(batch, logits)
        if self.logits_hook is not None:
            self.logits_hook(batch, logits)   # e.g. grammar masks of constrained requests
        if greedy_sharded:
            # vocabulary-sharded argmax: only (value, index) pairs cross the link
            ids, lp = self.model.greedy_from_local(logits), None
        elif batch.all_greedy and not want_lp:
            ids, lp = ops.sample(logits, None, None, None)
        else:
            ids, lp = ops.sample(logits, temperature, top_k, top_p, seed=int(batch.seeds[0]) if n_real else 0,
                                 offset=self.sample_offset, want_logprob=want_lp)
            self.sample_offset += 4
        self.prev_ids = ids
        out = StepOutput(batch.batch_id, n_real, ids, lp, None, None, None)
        if want_host:
            if self.cuda:
                st.ids_host[:NS].copy_(ids[:NS], non_blocking=True)
                self.d2h_bytes += n_real * 8
                if lp is not None:
                    st.lp_host[:NS].copy_(lp[:NS], non_blocking=True)
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
        ids_t = torch.from_numpy(ids).to(dev)
        cnt_t = torch.from_numpy(counts).to(dev)
        n = ids.shape[0]
        f = torch.from_numpy(batch.frequency_penalty).to(dev)
        p = torch.from_numpy(batch.presence_penalty).to(dev)
        r = torch.from_numpy(batch.repetition_penalty).to(dev)
        ops.apply_penalties(logits[:n], ids_t, cnt_t, f, p, r)
