"""Layer building blocks shared by the model zoo: TP linears, embedding, attention, MLP, norms.

Capability parity with the reference's layers/common (ColumnParallel / QKVParallel / RowParallel /
Replicated linears `linear.cpp:609-745, 1198-1285, 1647-1942`; `word_embedding_impl.cpp:48-56`;
`qwen2_attention.cpp:56-195` incl. KV-head replication when n_kv_heads < tp; `dense_mlp.cpp:124-170`;
`rms_norm.cpp`).  Modules are thin holders of inference-only tensors; every forward is a sequence of
ops from ``xllm_b200.ops`` (sm_100a kernels on CUDA, PyTorch references on CPU).
"""
from __future__ import annotations

import os

import math
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch

from .. import ops
from ..ops import reference
from ..parallel.state import ParallelState, single


# ----------------------------------------------------------------------------------- metadata
@dataclass
class AttentionMetadata:
    """Per-step attention inputs (device tensors).  Decode sequences occupy the first `n_decode`
    rows of every per-sequence tensor and the first `n_decode` token rows."""
    n_decode: int
    n_prefill: int
    slots: torch.Tensor          # [T] int32 cache slot of every new token (-1: skip)
    block_table: torch.Tensor    # [B, max_blocks] int32
    kv_lens: torch.Tensor        # [B] int32
    cu_q: torch.Tensor           # [B + 1] int32
    max_q_len: int = 1
    max_kv_len: int = 0
    decode_splits: int = 1
    decode_workspace: Optional[torch.Tensor] = None
    # multimodal rotary embedding: per-row cos|sin table [T, rot_dim] used instead of the model's
    # position-indexed cache (row i of the table belongs to token row i)
    rope_table: Optional[torch.Tensor] = None
    rope_rows: Optional[torch.Tensor] = None
    # the step has a fixed padded shape (CUDA-graph replay): token rows that belong to no sequence
    # exist, and whatever a kernel leaves unwritten for them must still be finite
    padded: bool = False
    # called with a layer's K cache right after the layer has written its new KV rows (prefill side
    # of a disaggregated pair: the layer's blocks are pushed to the decode instance while the next
    # layer computes)
    kv_hook: Optional[Callable] = None
    # fixed-step beam generation: every sequence row is a REQUEST whose cu_q rows are its beams; the
    # new tokens' KV goes to the beams' tail cache (`slots` index it) and attention runs over the shared
    # prompt pages plus each beam's tail (ops/xattn.py).  Object with tail_of(k_cache) -> (ku, vu), anc,
    # n_tail, max_rows.
    xattn: Optional[object] = None

    @property
    def n_seqs(self):
        return self.n_decode + self.n_prefill


# ----------------------------------------------------------------------------------- param registry
class Module:
    """Minimal parameter container: name -> (tensor, loader).  Loaders copy (a shard of) a
    checkpoint tensor into the parameter; fused parameters register one loader per source name."""

    def __init__(self):
        self._params: Dict[str, torch.Tensor] = {}
        self._loaders: Dict[str, Callable[[torch.Tensor], None]] = {}
        self._children: Dict[str, "Module"] = {}

    def copy_params_from(self, src: Dict[str, torch.Tensor]):
        """Copies another instance's parameters (name -> tensor, e.g. `dict(other.named_params())`) into this
        one, converting between the plain and the interleaved gate|up row layouts where the two differ (a CUDA
        bf16 model stores dense-MLP gate_up weights interleaved, a CPU model does not)."""
        from ..ops.gemm_tcgen05 import deinterleave_gate_up, interleave_gate_up
        for n, t in self.named_params():
            s = src[n]
            di, si = bool(getattr(t, "_xllm_interleaved", False)), bool(getattr(s, "_xllm_interleaved", False))
            if di and not si:
                s = interleave_gate_up(*s.chunk(2, dim=-2))
            elif si and not di:
                s = torch.cat(deinterleave_gate_up(s), dim=-2)
            t.copy_(s.to(t.dtype))

    def add_param(self, name, tensor, loaders: Optional[Dict[str, Callable]] = None):
        self._params[name] = tensor
        if loaders is None:
            loaders = {name: lambda w, t=tensor: t.copy_(w.to(t.dtype))}
        self._loaders.update(loaders)
        return tensor

    def add_module(self, name, mod):
        self._children[name] = mod
        return mod

    def named_params(self, prefix=""):
        for n, t in self._params.items():
            yield prefix + n, t
        for cn, c in self._children.items():
            yield from c.named_params(prefix + cn + ".")

    def named_loaders(self, prefix=""):
        for n, f in self._loaders.items():
            yield prefix + n, f
        for cn, c in self._children.items():
            yield from c.named_loaders(prefix + cn + ".")

    def param_bytes(self):
        return sum(t.numel() * t.element_size() for _, t in self.named_params())

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]], strict=True):
        loaders = dict(self.named_loaders())
        seen = set()
        # a model whose checkpoints name or pack tensors differently (fused gate_up_proj, w1/w2/w3
        # experts) defines `remap_weight(name, tensor) -> [(name, tensor), ...]`
        remap = getattr(self, "remap_weight", None)
        for name0, w0 in weights:
            for name, w in (remap(name0, w0) if remap is not None else ((name0, w0),)):
                f = loaders.get(name)
                if f is None:
                    continue
                f(w)
                seen.add(name)
        missing = [n for n in loaders if n not in seen]
        if strict and missing:
            raise KeyError(f"weights missing from checkpoint: {missing[:8]} (+{max(0, len(missing) - 8)} more)")
        return missing

    @torch.no_grad()
    def init_random(self, std=0.02, seed=0):
        """Deterministic N(0, std) weights; norm weights are set to 1."""
        for i, (name, t) in enumerate(self.named_params()):
            if t.dtype == torch.float8_e4m3fn:
                # an e4m3 weight and its block scales: q ~ N(0, 96) (well inside +-448), scale = std / 96
                g = torch.Generator(device=t.device)
                g.manual_seed(seed * 1000003 + i)
                w = torch.empty(t.shape, dtype=torch.float32, device=t.device).normal_(0.0, 96.0, generator=g)
                t.copy_(w.clamp_(-448, 448).to(t.dtype))
                continue
            if name.endswith("weight_scale_inv") or name.endswith("_scale"):
                t.fill_(std / 96.0)
                continue
            if t.dtype in (torch.uint8, torch.int32, torch.int64):
                continue
            if name.endswith("norm.weight") or name.endswith("layernorm.weight") or ".norm." in name \
                    or name.endswith("_norm.weight"):
                t.fill_(1.0)
                continue
            g = torch.Generator(device=t.device)
            g.manual_seed(seed * 1000003 + i)
            t.normal_(0.0, std, generator=g)


def _shard(w, dim, rank, size):
    if size == 1:
        return w
    n = w.shape[dim] // size
    return w.narrow(dim, rank * n, n)


FP8 = torch.float8_e4m3fn


def _to_fp8_blocks(w):
    """A bf16 / fp32 weight quantised to e4m3 in 128 x 128 blocks: (q, scales)."""
    from ..ops import fp8 as fp8_ops
    return fp8_ops.quant_block128_ref(w.float())


def _fp8_linear(x, w_q, w_scale, bias=None, out=None):
    """x @ dequant(w_q, w_scale)^T: the block-scaled tcgen05 GEMM on CUDA (activations quantised per
    token in groups of 128), the dequantised product on CPU."""
    from ..ops import fp8 as fp8_ops
    if x.is_cuda:
        y = fp8_ops.linear_block_fp8(x, w_q, w_scale, out=out)
    else:
        w = fp8_ops.dequant_block128_ref(w_q, w_scale, torch.float32)
        y = (x.float() @ w.T).to(x.dtype)
        if out is not None:
            out.copy_(y)
            y = out
    if bias is not None:
        y = y + bias
    return y


class _Fp8Weight:
    """Storage and loaders of one block-scaled fp8 weight [rows, cols] (+ scales [rows / 128, cols / 128]).
    `parts`: list of (source name, row offset, rows, shard fn) for fused weights; a source tensor may
    arrive as e4m3 (then its `weight_scale_inv` follows or precedes it) or in a wider type (quantised
    here)."""

    def __init__(self, rows, cols, device):
        self.q = torch.zeros(rows, cols, dtype=FP8, device=device)
        self.scale = torch.ones((rows + 127) // 128, (cols + 127) // 128, dtype=torch.float32, device=device)

    def loaders(self, name, row0, rows, shard_w, shard_s):
        """-> {name.weight: fn, name.weight_scale_inv: fn} writing rows [row0, row0 + rows)."""
        q, scale = self.q, self.scale

        def lw(w):
            w = shard_w(w)
            if w.dtype == FP8:
                q[row0:row0 + rows].copy_(w)
            else:
                wq, ws = _to_fp8_blocks(w)
                q[row0:row0 + rows].copy_(wq)
                scale[row0 // 128: row0 // 128 + ws.shape[0]].copy_(ws)

        def ls(sc):
            sc = shard_s(sc.float())
            scale[row0 // 128: row0 // 128 + sc.shape[0]].copy_(sc)

        return {f"{name}weight": lw, f"{name}weight_scale_inv": ls}


class Linear(Module):
    """y = x W^T (+ b). `parallel`: None (replicated), 'column' (shard dim 0), 'row' (shard dim 1)."""

    def __init__(self, in_f, out_f, bias, dtype, device, ps: ParallelState = None, parallel=None,
                 reduce=True, gather_output=False, fuse_reduce=True, quant=None):
        super().__init__()
        self.ps = ps or single()
        self.fuse_reduce = fuse_reduce      # False: a plain all-reduce, for layers that norm the sum by itself
        tp, rank = self.ps.tp_size, self.ps.tp_rank
        self.parallel = parallel if tp > 1 else None
        self.reduce = reduce
        self.gather_output = gather_output
        out_l = out_f // tp if self.parallel == "column" else out_f
        in_l = in_f // tp if self.parallel == "row" else in_f
        dim = {"column": 0, "row": 1}.get(self.parallel)
        # quant == "fp8_block": the weight stays e4m3 with 128 x 128 block scales and the product runs on
        # the block-scaled GEMM (needs in_l % 128 == 0; shards must fall on block boundaries)
        self.fp8 = None
        if quant == "fp8_block" and in_l % 128 == 0 and (dim is None or (out_l % 128 == 0 and in_l % 128 == 0)):
            self.fp8 = _Fp8Weight(out_l, in_l, device)
            self.weight = self.fp8.q
            sh_w = (lambda w: _shard(w, dim, rank, tp)) if dim is not None else (lambda w: w)
            sh_s = (lambda sc: _shard(sc, dim, rank, tp)) if dim is not None else (lambda sc: sc)
            self._params["weight"] = self.fp8.q
            self._params["weight_scale_inv"] = self.fp8.scale
            self._loaders.update(self.fp8.loaders("", 0, out_l, sh_w, sh_s))
        else:
            self.weight = torch.empty(out_l, in_l, dtype=dtype, device=device)

            def load_w(w, t=self.weight):
                t.copy_((_shard(w, dim, rank, tp) if dim is not None else w).to(t.dtype))

            self.add_param("weight", self.weight, {"weight": load_w})
        self.bias = None
        if bias:
            self.bias = torch.zeros(out_l, dtype=dtype, device=device)

            def load_b(b, t=self.bias):
                t.copy_((_shard(b, 0, rank, tp) if self.parallel == "column" else b).to(t.dtype))

            self.add_param("bias", self.bias, {"bias": load_b})

    def forward(self, x):
        bias = self.bias
        if self.parallel == "row" and self.ps.tp_rank != 0:
            bias = None  # added once, by rank 0, before the reduction
        if self.parallel == "row" and self.reduce:
            comm = self.ps.comm if self.fuse_reduce else None
            if comm is not None and x.is_cuda:
                # the partial result goes to the symmetric buffer; the cross-rank sum is fused
                # into the add+RMSNorm that follows (TpComm.allreduce_norm)
                T = x.shape[0]
                if self.fp8 is not None:
                    return _fp8_linear(x, self.fp8.q, self.fp8.scale, bias, out=comm.partial_buffer(T))
                if comm.push_supported(x, self.weight, bias):
                    # prefill-size batches: the GEMM's epilogue pushes each tile to the rank that
                    # reduces those rows (GEMM -> reduce-scatter in one kernel, TpComm.push_gemm)
                    return comm.push_gemm(x, self.weight)
                return ops.linear(x, self.weight, bias, out=comm.partial_buffer(T))
        if self.fp8 is not None:
            y = _fp8_linear(x, self.fp8.q, self.fp8.scale, bias)
        else:
            y = ops.linear(x, self.weight, bias)
        if self.parallel == "row" and self.reduce:
            y = self.ps.all_reduce(y)
        elif self.parallel == "column" and self.gather_output:
            y = self.ps.all_gather(y, dim=-1)
        return y

    __call__ = forward


class MergedColumnLinear(Module):
    """Several column-parallel projections of the same input fused into one GEMM
    (gate_proj|up_proj, q|k|v).  `sizes` are full (unsharded) output sizes, `names` the checkpoint
    sub-module names; `replicas[i]` > 1 means that shard i is replicated across that many ranks
    (KV heads when n_kv_heads < tp)."""

    def __init__(self, in_f, sizes: List[int], names: List[str], bias, dtype, device,
                 ps: ParallelState = None, shard_counts: Optional[List[int]] = None, quant=None, interleave: bool = False):
        super().__init__()
        self.ps = ps or single()
        self.interleaved = False
        tp, rank = self.ps.tp_size, self.ps.tp_rank
        counts = shard_counts or [tp] * len(sizes)
        self.local_sizes = [s // c for s, c in zip(sizes, counts)]
        total = sum(self.local_sizes)
        self.fp8 = None
        if quant == "fp8_block" and in_f % 128 == 0 and all(n % 128 == 0 for n in self.local_sizes) and not bias:
            self.fp8 = _Fp8Weight(total, in_f, device)
            self.weight = self.fp8.q
            self.bias = None
            off = 0
            for name, cnt, loc in zip(names, counts, self.local_sizes):
                idx = rank * cnt // tp
                self._loaders.update(self.fp8.loaders(f"{name}.", off, loc,
                                                      lambda w, i=idx, n=loc: w.narrow(0, i * n, n),
                                                      lambda sc, i=idx, n=loc: sc.narrow(0, i * n // 128, n // 128)))
                off += loc
            self._params["weight"] = self.fp8.q
            self._params["weight_scale_inv"] = self.fp8.scale
            return
        self.weight = torch.empty(total, in_f, dtype=dtype, device=device)
        self.bias = torch.zeros(total, dtype=dtype, device=device) if bias else None
        # gate|up of a gated MLP, rows interleaved in groups of 128 = [64 gate | the same 64 up]: the layout
        # whose GEMM applies the activation in its epilogue (ops/gemm_tcgen05.gemm_act_mul)
        self.interleaved = bool(interleave and len(sizes) == 2 and not bias and self.local_sizes[0] == self.local_sizes[1]
                                and self.local_sizes[0] % 64 == 0)
        self.weight._xllm_interleaved = self.interleaved
        loaders = {}
        off = 0
        for part, (name, full, cnt, loc) in enumerate(zip(names, sizes, counts, self.local_sizes)):
            idx = rank * cnt // tp  # which shard of this projection the rank holds

            def lw(w, o=off, n=loc, i=idx, t=self.weight, p=part):
                src = w.narrow(0, i * n, n).to(t.dtype)
                if self.interleaved:
                    t.view(n // 64, 2, 64, t.shape[1])[:, p].copy_(src.reshape(n // 64, 64, t.shape[1]))
                else:
                    t[o:o + n].copy_(src)

            loaders[f"{name}.weight"] = lw
            if bias:
                def lb(b, o=off, n=loc, i=idx, t=self.bias):
                    t[o:o + n].copy_(b.narrow(0, i * n, n).to(t.dtype))

                loaders[f"{name}.bias"] = lb
            off += loc
        self._params["weight"] = self.weight
        if bias:
            self._params["bias"] = self.bias
        self._loaders.update(loaders)

    def forward(self, x):
        if self.fp8 is not None:
            return _fp8_linear(x, self.fp8.q, self.fp8.scale)
        return ops.linear(x, self.weight, self.bias)

    __call__ = forward


class VocabEmbedding(Module):
    """Vocabulary-sharded embedding: each TP rank holds V/tp rows, out-of-shard ids give zeros and
    the partial results are summed (the reference shards the hidden dim and all-gathers,
    word_embedding_impl.cpp:48-56; summing a vocab-sharded lookup lets the lm_head share the
    same shard when embeddings are tied)."""

    def __init__(self, vocab, hidden, dtype, device, ps: ParallelState = None):
        super().__init__()
        self.ps = ps or single()
        tp, rank = self.ps.tp_size, self.ps.tp_rank
        self.vocab = vocab
        self.shard = (vocab + tp - 1) // tp
        self.start = rank * self.shard
        rows = max(0, min(self.shard, vocab - self.start))
        self.rows = rows
        self.weight = torch.zeros(self.shard, hidden, dtype=dtype, device=device)

        def lw(w, t=self.weight):
            t[:rows].copy_(w[self.start:self.start + rows].to(t.dtype))

        self.add_param("weight", self.weight, {"weight": lw})

    def forward(self, ids):
        comm = self.ps.comm
        if self.ps.tp_size > 1 and comm is not None and self.weight.is_cuda:
            T = ids.shape[0]
            ops.embedding(ids, self.weight, self.start, out=comm.partial_buffer(T))
            return comm.allreduce(T)
        y = ops.embedding(ids, self.weight, self.start)
        if self.ps.tp_size > 1:
            y = self.ps.all_reduce(y)
        return y

    __call__ = forward


class LMHead(Module):
    """Vocab-parallel output projection with all-gather of the logits shards."""

    def __init__(self, vocab, hidden, dtype, device, ps: ParallelState = None, tied: Optional[VocabEmbedding] = None):
        super().__init__()
        self.ps = ps or single()
        tp, rank = self.ps.tp_size, self.ps.tp_rank
        self.vocab = vocab
        self.shard = (vocab + tp - 1) // tp
        self.start = rank * self.shard
        rows = max(0, min(self.shard, vocab - self.start))
        if tied is not None:
            self.weight = tied.weight
        else:
            self.weight = torch.zeros(self.shard, hidden, dtype=dtype, device=device)

            def lw(w, t=self.weight):
                t[:rows].copy_(w[self.start:self.start + rows].to(t.dtype))

            self.add_param("weight", self.weight, {"weight": lw})

    def forward(self, x):
        return self.gather(self.forward_local(x))

    def forward_local(self, x):
        """This rank's shard of the logits: columns [start, start + shard) of the vocabulary."""
        return ops.linear(x, self.weight)

    def gather(self, y):
        if self.ps.tp_size > 1:
            y = self.ps.all_gather(y, dim=-1)
        return y[..., :self.vocab] if y.shape[-1] != self.vocab else y

    def greedy_from_local(self, y):
        """argmax over the whole vocabulary from the local shards: every rank reduces its own shard
        and only (value, index) pairs cross the link — 16 bytes per row instead of the vocabulary
        (the reference all-gathers the logits before sampling, lm_head + sampler.cpp)."""
        rows = max(0, min(self.shard, self.vocab - self.start))
        yl = y[..., :rows].float() if rows < y.shape[-1] else y.float()
        v, i = yl.max(dim=-1)
        if self.ps.tp_size == 1:
            return i
        pack = torch.stack([v, (i + self.start).to(torch.float64).to(torch.float32)], dim=-1)   # indices < 2^24 are exact
        if self.vocab >= (1 << 24):
            raise ValueError("vocabulary too large for the packed greedy reduction")
        allp = self.ps.all_gather(pack.contiguous(), dim=0).view(self.ps.tp_size, *pack.shape)
        best = allp[..., 0].argmax(dim=0)                     # ties go to the lowest rank = lowest index
        return allp[..., 1].gather(0, best[None])[0].to(torch.int64)

    __call__ = forward


class RMSNorm(Module):
    def __init__(self, hidden, eps, dtype, device, gemma=False):
        super().__init__()
        self.eps = eps
        self.gemma = gemma
        self.weight = self.add_param("weight", torch.ones(hidden, dtype=dtype, device=device))

    def forward(self, x, residual=None):
        return ops.rmsnorm(x, self.weight, self.eps, residual=residual, gemma=self.gemma)

    __call__ = forward


class RotaryEmbedding:
    """fp32 cos/sin cache [max_pos, rot_dim] built once per (rot_dim, theta, scaling)."""
    _cache: Dict[Tuple, torch.Tensor] = {}

    def __init__(self, rot_dim, max_pos, theta, scaling, device, interleaved=False):
        key = (rot_dim, max_pos, theta, str(scaling), str(device))
        if key not in RotaryEmbedding._cache:
            RotaryEmbedding._cache[key] = reference.build_cos_sin_cache(rot_dim, max_pos, theta, scaling, device)
        self.cos_sin = RotaryEmbedding._cache[key]
        self.rot_dim = rot_dim
        self.interleaved = interleaved


class Attention(Module):
    """GQA self-attention over the paged cache: fused QKV GEMM -> (qk-norm + RoPE + KV write) ->
    paged decode / prefill attention -> row-parallel o_proj."""

    def __init__(self, args, layer_idx, dtype, device, ps: ParallelState = None, rope: RotaryEmbedding = None,
                 fuse_reduce=True):
        super().__init__()
        self.ps = ps or single()
        tp = self.ps.tp_size
        self.d = args.head_dim
        self.nq = args.num_attention_heads // tp
        self.nkv_total = args.num_key_value_heads
        self.nkv = max(1, self.nkv_total // tp)
        kv_shards = min(tp, self.nkv_total)  # KV heads are replicated when there are fewer than tp
        H = args.hidden_size
        self.qkv = self.add_module("qkv_proj", MergedColumnLinear(
            H, [args.num_attention_heads * self.d, self.nkv_total * self.d, self.nkv_total * self.d],
            ["q_proj", "k_proj", "v_proj"], args.attention_bias, dtype, device, self.ps,
            shard_counts=[tp, kv_shards, kv_shards]))
        self.o_proj = self.add_module("o_proj", Linear(args.num_attention_heads * self.d, H, False, dtype, device,
                                                       self.ps, parallel="row", fuse_reduce=fuse_reduce))
        self.q_norm = self.k_norm = None
        if args.qk_norm:
            self.q_norm = self.add_module("q_norm", RMSNorm(self.d, args.rms_norm_eps, dtype, device))
            self.k_norm = self.add_module("k_norm", RMSNorm(self.d, args.rms_norm_eps, dtype, device))
        self.eps = args.rms_norm_eps
        self.rope = rope
        self.scale = 1.0 / math.sqrt(self.d)
        self.window = args.sliding_window

    # checkpoint names are self_attn.{q,k,v}_proj -> route them into the fused module
    def named_loaders(self, prefix=""):
        for n, f in super().named_loaders(prefix):
            yield n.replace("qkv_proj.", ""), f

    def forward(self, x, positions, meta: AttentionMetadata, k_cache, v_cache):
        return self._attend(self.qkv(x), positions, meta, k_cache, v_cache)

    def _attend(self, qkv, positions, meta: AttentionMetadata, k_cache, v_cache, gate=None):
        cos_sin = self.rope.cos_sin
        if meta.rope_table is not None:
            cos_sin, positions = meta.rope_table, meta.rope_rows
        if meta.xattn is not None:
            from ..ops import xattn as _xattn
            xa = meta.xattn
            ku, vu = xa.tail_of(k_cache)
            q = ops.rope_kv_write(qkv, self.nq, self.nkv, self.d, positions, cos_sin, self.rope.rot_dim,
                                  slots=meta.slots, k_cache=ku, v_cache=vu,
                                  q_norm_w=self._norm_w(self.q_norm), k_norm_w=self._norm_w(self.k_norm), eps=self.eps,
                                  interleaved=self.rope.interleaved)
            out = _xattn.xattention(q, k_cache, v_cache, meta.block_table, meta.cu_q, meta.kv_lens, xa.max_rows,
                                    ku, vu, xa.anc, xa.n_tail, self.scale)
            out = out.view(q.shape[0], self.nq * self.d)
            if gate is not None:
                out = out * torch.sigmoid(gate.float()).to(out.dtype)
            return self.o_proj(out)
        q = ops.rope_kv_write(qkv, self.nq, self.nkv, self.d, positions, cos_sin, self.rope.rot_dim,
                              slots=meta.slots, k_cache=k_cache, v_cache=v_cache,
                              q_norm_w=self._norm_w(self.q_norm), k_norm_w=self._norm_w(self.k_norm), eps=self.eps,
                              interleaved=self.rope.interleaved)
        if meta.kv_hook is not None:
            meta.kv_hook(k_cache)
        T = q.shape[0]
        out = (torch.zeros if meta.padded else torch.empty)((T, self.nq, self.d), dtype=q.dtype, device=q.device)
        nd = meta.n_decode
        if nd > 0:
            ops.paged_decode_attention(q[:nd], k_cache, v_cache, meta.block_table[:nd], meta.kv_lens[:nd],
                                       self.scale, splits=meta.decode_splits,
                                       workspace=meta.decode_workspace, out=out[:nd], window=self.window)
        if meta.n_prefill > 0:
            # cu_q holds absolute token rows, so the full q / out tensors are passed
            ops.paged_prefill_attention(q, k_cache, v_cache, meta.block_table[nd:], meta.cu_q[nd:],
                                        meta.kv_lens[nd:], meta.max_q_len, self.scale, causal=True,
                                        window=self.window, out=out)
        out = out.view(T, self.nq * self.d)
        if gate is not None:                               # per-element output gate (Qwen3-Next)
            out = out * torch.sigmoid(gate.float()).to(out.dtype)
        return self.o_proj(out)

    @staticmethod
    def _norm_w(norm):
        if norm is None:
            return None
        return norm.weight + 1.0 if norm.gemma else norm.weight       # zero-centred weights

    __call__ = forward


class DenseMLP(Module):
    """SwiGLU MLP: fused gate|up column-parallel GEMM -> silu·mul -> row-parallel down GEMM."""

    def __init__(self, hidden, inter, act, dtype, device, ps: ParallelState = None, reduce=True, fuse_reduce=True,
                 quant=None):
        super().__init__()
        self.ps = ps or single()
        self.act = act
        # on a CUDA device the gate and up rows are stored interleaved, so that prompt-size batches run the
        # GEMM whose epilogue applies the gated activation (XLLM_FUSED_ACT=0 keeps the plain layout)
        il = (torch.device(device).type == "cuda" and dtype == torch.bfloat16 and quant is None
              and act in ("silu", "gelu", "gelu_tanh", "gelu_pytorch_tanh") and os.environ.get("XLLM_FUSED_ACT", "1") != "0")
        self.gate_up = self.add_module("gate_up_proj", MergedColumnLinear(
            hidden, [inter, inter], ["gate_proj", "up_proj"], False, dtype, device, self.ps, quant=quant, interleave=il))
        self.down = self.add_module("down_proj", Linear(inter, hidden, False, dtype, device, self.ps,
                                                        parallel="row", reduce=reduce, fuse_reduce=fuse_reduce,
                                                        quant=quant))

    def named_loaders(self, prefix=""):
        for n, f in super().named_loaders(prefix):
            yield n.replace("gate_up_proj.", ""), f

    def hidden(self, x):
        """act(x W_gate^T) * (x W_up^T): the input of the down projection, whatever the row layout of gate|up."""
        gu = self.gate_up
        if gu.interleaved:
            from ..ops import gemm, gemm_tcgen05
            if (x.is_cuda and x.dim() == 2 and x.shape[0] > 512 and gemm.gemm_mode() != "cublas" and gu.weight.shape[0] % 256 == 0
                    and gemm_tcgen05.supported(x, gu.weight)):
                return gemm_tcgen05.gemm_act_mul(x, gu.weight, self.act)
            y = gu(x)
            return gemm_tcgen05.act_and_mul_interleaved(y.view(-1, y.shape[-1]), self.act).view(*y.shape[:-1], -1)
        return ops.act_and_mul(gu(x), self.act)

    def forward(self, x):
        return self.down(self.hidden(x))

    __call__ = forward
