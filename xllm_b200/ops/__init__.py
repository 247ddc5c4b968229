"""Operator front end: every op runs the hand-written sm_100a kernel on CUDA tensors and the
PyTorch reference on CPU tensors (no third path).

Counterpart of the platform-dispatching `xllm::kernel::*` free functions of the reference
(xllm/core/kernels/ops_api.h:27-290) — minus the dispatch: there is one target.
"""
from __future__ import annotations

import os

import torch

from . import _lib, reference
from ._lib import check, ptr, stream

from . import _debug  # noqa: E402

_launch_count = 0


def launches() -> int:
    """Number of library kernel launchers invoked by this process (eager calls; a CUDA-graph
    replay re-issues the launches recorded at capture without passing through here)."""
    return _launch_count


def _count(n=1):
    global _launch_count
    _launch_count += n


def _lib_():
    return _lib.load()


def _index(t, dtype, name):
    """Index-like kernel input (token ids, positions, slots, lengths): the kernels read it as a dense
    array of `dtype` through a raw pointer, so a strided view or another integer width must be copied."""
    if t is None:
        return None
    if t.dtype != dtype:
        raise TypeError(f"{name}: expected {dtype}, got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


def _bf16(t, name):
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name}: CUDA kernels take bf16, got {t.dtype}")


# ----------------------------------------------------------------------------- norms / act
def rmsnorm(x, w, eps=1e-6, residual=None, out=None, gemma=False):
    """y = rmsnorm(x (+ residual)) * w.  `residual`, when given, is updated in place to x + residual."""
    if not x.is_cuda:
        y, new_res = reference.rmsnorm(x, w, eps, residual, gemma)
        if residual is not None:
            residual.copy_(new_res)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _bf16(x, "rmsnorm")
    hidden = x.shape[-1]
    x2 = x.reshape(-1, hidden)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    if out is None:
        out = torch.empty(x2.shape, dtype=x.dtype, device=x.device)
    o2 = out.reshape(-1, hidden)
    if residual is not None:
        assert residual.is_contiguous()
    check(_lib_().xllm_rmsnorm(ptr(o2), ptr(x2), ptr(residual), ptr(w), x2.shape[0], hidden, eps,
                               x2.stride(0), o2.stride(0), int(gemma), stream()), "rmsnorm")
    _count()
    return out.reshape(x.shape)


def act_and_mul(x, act="silu", out=None):
    if not x.is_cuda:
        return reference.act_and_mul(x, act)
    _bf16(x, "act_and_mul")
    d = x.shape[-1] // 2
    x2 = x.reshape(-1, 2 * d)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    if out is None:
        out = torch.empty((x2.shape[0], d), dtype=x.dtype, device=x.device)
    code = {"silu": 0, "gelu": 1, "gelu_tanh": 2, "gelu_pytorch_tanh": 2}[act]
    check(_lib_().xllm_act_and_mul(ptr(out), ptr(x2), x2.shape[0], d, x2.stride(0), code, stream()),
          "act_and_mul")
    _count()
    return out.reshape(*x.shape[:-1], d)


def silu_and_mul(x, out=None):
    return act_and_mul(x, "silu", out)


# ----------------------------------------------------------------------------- rope + kv write
def rope_kv_write(qkv, nq, nkv, d, positions, cos_sin, rot, slots=None, k_cache=None, v_cache=None,
                  q_norm_w=None, k_norm_w=None, eps=1e-6, interleaved=False, q_out=None,
                  return_kv=False):
    """Per-head RMSNorm (optional) + RoPE on packed QKV, K/V scattered into the paged cache.

    Returns q [T, nq, d] (and dense k, v when return_kv)."""
    T = qkv.shape[0]
    if _debug.enabled():
        _debug.check_range(positions, 0, cos_sin.shape[0], "rope_kv_write positions")
        if k_cache is not None and slots is not None:
            _debug.check_range(slots, 0, k_cache.shape[0] * k_cache.shape[2], "rope_kv_write slots", allow_negative_skip=True)
    if not qkv.is_cuda:
        q, k, v = reference.rope_kv(qkv, nq, nkv, d, positions, cos_sin, rot, q_norm_w, k_norm_w,
                                    eps, interleaved)
        if k_cache is not None and slots is not None:
            reference.write_kv_cache(k, v, k_cache, v_cache, slots)
        return (q, k, v) if return_kv else q
    _bf16(qkv, "rope_kv_write")
    assert qkv.stride(-1) == 1
    positions = _index(positions, torch.int64, "rope_kv_write positions")
    slots = _index(slots, torch.int32, "rope_kv_write slots")
    if q_out is None:
        q_out = torch.empty((T, nq, d), dtype=qkv.dtype, device=qkv.device)
    k_out = v_out = None
    if return_kv:
        k_out = torch.empty((T, nkv, d), dtype=qkv.dtype, device=qkv.device)
        v_out = torch.empty((T, nkv, d), dtype=qkv.dtype, device=qkv.device)
    page = k_cache.shape[2] if k_cache is not None else 1
    check(_lib_().xllm_rope_kv(ptr(qkv), qkv.stride(0), ptr(q_out), ptr(k_cache), ptr(v_cache),
                               ptr(k_out), ptr(v_out), ptr(q_norm_w), ptr(k_norm_w), ptr(cos_sin),
                               ptr(positions), ptr(slots), T, nq, nkv, d, rot, page,
                               int(interleaved), eps, stream()), "rope_kv")
    _count()
    return (q_out, k_out, v_out) if return_kv else q_out


# ----------------------------------------------------------------------------- attention
def decode_splits(batch, nkv, group, max_kv_len=None, n_sm=148):
    """Split-KV factor.  Without a context length: enough CTAs to cover ~2 per SM.  With one: the factor in
    1..16 that minimises (waves of CTAs over 2 resident per SM) x (tokens per split + a fixed cost for the
    split's set-up and its share of the merge), never less than 256 tokens per split — so that 128 CTAs of
    16k tokens become 2 x 8k in one wave instead of 3 x 5.5k in two."""
    ctas = batch * nkv * ((group + 15) // 16)
    slots = 2 * n_sm
    if max_kv_len is None:
        # the context is not known (a graph captured per batch size): of the two factors around one wave of
        # CTAs, the one that fills its waves better (128 CTAs: 2 x 128 in one wave, not 3 x 128 in 1.3)
        lo, hi = max(1, min(16, slots // ctas)), max(1, min(16, (slots + ctas - 1) // ctas))
        eff = lambda s_: (ctas * s_) / (((ctas * s_ + slots - 1) // slots) * slots)
        return hi if eff(hi) >= eff(lo) else lo
    best, best_cost = 1, None
    for s in range(1, 17):
        if s > 1 and max_kv_len // s < 256:
            break
        waves = (ctas * s + slots - 1) // slots
        cost = waves * ((max_kv_len + s - 1) // s + (192 if s > 1 else 0))
        if best_cost is None or cost < best_cost * 0.97:      # a larger factor must pay for its merge
            best, best_cost = s, cost
    return best


def decode_workspace(batch, nq, d, splits, device):
    if splits <= 1:
        return None
    return torch.empty(batch * nq * splits * (d + 1), dtype=torch.float32, device=device)


def paged_decode_attention(q, k_cache, v_cache, block_table, seq_lens, scale, splits=None,
                           workspace=None, out=None, window=0):
    """q: [B, nq, d] (one query token per sequence) -> [B, nq, d].  `window` > 0: every query sees
    its last `window` positions only (pages before them are not read)."""
    window = int(window or 0)
    _debug.check_block_table(block_table, seq_lens, k_cache.shape[0], k_cache.shape[2], "paged_decode_attention")
    if not q.is_cuda:
        y = reference.paged_decode_attention(q, k_cache, v_cache, block_table, seq_lens, scale, window)
        if out is not None:
            out.copy_(y)
            return out
        return y
    _bf16(q, "paged_decode_attention")
    seq_lens = _index(seq_lens, torch.int32, "paged_decode_attention seq_lens")
    assert block_table.dtype == torch.int32 and block_table.stride(-1) == 1
    B, nq, d = q.shape
    nkv, page = k_cache.shape[1], k_cache.shape[2]
    if splits is None:
        splits = decode_splits(B, nkv, nq // nkv)
    if splits > 1 and workspace is None:
        workspace = decode_workspace(B, nq, d, splits, q.device)
    if out is None:
        out = torch.empty((B, nq, d), dtype=q.dtype, device=q.device)
    assert q.stride(-1) == 1 and q.stride(1) == d
    if window > 0:
        check(_lib_().xllm_paged_decode_attn_window(ptr(out), ptr(q), q.stride(0), ptr(k_cache), ptr(v_cache),
                                                    ptr(block_table), block_table.stride(0), ptr(seq_lens), B,
                                                    nq, nkv, d, page, scale, splits, ptr(workspace), window, stream()),
              "paged_decode_attn_window")
    else:
        check(_lib_().xllm_paged_decode_attn(ptr(out), ptr(q), q.stride(0), ptr(k_cache), ptr(v_cache),
                                             ptr(block_table), block_table.stride(0), ptr(seq_lens), B,
                                             nq, nkv, d, page, scale, splits, ptr(workspace), stream()),
              "paged_decode_attn")
    _count(2 if splits > 1 else 1)
    return out


def paged_prefill_attention(q, k_cache, v_cache, block_table, cu_q, kv_lens, max_q_len, scale,
                            causal=True, window=0, out=None):
    """q: [T, nq, d] ragged by cu_q -> [T, nq, d]; attends to cache positions [0, kv_len)."""
    if _debug.enabled():
        _debug.check_block_table(block_table, kv_lens, k_cache.shape[0], k_cache.shape[2], "paged_prefill_attention")
        _debug.check_range(cu_q, 0, q.shape[0] + 1, "paged_prefill_attention cu_q")
    if not q.is_cuda:
        y = reference.paged_attention(q, k_cache, v_cache, block_table, cu_q, kv_lens, scale,
                                      causal, window)
        if out is not None:
            r0 = int(cu_q[0])
            out[r0:].copy_(y[r0:])
            return out
        return y
    _bf16(q, "paged_prefill_attention")
    cu_q = _index(cu_q, torch.int32, "paged_prefill_attention cu_q")
    kv_lens = _index(kv_lens, torch.int32, "paged_prefill_attention kv_lens")
    assert block_table.dtype == torch.int32 and block_table.stride(-1) == 1
    T, nq, d = q.shape
    nkv, page = k_cache.shape[1], k_cache.shape[2]
    if out is None:
        out = torch.empty((T, nq, d), dtype=q.dtype, device=q.device)
    assert q.stride(-1) == 1 and q.stride(1) == d
    B = kv_lens.shape[0]
    if (d == 128 and window == 0 and page in (16, 32, 64, 128) and k_cache.is_contiguous() and v_cache.is_contiguous()
            and os.environ.get("XLLM_PREFILL_ATTN", "tcgen05") != "legacy"):
        # tcgen05 / TMEM kernel (csrc/kernels/attn_prefill_tc.cu)
        check(_lib_().xllm_paged_prefill_attn_tc(ptr(out), out.stride(0), ptr(q), q.stride(0), T, ptr(k_cache),
                                                 ptr(v_cache), k_cache.shape[0], ptr(block_table),
                                                 block_table.stride(0), ptr(cu_q), ptr(kv_lens), B, int(max_q_len),
                                                 nq, nkv, page, scale, int(causal), stream()),
              "paged_prefill_attn_tc")
        _count()
        return out
    check(_lib_().xllm_paged_prefill_attn(ptr(out), out.stride(0), ptr(q), q.stride(0), ptr(k_cache),
                                          ptr(v_cache), ptr(block_table), block_table.stride(0),
                                          ptr(cu_q), ptr(kv_lens), B, int(max_q_len), nq, nkv, d,
                                          page, scale, int(causal), int(window), stream()),
          "paged_prefill_attn")
    _count()
    return out


# ----------------------------------------------------------------------------- sampling
def sample(logits, temperature=None, top_k=None, top_p=None, seed=0, offset=0, want_logprob=False,
           generator=None, out_ids=None, seeds=None, offsets=None, out_logprob=None):
    """Returns (ids int64 [B], logprob fp32 [B] | None).

    `seeds` (uint64/int64 [B]) and `offsets` (int32 [B]) give every row its own random stream: the seed
    of the row's sequence and the number of draws it has made so far.  Without them the batch-level
    (`seed`, `offset`) pair is used with the row index as the sub-stream."""
    if not logits.is_cuda:
        if seeds is not None and generator is None:
            ids = torch.empty(logits.shape[0], dtype=torch.int64)
            lp = torch.empty(logits.shape[0], dtype=torch.float32) if want_logprob else None
            for r in range(logits.shape[0]):
                g = torch.Generator().manual_seed((int(seeds[r]) * 1000003 + int(offsets[r] if offsets is not None else 0))
                                                  & 0x7FFFFFFFFFFFFFFF)
                sl = slice(r, r + 1)
                i, l = reference.sample(logits[sl], None if temperature is None else temperature[sl],
                                        None if top_k is None else top_k[sl], None if top_p is None else top_p[sl],
                                        g, want_logprob)
                ids[r] = i[0]
                if want_logprob:
                    lp[r] = l[0]
            return ids, lp
        if generator is None:       # the same (seed, offset) gives the same draw, as on the device
            generator = torch.Generator().manual_seed((int(seed) * 1000003 + int(offset)) & 0x7FFFFFFFFFFFFFFF)
        return reference.sample(logits, temperature, top_k, top_p, generator, want_logprob)
    B, V = logits.shape
    assert logits.stride(-1) == 1
    dt = 0 if logits.dtype == torch.bfloat16 else 1
    if dt == 1 and logits.dtype != torch.float32:
        logits = logits.float()
    if out_ids is None:
        out_ids = torch.empty(B, dtype=torch.int64, device=logits.device)
    lp = out_logprob
    if lp is None and want_logprob:
        lp = torch.empty(B, dtype=torch.float32, device=logits.device)
    if seeds is not None:
        check(_lib_().xllm_sample_rows(ptr(logits), logits.stride(0), dt, B, V, ptr(temperature), ptr(top_k),
                                       ptr(top_p), ptr(out_ids), ptr(lp), ptr(seeds), ptr(offsets), stream()),
              "sample_rows")
    else:
        check(_lib_().xllm_sample(ptr(logits), logits.stride(0), dt, B, V, ptr(temperature), ptr(top_k),
                                  ptr(top_p), ptr(out_ids), ptr(lp), int(seed), int(offset), stream()),
              "sample")
    _count()
    return out_ids, lp


def top_logprobs(logits, n):
    """The n most likely tokens of every row and their log-probabilities under softmax(logits):
    (ids int32 [B, n], logprobs fp32 [B, n]), most likely first."""
    if not logits.is_cuda:
        lp = torch.log_softmax(logits.float(), dim=-1)
        v, i = lp.topk(n, dim=-1)
        return i.to(torch.int32), v
    B, V = logits.shape
    assert logits.stride(-1) == 1
    dt = 0 if logits.dtype == torch.bfloat16 else 1
    if dt == 1 and logits.dtype != torch.float32:
        logits = logits.float()
    ids = torch.empty((B, n), dtype=torch.int32, device=logits.device)
    lp = torch.empty((B, n), dtype=torch.float32, device=logits.device)
    check(_lib_().xllm_top_logprobs(ptr(logits), logits.stride(0), dt, B, V, int(n), ptr(ids), ptr(lp), stream()),
          "top_logprobs")
    _count()
    return ids, lp


def apply_penalties(logits, ids, counts, freq=None, presence=None, repetition=None):
    if not logits.is_cuda:
        return reference.apply_penalties(logits, ids, counts, freq, presence, repetition)
    B, V = logits.shape
    dt = 0 if logits.dtype == torch.bfloat16 else 1
    check(_lib_().xllm_apply_penalties(ptr(logits), logits.stride(0), dt, B, V, ptr(ids), ptr(counts),
                                       ids.shape[1], ptr(freq), ptr(presence), ptr(repetition),
                                       stream()), "apply_penalties")
    _count()
    return logits


# ----------------------------------------------------------------------------- data movement
def embedding(ids, table, vocab_start=0, out=None):
    _debug.check_range(ids, 0, 1 << 31, "embedding ids")           # a vocabulary shard zero-fills ids of other shards
    if not table.is_cuda:
        loc = ids - vocab_start
        ok = (loc >= 0) & (loc < table.shape[0])
        y = table[loc.clamp(0, table.shape[0] - 1)]
        return y * ok[:, None].to(y.dtype)
    _bf16(table, "embedding")
    ids = _index(ids, torch.int64, "embedding ids")
    T, H = ids.shape[0], table.shape[1]
    if out is None:
        out = torch.empty((T, H), dtype=table.dtype, device=table.device)
    check(_lib_().xllm_embedding(ptr(out), ptr(table), ptr(ids), T, H, vocab_start,
                                 vocab_start + table.shape[0], stream()), "embedding")
    _count()
    return out


def gather_rows(x, idx, out=None):
    _debug.check_range(idx, 0, x.shape[0], "gather_rows idx")
    if not x.is_cuda:
        return x[idx]
    rows = idx.shape[0]
    row_bytes = x.shape[1] * x.element_size()
    if row_bytes % 16 != 0 or (x.stride(0) * x.element_size()) % 16 != 0:
        return x[idx]
    if out is None:
        out = torch.empty((rows, x.shape[1]), dtype=x.dtype, device=x.device)
    check(_lib_().xllm_gather_rows(ptr(out), ptr(x), ptr(idx), rows, row_bytes,
                                   x.stride(0) * x.element_size(), stream()), "gather_rows")
    _count()
    return out


def block_copy(cache_ptr_table, n_layers, pairs, block_bytes):
    """cache_ptr_table: int64 device tensor of base pointers; pairs: int32 [n, 2] device tensor."""
    check(_lib_().xllm_block_copy(ptr(cache_ptr_table), n_layers, ptr(pairs), pairs.shape[0],
                                  block_bytes, stream()), "block_copy")
    _count()


def decode_advance(tokens, positions, seq_lens, slots, block_table, sampled, page):
    if not tokens.is_cuda:
        m = seq_lens > 0
        tokens[m] = sampled[m]
        positions[m] += 1
        seq_lens[m] += 1
        pos = positions[m]
        rows = torch.nonzero(m).flatten()
        slots[m] = (block_table[rows, (pos // page).long()] * page + (pos % page)).to(slots.dtype)
        return
    check(_lib_().xllm_decode_advance(ptr(tokens), ptr(positions), ptr(seq_lens), ptr(slots),
                                      ptr(block_table), block_table.stride(0), ptr(sampled),
                                      tokens.shape[0], page, stream()), "decode_advance")
    _count()


def resolve_placeholders(tokens, prev):
    if not tokens.is_cuda:
        neg = tokens < 0
        tokens[neg] = prev[(-tokens[neg] - 1).long()]
        return tokens
    check(_lib_().xllm_resolve_placeholders(ptr(tokens), ptr(prev), tokens.numel(), prev.numel(),
                                            stream()), "resolve_placeholders")
    _count()
    return tokens


from .gemm import linear  # noqa: E402,F401
