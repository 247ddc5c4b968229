"""Beam attention for fixed-step generation: the beams of a request share the prompt's paged KV and add a
tail of at most `TAIL_MAX` generated tokens each.

Parity: xllm/core/layers/cuda/xattention.cpp with kernels/cuda/xattention/{decoder_reshape_and_cache,
cache_select,lse_combine}.cu (two-stage shared / unshared attention for generative recommendation).

Layout
  * prompt KV: the engine's paged cache, one block table row per REQUEST;
  * tail KV: `ku`, `vu` [tail_rows, nkv, tail_cap, d] — token t of the beam that occupied row r at step t
    is at [r, :, t, :], i.e. a paged cache whose page is a beam row, so the ordinary rotary + KV-write
    kernel fills it with slot = r * tail_cap + t;
  * `anc` int32 [tail_cap, rows]: anc[t, row] is the row that held `row`'s ancestor at step t
    (anc[n_tail - 1, row] == row).  After a beam step with parents `par`, `anc = anc[:, par]` — the KV
    itself never moves.

On CUDA with head_dim 128 the shared stage is one non-causal pass of the tcgen05 prefill kernel (beams are
the query rows; it also returns the rows' log-sum-exp) and `xattn_tail_merge_kernel` adds the tail.
"""
from __future__ import annotations

import math

import torch

from . import _lib
from ._lib import I, L, P, F, check, ptr, stream

TAIL_MAX = 8

_lib.register_signature("xllm_paged_prefill_attn_tc_lse",
                        [P, L, P, L, L, P, P, L, P, I, P, P, I, I, I, I, I, F, I, P, P])
_lib.register_signature("xllm_xattn_tail_merge", [P, L, P, P, L, P, P, P, I, I, I, I, I, I, I, F, P])


def xattention_reference(q, k_cache, v_cache, block_table, cu_q, kv_lens, ku, vu, anc, n_tail, scale):
    """fp32 oracle: every row attends to its request's whole prompt and to its own tail."""
    T, nq, d = q.shape
    nkv, page = k_cache.shape[1], k_cache.shape[2]
    g = nq // nkv
    out = torch.zeros(T, nq, d, dtype=torch.float32, device=q.device)
    for b in range(len(kv_lens)):
        r0, r1 = int(cu_q[b]), int(cu_q[b + 1])
        if r1 == r0:
            continue
        kl = int(kv_lens[b])
        nb = (kl + page - 1) // page
        blocks = block_table[b, :nb].long()
        kp = k_cache[blocks].permute(1, 0, 2, 3).reshape(nkv, nb * page, d)[:, :kl].float()
        vp = v_cache[blocks].permute(1, 0, 2, 3).reshape(nkv, nb * page, d)[:, :kl].float()
        for row in range(r0, r1):
            ks, vs = [kp], [vp]
            for t in range(n_tail):
                src = int(anc[t, row])
                ks.append(ku[src, :, t].float()[:, None])
                vs.append(vu[src, :, t].float()[:, None])
            k = torch.cat(ks, 1).repeat_interleave(g, 0)       # [nq, kl + n_tail, d]
            v = torch.cat(vs, 1).repeat_interleave(g, 0)
            s = torch.einsum("hd,hkd->hk", q[row].float(), k) * scale
            out[row] = torch.einsum("hk,hkd->hd", torch.softmax(s, -1), v)
    return out.to(q.dtype)


def supported(q, k_cache) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and k_cache.shape[2] in (16, 32, 64, 128)
            and k_cache.is_contiguous())


def xattention(q, k_cache, v_cache, block_table, cu_q, kv_lens, max_rows, ku, vu, anc, n_tail: int, scale: float,
               out=None):
    """q [T, nq, d] (rows of request b: cu_q[b]:cu_q[b+1], at most `max_rows` per request) -> [T, nq, d]."""
    assert 0 <= n_tail <= min(TAIL_MAX, ku.shape[2])
    from . import _debug
    if _debug.enabled():
        _debug.check_block_table(block_table, kv_lens, k_cache.shape[0], k_cache.shape[2], "xattention")
        _debug.check_range(anc[:n_tail], 0, ku.shape[0], "xattention ancestor rows")
        _debug.check_range(cu_q, 0, q.shape[0] + 1, "xattention cu_q")
    if not supported(q, k_cache):
        if q.is_cuda:
            from .gemm import _note_fallback
            _note_fallback("xattention shape", q, k_cache)
        y = xattention_reference(q, k_cache, v_cache, block_table, cu_q, kv_lens, ku, vu, anc, n_tail, scale)
        if out is not None:
            out.copy_(y)
            return out
        return y
    T, nq, d = q.shape
    nkv, page = k_cache.shape[1], k_cache.shape[2]
    assert q.stride(-1) == 1 and q.stride(1) == d
    assert block_table.dtype == torch.int32 and block_table.stride(-1) == 1
    cu_q, kv_lens = cu_q.to(torch.int32).contiguous(), kv_lens.to(torch.int32).contiguous()
    if out is None:
        out = torch.empty((T, nq, d), dtype=q.dtype, device=q.device)
    lse = torch.empty((T, nq), dtype=torch.float32, device=q.device)
    lib = _lib.load()
    B = kv_lens.shape[0]
    check(lib.xllm_paged_prefill_attn_tc_lse(ptr(out), out.stride(0), ptr(q), q.stride(0), T, ptr(k_cache), ptr(v_cache),
                                             k_cache.shape[0], ptr(block_table), block_table.stride(0), ptr(cu_q),
                                             ptr(kv_lens), B, int(max_rows), nq, nkv, page, scale, 0, ptr(lse), stream()),
          "xattention shared stage")
    anc = (anc if anc.dtype == torch.int32 else anc.to(torch.int32))
    if anc.stride(-1) != 1:
        anc = anc.contiguous()
    check(lib.xllm_xattn_tail_merge(ptr(out), out.stride(0), ptr(lse), ptr(q), q.stride(0), ptr(ku), ptr(vu), ptr(anc),
                                    anc.stride(0), int(n_tail), T, nq, nkv, d, ku.shape[2], scale, stream()),
          "xattention tail merge")
    from . import _count
    _count(2)
    return out


def default_scale(d: int) -> float:
    return 1.0 / math.sqrt(d)
