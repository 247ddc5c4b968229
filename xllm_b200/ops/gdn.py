"""Gated delta rule (linear attention): the per-token state update of Qwen3-Next style layers.

`decode_step` advances a batch of per-request states by one token.  On CUDA it is one kernel
(csrc/kernels/gdn.cu: the state crosses HBM once in each direction); elsewhere the same arithmetic in
tensor ops, which is also the reference the GPU test compares against."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import I, L, P, check, ptr, stream

_lib.register_signature("xllm_gdn_decode_step", [P, P, P, P, P, P, P, P, I, I, I, I, P])
_lib.register_signature("xllm_gdn_prefill", [P, L, I, P, P, P, P, P, P, I, I, I, I, P])


def decode_step_reference(S, q, k, v, g, beta):
    """S [B, nv, dk, dv]; q, k [B, nv, dk]; v [B, nv, dv]; g, beta [B, nv] (fp32).  Returns (S', o [B, nv, dv])."""
    S = S * g.exp()[:, :, None, None]
    delta = (v - (S * k[..., None]).sum(-2)) * beta[..., None]
    S = S + k[..., None] * delta[:, :, None, :]
    return S, (S * q[..., None]).sum(-2)


def decode_step(state, slots, q, k, v, g, beta, out=None):
    """Updates `state[slots]` ([n_slots, nv, dk, dv] fp32) in place and returns o [B, nv, dv] (fp32)."""
    B, nv, dk = q.shape
    dv = v.shape[-1]
    if not state.is_cuda:
        S, o = decode_step_reference(state[slots], q.float(), k.float(), v.float(), g.float(), beta.float())
        state[slots] = S
        if out is not None:
            out.copy_(o)
            return out
        return o
    assert state.dtype == torch.float32 and state.is_contiguous() and slots.dtype == torch.int64
    q, k, v = q.float().contiguous(), k.float().contiguous(), v.float().contiguous()
    g, beta = g.float().contiguous(), beta.float().contiguous()
    if out is None or not out.is_contiguous() or out.dtype != torch.float32:
        res = torch.empty(B, nv, dv, dtype=torch.float32, device=q.device)
    else:
        res = out
    check(_lib.load().xllm_gdn_decode_step(ptr(state), ptr(slots.contiguous()), ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta),
                                           ptr(res), B, nv, dk, dv, stream()), "gdn_decode_step")
    if out is not None and res is not out:
        out.copy_(res)
        return out
    return res


def prefill_reference(S, q, k, v, g, beta):
    """The recurrence over the n tokens of one sequence: S [nv, dk, dv]; q, k [n, nv, dk]; v [n, nv, dv];
    g, beta [n, nv].  Returns (S', o [n, nv, dv])."""
    out = []
    S = S[None]
    for t in range(q.shape[0]):
        S, o = decode_step_reference(S, q[t:t + 1], k[t:t + 1], v[t:t + 1], g[t:t + 1], beta[t:t + 1])
        out.append(o[0])
    return S[0], torch.stack(out) if out else v.new_zeros(0, *v.shape[1:])


def prefill(state, slot: int, fresh: bool, q, k, v, g, beta, out=None):
    """Advances `state[slot]` over the n tokens of a prompt chunk in place (from zero when `fresh`) and
    returns o [n, nv, dv] fp32.  One kernel on CUDA for dk in {32, 64, 128, 256}."""
    n, nv, dk = q.shape
    dv = v.shape[-1]
    if not state.is_cuda or dk not in (32, 64, 128, 256):
        S0 = torch.zeros_like(state[slot]) if fresh else state[slot]
        S, o = prefill_reference(S0, q.float(), k.float(), v.float(), g.float(), beta.float())
        state[slot] = S
        if out is not None:
            out.copy_(o)
            return out
        return o
    assert state.dtype == torch.float32 and state.is_contiguous()
    q, k, v = q.float().contiguous(), k.float().contiguous(), v.float().contiguous()
    g, beta = g.float().contiguous(), beta.float().contiguous()
    res = out if (out is not None and out.is_contiguous() and out.dtype == torch.float32) else \
        torch.empty(n, nv, dv, dtype=torch.float32, device=q.device)
    check(_lib.load().xllm_gdn_prefill(ptr(state), int(slot), int(bool(fresh)), ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta),
                                       ptr(res), n, nv, dk, dv, stream()), "gdn_prefill")
    from . import _count
    _count()
    if out is not None and res is not out:
        out.copy_(res)
        return out
    return res
