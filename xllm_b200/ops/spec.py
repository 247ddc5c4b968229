"""Speculative-decoding verification (rejection sampling) — kernel front end and reference.

Parity: RejectionSampler::forward (xllm/core/framework/sampling/rejection_sampler.cpp:65-360).
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import I, P, U64, check, ptr, stream

_lib.register_signature("xllm_spec_verify", [P, P, P, P, P, P, I, I, I, U64, U64, P])
_lib.register_signature("xllm_spec_verify_rows", [P, P, P, P, P, P, I, I, I, P, P, P])


def verify_reference(draft_ids, target_probs, draft_probs=None, greedy=None, generator=None):
    """Returns (tokens [B, K+1] int64 padded with -1, lengths [B] int32)."""
    B, K = draft_ids.shape
    out = torch.full((B, K + 1), -1, dtype=torch.int64)
    lens = torch.zeros(B, dtype=torch.int32)
    for b in range(B):
        g = bool(greedy[b]) if greedy is not None else False
        n = 0
        for i in range(K + 1):
            p = target_probs[b, i].float().cpu()
            if i == K:
                out[b, n] = int(p.argmax()) if g else int(torch.multinomial(p, 1, generator=generator))
                n += 1
                break
            x = int(draft_ids[b, i])
            if g:
                t = int(p.argmax())
                out[b, n] = t
                n += 1
                if t != x:
                    break
                continue
            q = draft_probs[b, i].float().cpu() if draft_probs is not None else torch.nn.functional.one_hot(
                torch.tensor(x), p.numel()).float()
            u = float(torch.rand((), generator=generator))
            if q[x] > 0 and u * q[x] <= p[x]:
                out[b, n] = x
                n += 1
                continue
            r = (p - q).clamp_min(0)
            out[b, n] = int(torch.multinomial(r / r.sum(), 1, generator=generator)) if r.sum() > 0 else int(p.argmax())
            n += 1
            break
        lens[b] = n
    return out, lens


def verify(draft_ids, target_probs, draft_probs=None, greedy=None, seed=0, offset=0, generator=None, seeds=None,
           offsets=None):
    """`seeds` / `offsets` ([B] int64 / int32): one random stream per row (the row's sequence seed and
    the tokens it has generated so far) instead of the batch-level (`seed`, `offset`)."""
    if not target_probs.is_cuda:
        if seeds is not None and generator is None:
            B, K = draft_ids.shape
            out = torch.full((B, K + 1), -1, dtype=torch.int64)
            lens = torch.zeros(B, dtype=torch.int32)
            for b in range(B):
                g = torch.Generator().manual_seed((int(seeds[b]) * 1000003 + 7919 * int(offsets[b] if offsets is not None else 0))
                                                  & 0x7FFFFFFFFFFFFFFF)
                o, l = verify_reference(draft_ids[b:b + 1], target_probs[b:b + 1],
                                        None if draft_probs is None else draft_probs[b:b + 1],
                                        None if greedy is None else greedy[b:b + 1], g)
                out[b], lens[b] = o[0], l[0]
            return out, lens
        return verify_reference(draft_ids, target_probs, draft_probs, greedy, generator)
    B, K = draft_ids.shape
    V = target_probs.shape[-1]
    assert target_probs.dtype == torch.float32 and target_probs.is_contiguous()
    out = torch.empty(B, K + 1, dtype=torch.int64, device=target_probs.device)
    lens = torch.empty(B, dtype=torch.int32, device=target_probs.device)
    g8 = greedy.to(torch.uint8) if greedy is not None else None
    if seeds is not None:
        check(_lib.load().xllm_spec_verify_rows(ptr(draft_ids), ptr(target_probs), ptr(draft_probs), ptr(g8), ptr(out),
                                                ptr(lens), B, K, V, ptr(seeds), ptr(offsets), stream()), "spec_verify")
        from . import _count
        _count()
        return out, lens
    check(_lib.load().xllm_spec_verify(ptr(draft_ids), ptr(target_probs), ptr(draft_probs), ptr(g8), ptr(out), ptr(lens),
                                       B, K, V, int(seed), int(offset), stream()), "spec_verify")
    from . import _count
    _count()
    return out, lens
