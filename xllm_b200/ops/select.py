"""Selection ops of beam search and generative recommendation: log-softmax, radix top-k, beam step.

On CUDA these are the kernels of `csrc/kernels/beam.cu`; the CPU forms below are their fp32
references.  The reference's counterparts are xllm/core/kernels/cuda/air_log_softmax_last_dim.cu,
topk_last_dim.cuh and rec_beam_search.cu.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _lib
from ._lib import I, L, P, check, ptr, stream

_lib.register_signature("xllm_log_softmax", [P, L, I, I, I, P, P])
_lib.register_signature("xllm_radix_topk", [P, L, I, I, I, I, I, P, P, P])
_lib.register_signature("xllm_beam_step", [P, P, P, I, I, I, I, P, P, P, P])

MAX_K = 2048


def _dtype_code(x):
    if x.dtype == torch.bfloat16:
        return 0
    if x.dtype == torch.float32:
        return 1
    raise TypeError(f"expected bf16 or fp32 logits, got {x.dtype}")


def log_softmax(x: torch.Tensor) -> torch.Tensor:
    """[rows, V] -> fp32 log-probabilities."""
    if not x.is_cuda:
        return torch.log_softmax(x.float(), dim=-1)
    assert x.dim() == 2 and x.stride(1) == 1
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    check(_lib.load().xllm_log_softmax(ptr(x), x.stride(0), _dtype_code(x), x.shape[0], x.shape[1], ptr(out), stream()),
          "log_softmax")
    from . import _count
    _count()
    return out


def topk_reference(x: torch.Tensor, k: int, normalize: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Values descending, ties to the lowest index (a stable sort)."""
    v = x.float()
    # the order is that of the logits themselves (subtracting the normaliser can round two different
    # logits to the same log-probability)
    order = torch.sort(v, dim=-1, descending=True, stable=True).indices[:, :k]
    if normalize:
        v = torch.log_softmax(v, dim=-1)
    return v.gather(1, order), order.to(torch.int32)


def topk(x: torch.Tensor, k: int, normalize: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """The k largest entries of every row: (values fp32 [rows, k], indices int32 [rows, k]), sorted
    descending, ties to the lowest index.  normalize=True returns log-probabilities of the row."""
    assert x.dim() == 2 and 1 <= k <= x.shape[1]
    if not x.is_cuda or k > MAX_K or x.shape[1] >= (1 << 24):
        return topk_reference(x, k, normalize)
    assert x.stride(1) == 1
    rows, V = x.shape
    vals = torch.empty((rows, k), dtype=torch.float32, device=x.device)
    ids = torch.empty((rows, k), dtype=torch.int32, device=x.device)
    check(_lib.load().xllm_radix_topk(ptr(x), x.stride(0), _dtype_code(x), rows, V, k, int(normalize), ptr(vals), ptr(ids),
                                      stream()), "radix_topk")
    from . import _count
    _count()
    return vals, ids


def beam_step_reference(cand_lp, cand_ids, cum, n_out):
    B, W, k = cand_lp.shape
    score = (cand_lp.float() + cum.float()[:, :, None]).reshape(B, W * k)
    order = torch.sort(score, dim=-1, descending=True, stable=True).indices[:, :n_out]
    return (cand_ids.reshape(B, W * k).gather(1, order).to(torch.int32), (order // k).to(torch.int32),
            score.gather(1, order))


def beam_step(cand_lp: torch.Tensor, cand_ids: torch.Tensor, cum: torch.Tensor, n_out: int):
    """cand_lp / cand_ids [B, W, k]: the k best continuations of every beam; cum [B, W]: the beams'
    cumulative scores (-inf for a dead beam).  Returns (token, parent, score) [B, n_out] of the best
    n_out candidates per request, best first."""
    B, W, k = cand_lp.shape
    assert 1 <= n_out <= W * k
    if not cand_lp.is_cuda or n_out > MAX_K:
        return beam_step_reference(cand_lp, cand_ids, cum, n_out)
    cand_lp = cand_lp.float().contiguous()
    cand_ids = cand_ids.to(torch.int32).contiguous()
    cum = cum.float().contiguous()
    tok = torch.empty((B, n_out), dtype=torch.int32, device=cand_lp.device)
    par = torch.empty((B, n_out), dtype=torch.int32, device=cand_lp.device)
    sc = torch.empty((B, n_out), dtype=torch.float32, device=cand_lp.device)
    check(_lib.load().xllm_beam_step(ptr(cand_lp), ptr(cand_ids), ptr(cum), B, W, k, n_out, ptr(tok), ptr(par), ptr(sc),
                                     stream()), "beam_step")
    from . import _count
    _count()
    return tok, par, sc


def beam_topk(logits: torch.Tensor, cum: torch.Tensor, n_out: int):
    """One beam-search step from raw logits [W, V] of the live beams of ONE request and their
    cumulative scores [W]: (token, parent, score) [n_out] of the best continuations."""
    W, V = logits.shape
    k = min(n_out, V)
    lp, ids = topk(logits, k, normalize=True)
    tok, par, sc = beam_step(lp[None], ids[None], cum[None], min(n_out, W * k))
    return tok[0], par[0], sc[0]
