"""Python front end of the tcgen05/TMEM/TMA bf16 GEMM (`csrc/kernels/gemm_tcgen05.cu`)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import I, L, P, check, ptr, stream

_lib.register_signature("xllm_gemm_bf16", [P, P, P, P, I, I, I, L, L, L, I, I, P])
_lib.register_signature("xllm_gemm_error_status", [], I)


def supported(x, w) -> bool:
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not x.is_cuda:
        return False
    K = x.shape[-1]
    N = w.shape[0]
    if K % 8 or N % 8 or w.stride(-1) != 1 or x.stride(-1) != 1 or w.dim() != 2:
        return False
    if w.stride(0) % 8 or (w.data_ptr() & 15) or (x.data_ptr() & 15):
        return False
    return True


def gemm_nt(x, w, bias=None, out=None, tile_n: int = 0, pair: int = -1):
    """y[..., N] = x[..., K] @ w[N, K]^T (+ bias)."""
    K = x.shape[-1]
    N = w.shape[0]
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    M = x2.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    o2 = out.reshape(M, N)
    assert o2.stride(-1) == 1 and o2.stride(0) % 8 == 0
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.is_contiguous()
    from . import _count
    check(_lib.load().xllm_gemm_bf16(ptr(x2), ptr(w), ptr(o2), ptr(bias), M, N, K, x2.stride(0), w.stride(0),
                                     o2.stride(0), tile_n, pair, stream()), "gemm_bf16")
    _count()
    return out.reshape(*x.shape[:-1], N)


def error_status() -> int:
    """Non-zero when a bounded wait inside a GEMM kernel expired since the last query."""
    return int(_lib.load().xllm_gemm_error_status())
