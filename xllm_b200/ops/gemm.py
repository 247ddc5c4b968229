"""Dense linear layers: y = x @ W^T (+ bias), W stored [out_features, in_features] (K-major).

On CUDA bf16 the product runs on the hand-written tcgen05/TMEM/TMA kernel
(`csrc/kernels/gemm_tcgen05.cu`).  ``XLLM_GEMM=cublas`` switches to ``torch.nn.functional.linear``
(cuBLAS) — that is the reference's own choice for every unquantised linear
(xllm/core/kernels/cuda/matmul.cpp:21-25) and is kept as the timed baseline / oracle.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

_MODE = os.environ.get("XLLM_GEMM", "auto")


def set_gemm_mode(mode: str):
    """'auto' | 'tcgen05' | 'cublas'."""
    global _MODE
    assert mode in ("auto", "tcgen05", "cublas")
    _MODE = mode


def gemm_mode() -> str:
    return _MODE


# Library GEMMs taken on a CUDA device although the mode asked for the hand-written kernel: counted by
# shape so that a serving run can report them (`library_fallbacks()`), and raised as an error when
# XLLM_GEMM_STRICT=1 (the benchmark and the GPU tests of the engines set it).
_FALLBACKS: dict = {}


def library_fallbacks() -> dict:
    """{(reason, x shape, w shape): calls} of CUDA linears that went to the tensor library."""
    return dict(_FALLBACKS)


def _note_fallback(reason, x, w):
    key = (reason, tuple(x.shape[-2:]) if x.dim() > 1 else tuple(x.shape), tuple(w.shape))
    _FALLBACKS[key] = _FALLBACKS.get(key, 0) + 1
    if os.environ.get("XLLM_GEMM_STRICT", "0") == "1":
        raise RuntimeError(f"library GEMM fallback ({reason}): x={tuple(x.shape)} {x.dtype}, w={tuple(w.shape)} {w.dtype}")


def linear(x, w, bias=None, out=None):
    if x.is_cuda and _MODE != "cublas":
        if x.dtype == torch.bfloat16:
            from . import gemm_tcgen05
            if gemm_tcgen05.supported(x, w):
                return gemm_tcgen05.gemm_nt(x, w, bias=bias, out=out)
            if _MODE == "tcgen05":
                raise RuntimeError(f"tcgen05 GEMM does not support shapes x={tuple(x.shape)} w={tuple(w.shape)}")
            _note_fallback("shape or alignment", x, w)
        else:
            _note_fallback("dtype", x, w)
    y = F.linear(x, w, bias)
    if out is not None:
        out.copy_(y)
        return out
    return y
