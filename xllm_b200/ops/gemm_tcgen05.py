"""Python front end of the tcgen05/TMEM/TMA bf16 GEMM (`csrc/kernels/gemm_tcgen05.cu`)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import I, L, P, check, ptr, stream

_lib.register_signature("xllm_gemm_bf16", [P, P, P, P, I, I, I, L, L, L, I, I, I, I, P])
_lib.register_signature("xllm_gemm_error_status", [], I)
_lib.register_signature("xllm_gemm_prepare", [], I)
_lib.register_signature("xllm_gemm_set_k_per_stage", [I], None)
_lib.register_signature("xllm_gemm_set_dual_issue", [I], None)
_lib.register_signature("xllm_pack_weight_bf16", [P, P, I, I, L, P])


def supported(x, w) -> bool:
    if isinstance(w, PackedWeight):
        return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] == w.shape[1]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not x.is_cuda:
        return False
    K = x.shape[-1]
    N = w.shape[0]
    if K % 8 or N % 8 or w.stride(-1) != 1 or x.stride(-1) != 1 or w.dim() != 2:
        return False
    if w.stride(0) % 8 or (w.data_ptr() & 15) or (x.data_ptr() & 15):
        return False
    return True


class PackedWeight:
    """A bf16 weight [N, K] stored tile-packed as [N/64][K/64][64][64]."""

    __slots__ = ("data", "shape")

    def __init__(self, data, shape):
        self.data = data
        self.shape = tuple(shape)


def can_pack(w) -> bool:
    return (w.is_cuda and w.dtype == torch.bfloat16 and w.dim() == 2 and w.shape[0] % 64 == 0
            and w.shape[1] % 64 == 0 and w.stride(1) == 1 and w.stride(0) % 8 == 0)


def pack_weight(w) -> PackedWeight:
    N, K = w.shape
    out = torch.empty(N * K, dtype=w.dtype, device=w.device)
    check(_lib.load().xllm_pack_weight_bf16(ptr(out), ptr(w), N, K, w.stride(0), stream()), "pack_weight")
    return PackedWeight(out, (N, K))


def unpack_weight(pw: PackedWeight):
    N, K = pw.shape
    return pw.data.view(N // 64, K // 64, 64, 64).permute(0, 2, 1, 3).reshape(N, K)


def gemm_nt(x, w, bias=None, out=None, tile_n: int = 0, pair: int = -1, split_k: int = 0):
    """y[..., N] = x[..., K] @ w[N, K]^T (+ bias).  `w` is a tensor or a PackedWeight."""
    packed = isinstance(w, PackedWeight)
    if packed:
        pw, w_shape, w_ptr, w_ld = w, w.shape, w.data.data_ptr(), w.shape[1]
    else:
        w_shape, w_ptr, w_ld = w.shape, w.data_ptr(), w.stride(0)
    K = x.shape[-1]
    N = w_shape[0]
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1 or x2.stride(0) % 8 or (x2.data_ptr() & 15):
        x2 = x2.contiguous()
    M = x2.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    o2 = out.reshape(M, N)
    assert o2.stride(-1) == 1 and o2.stride(0) % 8 == 0
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.is_contiguous()
    from . import _count
    check(_lib.load().xllm_gemm_bf16(ptr(x2), w_ptr, ptr(o2), ptr(bias), M, N, K, x2.stride(0), w_ld,
                                     o2.stride(0), tile_n, pair, int(packed), split_k, stream()), "gemm_bf16")
    _count()
    return out.reshape(*x.shape[:-1], N)


def set_k_per_stage(n: int):
    """1 = one 64-element K block per ring stage; 2 (default) = two for tiles narrower than 256."""
    _lib.load().xllm_gemm_set_k_per_stage(int(n))


def set_dual_issue(on: bool):
    """Two MMA-issuing warps or one (default) for the narrow-tile kernels."""
    _lib.load().xllm_gemm_set_dual_issue(int(bool(on)))


def prepare():
    """Allocate the split-K scratch of the current device (before CUDA-graph capture)."""
    check(_lib.load().xllm_gemm_prepare(), "gemm_prepare")


def error_status() -> int:
    """Non-zero when a bounded wait inside a GEMM kernel expired since the last query."""
    return int(_lib.load().xllm_gemm_error_status())
