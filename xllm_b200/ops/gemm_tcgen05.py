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


_lib.register_signature("xllm_gemm_bf16_act_mul", [P, P, P, I, I, I, L, L, L, I, P])
_lib.register_signature("xllm_act_and_mul_interleaved", [P, P, L, I, L, I, P])

ACT_CODES = {"silu": 1, "gelu": 2, "gelu_tanh": 3, "gelu_pytorch_tanh": 3}


def gemm_act_mul(x, w_interleaved, act: str = "silu", out=None):
    """act(x W_gate^T) * (x W_up^T) in one launch.  `w_interleaved` [2I, K]: groups of 128 rows =
    [64 gate rows | the 64 up rows of the same features] (see `interleave_gate_up`); returns [T, I]."""
    T, K = x.shape
    N = w_interleaved.shape[0]
    if out is None:
        out = torch.empty((T, N // 2), dtype=x.dtype, device=x.device)
    check(_lib.load().xllm_gemm_bf16_act_mul(ptr(x), ptr(w_interleaved), ptr(out), T, N, K, x.stride(0),
                                             w_interleaved.stride(0), out.stride(0), ACT_CODES[act], stream()),
          "gemm_bf16_act_mul")
    from . import _count
    _count()
    return out


def act_and_mul_interleaved(y, act: str = "silu", out=None):
    """Gated activation of a [T, 2I] tensor in the interleaved (64 gate | 64 up) column layout -> [T, I]."""
    T, N = y.shape
    if not y.is_cuda:
        g, u = y.view(T, N // 128, 2, 64).unbind(2)
        f = {"silu": torch.nn.functional.silu, "gelu": torch.nn.functional.gelu}.get(
            act, lambda t: torch.nn.functional.gelu(t, approximate="tanh"))
        return (f(g.float()) * u.float()).to(y.dtype).reshape(T, N // 2)
    if out is None:
        out = torch.empty((T, N // 2), dtype=y.dtype, device=y.device)
    code = {"silu": 0, "gelu": 1, "gelu_tanh": 2, "gelu_pytorch_tanh": 2}[act]
    check(_lib.load().xllm_act_and_mul_interleaved(ptr(out), ptr(y), T, N // 2, y.stride(0), code, stream()),
          "act_and_mul_interleaved")
    from . import _count
    _count()
    return out


def interleave_gate_up(gate, up):
    """[..., I, K] + [..., I, K] -> [..., 2I, K] with groups of 128 rows = 64 of gate, then the same 64 of up
    (leading dimensions, e.g. experts, are kept)."""
    *lead, I, K = gate.shape
    return torch.stack([gate.reshape(*lead, I // 64, 64, K), up.reshape(*lead, I // 64, 64, K)],
                       dim=-3).reshape(*lead, 2 * I, K)


def deinterleave_gate_up(w):
    """Inverse of `interleave_gate_up`: (gate [..., I, K], up [..., I, K])."""
    *lead, N, K = w.shape
    v = w.reshape(*lead, N // 128, 2, 64, K)
    return v[..., 0, :, :].reshape(*lead, N // 2, K), v[..., 1, :, :].reshape(*lead, N // 2, K)


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
