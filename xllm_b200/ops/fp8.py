"""fp8 (e4m3) quantisation and scaled GEMM.

`scaled_mm` is the tcgen05 `kind::f8f6f4` GEMM with per-tensor / per-token / per-channel scales (the
capability of the reference's CUTLASS `cutlass_scaled_mm`, cutlass_w8a8/scaled_mm_entry.cu:56-108).
128 x 128 block-scaled weights (DeepSeek-V3 checkpoints) are held in fp8 and expanded to bf16 by
`dequant_block128` right before the bf16 GEMM.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import I, L, P, check, ptr, stream

_lib.register_signature("xllm_gemm_fp8", [P, P, P, P, P, P, I, I, I, I, I, L, L, L, P])
_lib.register_signature("xllm_quant_fp8_per_token", [P, P, P, P, L, I, L, P])
_lib.register_signature("xllm_quant_fp8_group128", [P, P, P, L, I, L, P])
_lib.register_signature("xllm_dequant_fp8_block128", [P, P, P, L, I, P])
_lib.register_signature("xllm_gemm_fp8_block", [P, P, P, P, P, I, I, I, L, L, L, P])
_lib.register_signature("xllm_gemm_fp8_block_grouped", [P, P, P, P, P, P, I, I, I, I, L, L, L, P])

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


# ------------------------------------------------------------------ references (CPU path / oracle)
def quant_per_token_ref(x, static_scale=None):
    xf = x.float()
    if static_scale is not None:
        s = static_scale.float().reshape(())
        return (xf / s).clamp(-FP8_MAX, FP8_MAX).to(FP8), None
    s = xf.abs().amax(-1).clamp_min(1e-10) / FP8_MAX
    return (xf / s[:, None]).clamp(-FP8_MAX, FP8_MAX).to(FP8), s


def quant_group128_ref(x):
    T, H = x.shape
    g = x.float().view(T, H // 128, 128)
    s = g.abs().amax(-1).clamp_min(1e-10) / FP8_MAX
    return (g / s[..., None]).clamp(-FP8_MAX, FP8_MAX).to(FP8).view(T, H), s


def quant_block128_ref(w):
    """[N, K] -> (fp8 [N, K], scales [ceil(N/128), ceil(K/128)])."""
    N, K = w.shape
    Np, Kp = (N + 127) // 128 * 128, (K + 127) // 128 * 128
    wp = torch.zeros(Np, Kp, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    b = wp.view(Np // 128, 128, Kp // 128, 128)
    s = b.abs().amax((1, 3)).clamp_min(1e-10) / FP8_MAX
    q = (b / s[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).view(Np, Kp)[:N, :K].to(FP8)
    return q.contiguous(), s


def dequant_block128_ref(q, scales, dtype=torch.bfloat16):
    N, K = q.shape
    s = scales.repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    return (q.float() * s).to(dtype)


# ------------------------------------------------------------------ kernels
def quant_per_token(x, static_scale=None):
    if not x.is_cuda:
        return quant_per_token_ref(x, static_scale)
    T, H = x.shape
    q = torch.empty(T, H, dtype=FP8, device=x.device)
    s = None if static_scale is not None else torch.empty(T, dtype=torch.float32, device=x.device)
    check(_lib.load().xllm_quant_fp8_per_token(ptr(q), ptr(s), ptr(x), ptr(static_scale), T, H, x.stride(0), stream()),
          "quant_fp8_per_token")
    return q, s


def quant_group128(x):
    if not x.is_cuda:
        return quant_group128_ref(x)
    T, H = x.shape
    q = torch.empty(T, H, dtype=FP8, device=x.device)
    s = torch.empty(T, H // 128, dtype=torch.float32, device=x.device)
    check(_lib.load().xllm_quant_fp8_group128(ptr(q), ptr(s), ptr(x), T, H, x.stride(0), stream()), "quant_fp8_group128")
    return q, s


def rmsnorm_group_quant(x, w, eps=1e-6, residual=None, gemma=False):
    """rmsnorm(x (+ residual)) * w written as e4m3 with one scale per (row, 128 columns): the norm and
    the activation quantisation of a block-scaled fp8 linear in one pass over the row.  `residual`,
    when given, is updated in place.  Returns (q [T, H] e4m3, scales [T, H / 128] fp32)."""
    if not x.is_cuda:
        from . import reference
        y, new_res = reference.rmsnorm(x, w, eps, residual, gemma)
        if residual is not None:
            residual.copy_(new_res)
        return quant_group128_ref(y.to(torch.bfloat16))
    T, H = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and H % 128 == 0
    if residual is not None:
        assert residual.is_contiguous()
    q = torch.empty(T, H, dtype=FP8, device=x.device)
    s = torch.empty(T, H // 128, dtype=torch.float32, device=x.device)
    check(_lib.load().xllm_rmsnorm_group_fp8(ptr(q), ptr(s), ptr(x), ptr(residual), ptr(w), T, H, float(eps),
                                             x.stride(0), int(gemma), stream()), "rmsnorm_group_fp8")
    from . import _count
    _count()
    return q, s


def dequant_block128(q, scales, out=None):
    if not q.is_cuda:
        return dequant_block128_ref(q, scales)
    N, K = q.shape
    if out is None:
        out = torch.empty(N, K, dtype=torch.bfloat16, device=q.device)
    check(_lib.load().xllm_dequant_fp8_block128(ptr(out), ptr(q), ptr(scales), N, K, stream()), "dequant_fp8_block128")
    return out


def scaled_mm(a_q, w_q, a_scale, w_scale, bias=None, out=None):
    """bf16 C = (a_q @ w_q^T) * a_scale * w_scale (+ bias).  a_scale: scalar tensor or [M];
    w_scale: scalar tensor or [N]."""
    if not a_q.is_cuda:
        y = (a_q.float() * a_scale.float().reshape(-1, 1)) @ (w_q.float() * w_scale.float().reshape(-1, 1)).T
        if bias is not None:
            y = y + bias.float()
        return y.to(torch.bfloat16)
    M, K = a_q.shape
    N = w_q.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a_q.device)
    check(_lib.load().xllm_gemm_fp8(ptr(a_q), ptr(w_q), ptr(out), ptr(bias), ptr(a_scale), ptr(w_scale),
                                    int(a_scale.numel() > 1), int(w_scale.numel() > 1), M, N, K, a_q.stride(0),
                                    w_q.stride(0), out.stride(0), stream()), "gemm_fp8")
    from . import _count
    _count()
    return out


# ------------------------------------------------------------------ block-scaled GEMM (1 x 128 activations, 128 x 128 weights)
def block_scaled_mm_ref(a_q, a_scale, w_q, w_scale):
    """fp32 reference: dequantise both operands block by block, multiply."""
    M, K = a_q.shape
    N = w_q.shape[0]
    a = a_q.float() * a_scale.float().repeat_interleave(128, 1)[:, :K]
    w = w_q.float() * w_scale.float().repeat_interleave(128, 0)[:N].repeat_interleave(128, 1)[:, :K]
    return (a @ w.T).to(torch.bfloat16)


def block_scaled_mm(a_q, a_scale, w_q, w_scale, out=None):
    """bf16 C[M, N] = sum_kb (a_q[:, kb] @ w_q[:, kb]^T) * a_scale[:, kb, None] * w_scale[n // 128, kb]:
    a_q [M, K] / w_q [N, K] e4m3, a_scale [M, K / 128], w_scale [ceil(N / 128), K / 128] fp32."""
    if not a_q.is_cuda:
        y = block_scaled_mm_ref(a_q, a_scale, w_q, w_scale)
        if out is not None:
            out.copy_(y)
            return out
        return y
    M, K = a_q.shape
    N = w_q.shape[0]
    assert a_q.dtype == FP8 and w_q.dtype == FP8 and a_q.stride(1) == 1 and w_q.stride(1) == 1
    assert a_scale.dtype == torch.float32 and a_scale.is_contiguous() and a_scale.shape == (M, K // 128)
    assert w_scale.dtype == torch.float32 and w_scale.is_contiguous() and w_scale.shape == ((N + 127) // 128, K // 128)
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a_q.device)
    check(_lib.load().xllm_gemm_fp8_block(ptr(a_q), ptr(w_q), ptr(out), ptr(a_scale), ptr(w_scale), M, N, K,
                                          a_q.stride(0), w_q.stride(0), out.stride(0), stream()), "gemm_fp8_block")
    from . import _count
    _count()
    return out


def block_scaled_mm_grouped(a_q, a_scale, w_q, w_scale, tile_expert, out):
    """Grouped form: rows of a_q are sorted by expert in 128-row tiles, tile_expert [rows / 128] int32
    (-1: unused); w_q [E, N, K] e4m3, w_scale [E, N / 128, K / 128]; out [rows, N] bf16."""
    E, N, K = w_q.shape
    rows = a_q.shape[0]
    assert a_q.dtype == FP8 and w_q.dtype == FP8 and w_q.is_contiguous() and w_scale.is_contiguous()
    assert a_scale.shape == (rows, K // 128) and a_scale.is_contiguous() and N % 128 == 0
    check(_lib.load().xllm_gemm_fp8_block_grouped(ptr(a_q), ptr(w_q), ptr(out), ptr(a_scale), ptr(w_scale),
                                                  ptr(tile_expert), E, rows, N, K, a_q.stride(0), K, out.stride(0),
                                                  stream()), "gemm_fp8_block_grouped")
    from . import _count
    _count()
    return out


def linear_block_fp8(x, w_q, w_scale, out=None):
    """y = x @ dequant(w_q, w_scale)^T with the activation quantised on the fly in 1 x 128 groups."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    a_q, a_s = quant_group128(x2 if x2.stride(-1) == 1 else x2.contiguous())
    y = block_scaled_mm(a_q, a_s, w_q, w_scale, out=out)
    return y.reshape(*lead, w_q.shape[0])
