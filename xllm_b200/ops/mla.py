"""Front end of the MLA kernels (`csrc/kernels/mla.cu`): latent-cache write + rotary embeddings, and
absorbed multi-head latent attention over the paged latent cache.  CPU tensors take the PyTorch
reference of the same math."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import F, I, L, P, check, ptr, stream

_lib.register_signature("xllm_mla_decode", [P, P, L, P, P, I, P, P, P, I, I, I, F, I, P, P])
_lib.register_signature("xllm_mla_cache_write", [P, L, P, F, P, P, P, P, P, L, L, P, I, I, P])
_lib.register_signature("xllm_mla_decode_workspace", [L, I, I], L)

LATENT, ROT = 512, 64


def rope_pairs(v, cos_sin_rows):
    """Rotary embedding on adjacent pairs of the last dimension; cos_sin_rows [T, rot] = cos | sin."""
    half = v.shape[-1] // 2
    cs = cos_sin_rows.float()
    shape = [cs.shape[0]] + [1] * (v.dim() - 2) + [half]
    cos, sin = cs[:, :half].reshape(shape), cs[:, half:].reshape(shape)
    vf = v.float()
    x1, x2 = vf[..., 0::2], vf[..., 1::2]
    return torch.stack([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).flatten(-2).to(v.dtype)


def cache_write(kv_a, norm_w, eps, cos_sin, positions, slots, cache, q_rope, q_cat):
    """cache row of every token's slot = [rmsnorm(kv_a[:, :512]) * w | rope(kv_a[:, 512:])];
    q_cat[..., 512:] = rope(q_rope) for every head.  cache: any tensor whose memory is rows of 576."""
    T = kv_a.shape[0]
    # the kernels are built for DeepSeek's widths (512 + 64); anything else (tiny test models) takes
    # the tensor-op form, on whatever device it lives
    if not kv_a.is_cuda or norm_w.shape[0] != LATENT or kv_a.shape[1] != LATENT + ROT:
        from . import reference
        lat = norm_w.shape[0]                      # the reference takes any latent / rotary width
        c, _ = reference.rmsnorm(kv_a[:, :lat].contiguous(), norm_w, eps)
        cs = cos_sin[positions.long()]
        row = torch.cat([c.to(kv_a.dtype), rope_pairs(kv_a[:, lat:], cs)], dim=-1)
        rows = cache.view(-1, kv_a.shape[1])
        if slots is not None:
            ok = slots >= 0
            rows.index_copy_(0, slots[ok].long(), row[ok].to(rows.dtype))
        if q_cat is not None:
            q_cat[..., lat:] = rope_pairs(q_rope, cs)
        return
    assert kv_a.dtype == torch.bfloat16 and kv_a.stride(1) == 1 and kv_a.shape[1] == LATENT + ROT
    assert cos_sin.dtype == torch.float32 and cos_sin.shape[1] == ROT and cache.is_contiguous()
    nh = 0
    if q_cat is not None:
        nh = q_cat.shape[1]
        assert q_cat.is_contiguous() and q_rope.stride(2) == 1 and q_rope.shape[2] == ROT
    check(_lib.load().xllm_mla_cache_write(ptr(kv_a), kv_a.stride(0), ptr(norm_w), float(eps), ptr(cos_sin), ptr(positions),
                                           ptr(slots), ptr(cache), ptr(q_rope) if q_cat is not None else None,
                                           q_rope.stride(0) if q_cat is not None else 0,
                                           q_rope.stride(1) if q_cat is not None else 0, ptr(q_cat), T, nh, stream()),
          "mla_cache_write")
    from . import _count
    _count()


def decode_reference(q_cat, cache, block_table, seq_lens, bt_rows, scale, latent=LATENT):
    rows = cache.view(-1, cache.shape[-1]).float()
    page = cache.shape[-2]
    N, nh, _ = q_cat.shape
    out = torch.zeros(N, nh, latent, dtype=torch.float32, device=q_cat.device)
    for n in range(N):
        sl = int(seq_lens[n])
        if sl <= 0:
            continue
        bt = block_table[int(bt_rows[n]) if bt_rows is not None else n]
        idx = (bt[: (sl + page - 1) // page].long()[:, None] * page + torch.arange(page, device=q_cat.device)).flatten()[:sl]
        ctx = rows[idx]
        s = (q_cat[n].float() @ ctx.T) * scale
        out[n] = torch.softmax(s, dim=-1) @ ctx[:, :latent]
    return out.to(q_cat.dtype)


def decode(q_cat, cache, block_table, scale, seq_lens=None, positions=None, bt_rows=None, splits=None, out=None,
           latent=LATENT):
    """out [N, nh, 512] = absorbed MLA attention of q_cat [N, nh, 576] over the latent cache
    [n_blocks, (1,) page, 576].  Row n sees seq_lens[n] tokens (or positions[n] + 1) of the sequence whose
    block-table row is bt_rows[n] (default n)."""
    N, nh, _ = q_cat.shape
    if not q_cat.is_cuda or latent != LATENT or q_cat.shape[2] != LATENT + ROT:
        lens = seq_lens if seq_lens is not None else positions + 1
        y = decode_reference(q_cat, cache, block_table, lens, bt_rows, scale, latent)
        if out is not None:
            out.copy_(y)
            return out
        return y
    assert q_cat.dtype == torch.bfloat16 and q_cat.stride(2) == 1 and q_cat.stride(1) == LATENT + ROT
    assert cache.is_contiguous() and block_table.dtype == torch.int32
    page = cache.shape[-2]
    if out is None:
        out = torch.empty((N, nh, LATENT), dtype=q_cat.dtype, device=q_cat.device)
    assert out.is_contiguous()
    if N == 0:
        return out
    if splits is None:
        from . import decode_splits
        splits = decode_splits(N, 1, nh)
    ws = None
    if splits > 1:
        ws = torch.empty(int(_lib.load().xllm_mla_decode_workspace(N, nh, splits)), dtype=torch.float32, device=q_cat.device)
    check(_lib.load().xllm_mla_decode(ptr(out), ptr(q_cat), q_cat.stride(0), ptr(cache), ptr(block_table),
                                      block_table.stride(0), ptr(seq_lens), ptr(positions), ptr(bt_rows), N, nh, page,
                                      float(scale), int(splits), ptr(ws), stream()), "mla_decode")
    from . import _count
    _count(2 if splits > 1 else 1)
    return out
