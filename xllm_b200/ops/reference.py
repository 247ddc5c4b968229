"""Plain PyTorch (fp32 math) references of every kernel in the sm_100a library.

They are the CPU execution path (unit tests, the tiny fp32 model) and the oracle the GPU
numerics tests compare against.
"""
from __future__ import annotations

import math

import torch


def rmsnorm(x, w, eps, residual=None, gemma=False):
    """Returns (normed, new_residual). new_residual = x + residual (rounded to x.dtype)."""
    xf = x.float()
    if residual is not None:
        xf = (xf + residual.float()).to(x.dtype).float()
        new_res = xf.to(x.dtype)
    else:
        new_res = None
    var = xf.pow(2).mean(-1, keepdim=True)
    wf = w.float()
    if gemma:
        wf = wf + 1.0
    y = xf * torch.rsqrt(var + eps) * wf
    return y.to(x.dtype), new_res


def act_and_mul(x, act="silu"):
    d = x.shape[-1] // 2
    a, b = x[..., :d].float(), x[..., d:].float()
    if act == "silu":
        g = torch.nn.functional.silu(a)
    elif act == "gelu":
        g = torch.nn.functional.gelu(a)
    else:
        g = torch.nn.functional.gelu(a, approximate="tanh")
    return (g * b).to(x.dtype)


def build_cos_sin_cache(rot_dim, max_pos, theta, scaling=None, device="cpu"):
    """fp32 [max_pos, rot_dim]: cos in the first half, sin in the second half.

    `scaling` follows HF `rope_scaling` (types: linear, dynamic (treated as base), llama3, yarn).
    Parity: xllm/core/layers/common/rotary_embedding_util.cpp of the reference.
    """
    half = rot_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / rot_dim))
    mscale = 1.0
    if scaling:
        typ = scaling.get("rope_type", scaling.get("type", "default"))
        factor = float(scaling.get("factor", 1.0))
        if typ == "linear":
            inv_freq = inv_freq / factor
        elif typ == "llama3":
            low = float(scaling.get("low_freq_factor", 1.0))
            high = float(scaling.get("high_freq_factor", 4.0))
            orig = float(scaling.get("original_max_position_embeddings", 8192))
            wavelen = 2 * math.pi / inv_freq
            smooth = (orig / wavelen - low) / (high - low)
            scaled = torch.where(wavelen > orig / low, inv_freq / factor, inv_freq)
            mid = (wavelen <= orig / low) & (wavelen >= orig / high)
            scaled = torch.where(mid, (1 - smooth) * inv_freq / factor + smooth * inv_freq, scaled)
            inv_freq = scaled
        elif typ == "yarn":
            orig = float(scaling.get("original_max_position_embeddings", 4096))
            beta_fast = float(scaling.get("beta_fast", 32))
            beta_slow = float(scaling.get("beta_slow", 1))

            def corr_dim(n_rot):
                return rot_dim * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(theta))

            lo = max(math.floor(corr_dim(beta_fast)), 0)
            hi = min(math.ceil(corr_dim(beta_slow)), rot_dim - 1)
            ramp = ((torch.arange(half, dtype=torch.float64) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
            mask = 1.0 - ramp
            inv_freq = inv_freq / factor * (1 - mask) + inv_freq * mask
            ms = float(scaling.get("mscale", 1.0))
            ms_all = float(scaling.get("mscale_all_dim", 0.0))

            def get_mscale(scale, m):
                return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

            if "attention_factor" in scaling:
                mscale = float(scaling["attention_factor"])
            elif ms_all:
                mscale = get_mscale(factor, ms) / get_mscale(factor, ms_all)
            else:
                mscale = get_mscale(factor, 1.0)
    t = torch.arange(max_pos, dtype=torch.float64)
    freqs = torch.outer(t, inv_freq)
    cache = torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1).float()
    return cache.to(device)


def rope_kv(qkv, nq, nkv, d, positions, cos_sin, rot, q_norm_w=None, k_norm_w=None, eps=1e-6,
            interleaved=False):
    """Returns (q [T,nq,d], k [T,nkv,d], v [T,nkv,d]) after optional per-head RMSNorm and RoPE."""
    T = qkv.shape[0]
    q, k, v = qkv.split([nq * d, nkv * d, nkv * d], dim=-1)
    q = q.reshape(T, nq, d)
    k = k.reshape(T, nkv, d)
    v = v.reshape(T, nkv, d)

    def norm(x, w):
        if w is None:
            return x.float()
        xf = x.float()
        y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype).float()
        return y * w.float()

    qf, kf = norm(q, q_norm_w), norm(k, k_norm_w)
    if cos_sin is not None:
        half = rot // 2
        cs = cos_sin[positions.long()].float()  # [T, rot]
        cos, sin = cs[:, None, :half], cs[:, None, half:]

        def rope(x):
            xr, xp = x[..., :rot], x[..., rot:]
            if interleaved:
                x1, x2 = xr[..., 0::2], xr[..., 1::2]
                o1 = x1 * cos - x2 * sin
                o2 = x2 * cos + x1 * sin
                out = torch.stack([o1, o2], dim=-1).flatten(-2)
            else:
                x1, x2 = xr[..., :half], xr[..., half:]
                out = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)
            return torch.cat([out, xp], dim=-1)

        qf, kf = rope(qf), rope(kf)
    return qf.to(qkv.dtype), kf.to(qkv.dtype), v.contiguous()


def write_kv_cache(k, v, k_cache, v_cache, slots):
    """k,v: [T, nkv, d]; caches [n_blocks, nkv, page, d]; slots [T] (negative => skip)."""
    page = k_cache.shape[2]
    valid = slots >= 0
    s = slots[valid].long()
    blk, off = s // page, s % page
    k_cache[blk, :, off, :] = k[valid]
    v_cache[blk, :, off, :] = v[valid]


def _gather_kv(cache, block_table_row, kv_len):
    page = cache.shape[2]
    n_pages = (kv_len + page - 1) // page
    blocks = block_table_row[:n_pages].long()
    x = cache[blocks]  # [n_pages, nkv, page, d]
    x = x.permute(1, 0, 2, 3).reshape(cache.shape[1], n_pages * page, cache.shape[3])
    return x[:, :kv_len]  # [nkv, kv_len, d]


def paged_attention(q, k_cache, v_cache, block_table, cu_q, kv_lens, scale, causal=True, window=0):
    """q: [T, nq, d]; returns [T, nq, d]. Sequence b owns q rows cu_q[b]:cu_q[b+1]."""
    out = torch.zeros_like(q)
    nq, nkv = q.shape[1], k_cache.shape[1]
    group = nq // nkv
    B = len(kv_lens)
    for b in range(B):
        qs, qe = int(cu_q[b]), int(cu_q[b + 1])
        ql, kl = qe - qs, int(kv_lens[b])
        if ql == 0 or kl == 0:
            continue
        k = _gather_kv(k_cache, block_table[b], kl).float().repeat_interleave(group, dim=0)
        v = _gather_kv(v_cache, block_table[b], kl).float().repeat_interleave(group, dim=0)
        qq = q[qs:qe].float().transpose(0, 1)  # [nq, ql, d]
        s = torch.einsum("hqd,hkd->hqk", qq, k) * scale
        qpos = torch.arange(ql, device=q.device)[:, None] + (kl - ql)
        kpos = torch.arange(kl, device=q.device)[None, :]
        mask = torch.zeros(ql, kl, dtype=torch.bool, device=q.device)
        if causal:
            mask |= kpos > qpos
        if window and window > 0:
            mask |= kpos <= qpos - window
        s = s.masked_fill(mask[None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        p = torch.nan_to_num(p, nan=0.0)
        o = torch.einsum("hqk,hkd->hqd", p, v)
        out[qs:qe] = o.transpose(0, 1).to(q.dtype)
    return out


def paged_decode_attention(q, k_cache, v_cache, block_table, seq_lens, scale, window=0):
    """q: [B, nq, d] one token per sequence."""
    B = q.shape[0]
    cu = torch.arange(B + 1, dtype=torch.int32, device=q.device)
    return paged_attention(q, k_cache, v_cache, block_table, cu, seq_lens, scale, causal=True, window=window)


def apply_penalties(logits, ids, counts, freq, presence, repetition):
    """In place. ids/counts: [B, U] (id < 0 => unused)."""
    B, V = logits.shape
    for b in range(B):
        m = (ids[b] >= 0) & (counts[b] > 0 if counts is not None else True)
        i = ids[b][m].long()
        c = counts[b][m].float() if counts is not None else torch.ones_like(i, dtype=torch.float)
        x = logits[b, i].float()
        if repetition is not None:
            r = float(repetition[b])
            x = torch.where(x > 0, x / r, x * r)
        f = float(freq[b]) if freq is not None else 0.0
        p = float(presence[b]) if presence is not None else 0.0
        x = x - f * c - p
        logits[b, i] = x.to(logits.dtype)
    return logits


def filtered_distribution(logits, temperature, top_k, top_p):
    """Probabilities after temperature / top-k / top-p, per row (fp32). Greedy rows -> one-hot."""
    B, V = logits.shape
    out = torch.zeros(B, V, dtype=torch.float32, device=logits.device)
    for b in range(B):
        t = float(temperature[b]) if temperature is not None else 0.0
        x = logits[b].float()
        if not t > 0:
            out[b, int(x.argmax())] = 1.0
            continue
        p = torch.softmax(x / t, dim=-1)
        k = int(top_k[b]) if top_k is not None else 0
        tp = float(top_p[b]) if top_p is not None else 1.0
        sp, si = torch.sort(p, descending=True, stable=True)
        keep = torch.ones(V, dtype=torch.bool, device=logits.device)
        if 0 < k < V:
            keep &= torch.arange(V, device=logits.device) < k
        if tp < 1.0:
            before = torch.cumsum(sp, 0) - sp
            keep &= before < tp
        # ties with the last kept value stay in (the kernel keeps {p >= threshold})
        thr = sp[keep].min()
        mask = p >= thr
        q = torch.where(mask, p, torch.zeros_like(p))
        out[b] = q / q.sum()
    return out


def sample(logits, temperature=None, top_k=None, top_p=None, generator=None, want_logprob=False):
    probs = filtered_distribution(logits, temperature, top_k, top_p)
    ids = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    for b in range(logits.shape[0]):
        t = float(temperature[b]) if temperature is not None else 0.0
        if not t > 0:
            ids[b] = probs[b].argmax()
        else:
            ids[b] = torch.multinomial(probs[b], 1, generator=generator)[0]
    lp = None
    if want_logprob:
        lp = torch.zeros(logits.shape[0], dtype=torch.float32, device=logits.device)
        for b in range(logits.shape[0]):
            t = float(temperature[b]) if temperature is not None else 0.0
            if not t > 0:
                lp[b] = torch.log_softmax(logits[b].float(), -1)[ids[b]]
            else:
                lp[b] = torch.log(probs[b, ids[b]])
    return ids, lp
