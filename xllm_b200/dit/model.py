"""A compact DiT (adaLN-zero transformer over latent patches) and its denoising loop with step
caches.  Parity in kind with the reference's DiT pipelines (xllm/models/dit/*): patchify, timestep
embedding, N blocks of (modulated attention + modulated MLP), unpatchify, an Euler flow-matching
sampler; the heavy pipelines (text encoders, VAE) are outside this build."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def timestep_embedding(t, dim):
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat([args.cos(), args.sin()], dim=-1)


class DiTBlock(torch.nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.heads = heads
        self.qkv = torch.nn.Linear(dim, 3 * dim)
        self.proj = torch.nn.Linear(dim, dim)
        self.fc1 = torch.nn.Linear(dim, 4 * dim)
        self.fc2 = torch.nn.Linear(4 * dim, dim)
        self.ada = torch.nn.Linear(dim, 6 * dim)

    def forward(self, x, c, st=None):
        """x: [B, T, D] (with sequence parallelism: this rank's T/sp tokens; attention then goes through
        the Ulysses all-to-all, parallel/dit_parallel.py)."""
        s1, b1, g1, s2, b2, g2 = self.ada(F.silu(c))[:, None].chunk(6, dim=-1)
        h = F.layer_norm(x, x.shape[-1:]) * (1 + s1) + b1
        B, T, D = h.shape
        q, k, v = self.qkv(h).view(B, T, 3, self.heads, D // self.heads).permute(2, 0, 3, 1, 4)
        if st is not None and st.sp_size > 1:
            from ..parallel.dit_parallel import ulysses_attention
            a = ulysses_attention(q.contiguous(), k.contiguous(), v.contiguous(), st).transpose(1, 2).reshape(B, T, D)
        else:
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, T, D)
        x = x + g1 * self.proj(a)
        h = F.layer_norm(x, x.shape[-1:]) * (1 + s2) + b2
        return x + g2 * self.fc2(F.gelu(self.fc1(h), approximate="tanh"))


class TinyDiT(torch.nn.Module):
    def __init__(self, in_ch=4, patch=2, dim=64, depth=4, heads=4, size=8):
        super().__init__()
        self.patch, self.in_ch, self.size = patch, in_ch, size
        self.embed = torch.nn.Linear(in_ch * patch * patch, dim)
        self.pos = torch.nn.Parameter(torch.randn(1, (size // patch) ** 2, dim) * 0.02)
        self.t_mlp = torch.nn.Sequential(torch.nn.Linear(dim, dim), torch.nn.SiLU(), torch.nn.Linear(dim, dim))
        self.blocks = torch.nn.ModuleList([DiTBlock(dim, heads) for _ in range(depth)])
        self.out = torch.nn.Linear(dim, in_ch * patch * patch)
        self.cond = torch.nn.Linear(dim, dim)      # conditioning vector (e.g. a pooled text embedding) -> modulation
        self.dim = dim

    def patchify(self, x):
        B, C, H, W = x.shape
        p = self.patch
        return x.view(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(B, (H // p) * (W // p), C * p * p)

    def unpatchify(self, y):
        B, T, _ = y.shape
        p, C, n = self.patch, self.in_ch, self.size // self.patch
        return y.view(B, n, n, C, p, p).permute(0, 3, 1, 4, 2, 5).reshape(B, C, n * p, n * p)

    def forward(self, x, t, cache=None, step=0, cond=None, st=None):
        """cond: [B, dim] conditioning vectors or None (the unconditional branch).  st: a
        DitParallelState; with sp_size > 1 the token sequence is sharded over the sp group between the
        patch embedding and the output projection."""
        c = self.t_mlp(timestep_embedding(t, self.dim))
        if cond is not None:
            c = c + self.cond(cond)
        h = self.embed(self.patchify(x)) + self.pos
        sp = st is not None and st.sp_size > 1
        if sp:
            from ..parallel.dit_parallel import gather_sequence, shard_sequence
            h = shard_sequence(h, st, dim=1)
        first = lambda z: self.blocks[0](z, c, st)

        def rest(z):
            for b in self.blocks[1:]:
                z = b(z, c, st)
            return z

        h = cache.run(step, h, first, rest) if cache is not None else rest(first(h))
        if sp:
            h = gather_sequence(h, st, dim=1)
        return self.unpatchify(self.out(h))

    @torch.no_grad()
    def sample(self, noise, steps=20, cache=None, cond=None, guidance_scale=1.0, st=None):
        """Euler integration of the predicted velocity from t = 1 to t = 0.  With a conditioning vector
        and guidance_scale != 1 every step evaluates the conditional and the unconditional branch
        (classifier-free guidance): on one rank as a batch of two, with a CFG group of two ranks one
        branch per rank and an all-gather of the two predictions."""
        x = noise
        ts = torch.linspace(1.0, 0.0, steps + 1)
        if cache is not None:
            cache.reset()
        guided = cond is not None and guidance_scale != 1.0
        cfg_parallel = guided and st is not None and st.cfg_size == 2
        for i in range(steps):
            t = ts[i].expand(x.shape[0]) * 1000
            if not guided:
                v = self.forward(x, t, cache, i, cond=cond, st=st)
            elif cfg_parallel:
                from ..parallel.dit_parallel import cfg_combine
                mine = cond if st.cfg_rank == 0 else None
                v = cfg_combine(self.forward(x, t, cache, i, cond=mine, st=st), st, guidance_scale)
            else:
                vc = self.forward(x, t, None, i, cond=cond, st=st)
                vu = self.forward(x, t, None, i, cond=None, st=st)
                v = vu + guidance_scale * (vc - vu)
            x = x + (ts[i + 1] - ts[i]) * v
        return x
