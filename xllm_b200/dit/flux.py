"""Flux-family diffusion transformer (MMDiT): double-stream blocks where image and text tokens keep their own
weights but attend jointly, single-stream blocks over the concatenation, AdaLN-Zero modulation by
(timestep, guidance, pooled text), 3-axis rotary positions, RMS-normalised q / k; with the flow-matching
Euler scheduler and the latent packing of the pipeline.

Parity: xllm/models/dit/flux/* (transformer_flux.h, the flow-match scheduler, pipeline_flux.h) of the
reference.  Parameter names follow the public checkpoints of the family (`transformer_blocks.N.attn.to_q`,
`single_transformer_blocks.N.proj_mlp`, `time_text_embed.timestep_embedder.linear_1`, ...), so a checkpoint's
`transformer/` directory loads by name.  No reference implementation of this family is installed here, so the
tests check the parts against independent formulations (rotary embedding against complex multiplication,
AdaLN-Zero identity at zero modulation, the joint attention against a dense computation, the scheduler
against its closed form) rather than against another library's output.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


@dataclass
class FluxArgs:
    in_channels: int = 64
    num_layers: int = 19                   # double-stream blocks
    num_single_layers: int = 38
    attention_head_dim: int = 128
    num_attention_heads: int = 24
    joint_attention_dim: int = 4096        # width of the T5 states
    pooled_projection_dim: int = 768       # width of the CLIP pooled state
    guidance_embeds: bool = True
    axes_dims_rope: Tuple[int, int, int] = (16, 56, 56)
    mlp_ratio: float = 4.0

    @property
    def inner(self) -> int:
        return self.attention_head_dim * self.num_attention_heads

    @staticmethod
    def from_config(cfg: dict) -> "FluxArgs":
        a = FluxArgs()
        for k in a.__dataclass_fields__:
            if cfg.get(k) is not None:
                v = cfg[k]
                setattr(a, k, tuple(v) if isinstance(v, list) else type(getattr(a, k))(v))
        return a


# ------------------------------------------------------------------------------------------ embeddings
def timestep_embedding(t: torch.Tensor, dim: int = 256, max_period: float = 10000.0) -> torch.Tensor:
    """Sinusoidal features [B, dim] = [cos | sin] of t x max_period^(-i / half)."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    ang = t.float()[:, None] * freqs[None]
    return torch.cat([ang.cos(), ang.sin()], dim=-1)


def rope_cos_sin(ids: torch.Tensor, axes: Sequence[int], theta: float = 10000.0):
    """ids [N, len(axes)] -> (cos, sin) [N, sum(axes)]: axis a owns axes[a] features, consecutive PAIRS share an
    angle pos_a x theta^(-2i / axes[a])."""
    cos, sin = [], []
    for a, d in enumerate(axes):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=ids.device) / d))
        ang = ids[:, a].double()[:, None] * inv[None]
        cos.append(ang.cos().repeat_interleave(2, dim=-1).float())
        sin.append(ang.sin().repeat_interleave(2, dim=-1).float())
    return torch.cat(cos, -1), torch.cat(sin, -1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, heads, N, d] with features in (real, imaginary) pairs."""
    xr, xi = x.float().reshape(*x.shape[:-1], -1, 2).unbind(-1)
    rot = torch.stack([-xi, xr], dim=-1).flatten(-2)
    return (x.float() * cos + rot * sin).to(x.dtype)


def _rms_head(x, w, eps=1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _ln(x, eps=1e-6):
    return F.layer_norm(x, x.shape[-1:], None, None, eps)


class FluxTransformer:
    """Functional module: parameters live in `self.p` under checkpoint names."""

    def __init__(self, args: FluxArgs, dtype=torch.float32, device="cpu"):
        self.args, self.dtype, self.device = args, dtype, torch.device(device)
        a, D = args, args.inner
        H = int(D * a.mlp_ratio)
        p: Dict[str, torch.Tensor] = {}

        def lin(name, out_f, in_f, bias=True):
            p[name + ".weight"] = torch.zeros(out_f, in_f, dtype=dtype, device=self.device)
            if bias:
                p[name + ".bias"] = torch.zeros(out_f, dtype=dtype, device=self.device)

        lin("x_embedder", D, a.in_channels)
        lin("context_embedder", D, a.joint_attention_dim)
        for e in ("timestep_embedder",) + (("guidance_embedder",) if a.guidance_embeds else ()):
            lin(f"time_text_embed.{e}.linear_1", D, 256)
            lin(f"time_text_embed.{e}.linear_2", D, D)
        lin("time_text_embed.text_embedder.linear_1", D, a.pooled_projection_dim)
        lin("time_text_embed.text_embedder.linear_2", D, D)
        hd = a.attention_head_dim
        for i in range(a.num_layers):
            b = f"transformer_blocks.{i}."
            lin(b + "norm1.linear", 6 * D, D)
            lin(b + "norm1_context.linear", 6 * D, D)
            for n in ("to_q", "to_k", "to_v", "add_q_proj", "add_k_proj", "add_v_proj", "to_out.0", "to_add_out"):
                lin(b + "attn." + n, D, D)
            for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
                p[b + f"attn.{n}.weight"] = torch.ones(hd, dtype=dtype, device=self.device)
            for ff in ("ff", "ff_context"):
                lin(b + ff + ".net.0.proj", H, D)
                lin(b + ff + ".net.2", D, H)
        for i in range(a.num_single_layers):
            b = f"single_transformer_blocks.{i}."
            lin(b + "norm.linear", 3 * D, D)
            lin(b + "proj_mlp", H, D)
            lin(b + "proj_out", D, D + H)
            for n in ("to_q", "to_k", "to_v"):
                lin(b + "attn." + n, D, D)
            for n in ("norm_q", "norm_k"):
                p[b + f"attn.{n}.weight"] = torch.ones(hd, dtype=dtype, device=self.device)
        lin("norm_out.linear", 2 * D, D)
        lin("proj_out", a.in_channels, D)
        self.p = p

    def init_random(self, std=0.02, seed=0):
        g = torch.Generator().manual_seed(seed)
        for k, t in self.p.items():
            if "norm_q" in k or "norm_k" in k or "norm_added" in k:
                t.fill_(1.0)
            elif k.endswith(".bias"):
                t.zero_()
            else:
                t.copy_((torch.randn(t.shape, generator=g) * std).to(t.dtype))

    def load_weights(self, weights, strict=True):
        seen = set()
        for name, w in weights:
            if name in self.p:
                self.p[name].copy_(w.to(self.dtype))
                seen.add(name)
            elif strict:
                raise KeyError(f"unexpected tensor {name}")
        if strict and set(self.p) - seen:
            raise KeyError(f"missing tensors: {sorted(set(self.p) - seen)[:5]}")
        return seen

    # ---------------------------------------------------------------------------------------- pieces
    def _lin(self, name, x):
        w, b = self.p[name + ".weight"], self.p.get(name + ".bias")
        if x.is_cuda and x.dtype == torch.bfloat16:
            # the tcgen05 GEMM with its bias epilogue (ops/gemm.py); shapes it cannot take are counted as fallbacks
            from ..ops import gemm
            return gemm.linear(x.reshape(-1, x.shape[-1]), w, b).view(*x.shape[:-1], w.shape[0])
        return F.linear(x, w, b)

    def conditioning(self, timestep, guidance, pooled):
        """temb [B, D] from t in [0, 1], the guidance scale and the pooled text state."""
        mlp = lambda e, v: self._lin(f"time_text_embed.{e}.linear_2", F.silu(self._lin(f"time_text_embed.{e}.linear_1", v)))
        emb = mlp("timestep_embedder", timestep_embedding(timestep * 1000.0).to(self.dtype))
        if self.args.guidance_embeds:
            g = guidance if guidance is not None else torch.ones_like(timestep)
            emb = emb + mlp("guidance_embedder", timestep_embedding(g * 1000.0).to(self.dtype))
        return emb + mlp("text_embedder", pooled.to(self.dtype))

    def _heads(self, x):
        B, N, _ = x.shape
        return x.view(B, N, self.args.num_attention_heads, self.args.attention_head_dim).transpose(1, 2)

    def _attend(self, q, k, v, cos, sin):
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v)
        return o.transpose(1, 2).reshape(o.shape[0], o.shape[2], -1)

    def double_block(self, i, img, txt, temb, cos, sin):
        b, p = f"transformer_blocks.{i}.", self.p
        mod = self._lin(b + "norm1.linear", F.silu(temb)).chunk(6, dim=1)           # shift, scale, gate (attn); shift, scale, gate (mlp)
        cmod = self._lin(b + "norm1_context.linear", F.silu(temb)).chunk(6, dim=1)
        x = _ln(img) * (1 + mod[1][:, None]) + mod[0][:, None]
        c = _ln(txt) * (1 + cmod[1][:, None]) + cmod[0][:, None]
        q = _rms_head(self._heads(self._lin(b + "attn.to_q", x)), p[b + "attn.norm_q.weight"])
        k = _rms_head(self._heads(self._lin(b + "attn.to_k", x)), p[b + "attn.norm_k.weight"])
        v = self._heads(self._lin(b + "attn.to_v", x))
        cq = _rms_head(self._heads(self._lin(b + "attn.add_q_proj", c)), p[b + "attn.norm_added_q.weight"])
        ck = _rms_head(self._heads(self._lin(b + "attn.add_k_proj", c)), p[b + "attn.norm_added_k.weight"])
        cv = self._heads(self._lin(b + "attn.add_v_proj", c))
        o = self._attend(torch.cat([cq, q], 2), torch.cat([ck, k], 2), torch.cat([cv, v], 2), cos, sin)   # text first
        nt = txt.shape[1]
        img = img + mod[2][:, None] * self._lin(b + "attn.to_out.0", o[:, nt:])
        txt = txt + cmod[2][:, None] * self._lin(b + "attn.to_add_out", o[:, :nt])
        ff = lambda pre, h: self._lin(b + pre + ".net.2", F.gelu(self._lin(b + pre + ".net.0.proj", h), approximate="tanh"))
        img = img + mod[5][:, None] * ff("ff", _ln(img) * (1 + mod[4][:, None]) + mod[3][:, None])
        txt = txt + cmod[5][:, None] * ff("ff_context", _ln(txt) * (1 + cmod[4][:, None]) + cmod[3][:, None])
        return img, txt

    def single_block(self, i, x, temb, cos, sin):
        b, p = f"single_transformer_blocks.{i}.", self.p
        shift, scale, gate = self._lin(b + "norm.linear", F.silu(temb)).chunk(3, dim=1)
        h = _ln(x) * (1 + scale[:, None]) + shift[:, None]
        q = _rms_head(self._heads(self._lin(b + "attn.to_q", h)), p[b + "attn.norm_q.weight"])
        k = _rms_head(self._heads(self._lin(b + "attn.to_k", h)), p[b + "attn.norm_k.weight"])
        o = self._attend(q, k, self._heads(self._lin(b + "attn.to_v", h)), cos, sin)
        mlp = F.gelu(self._lin(b + "proj_mlp", h), approximate="tanh")
        return x + gate[:, None] * self._lin(b + "proj_out", torch.cat([o, mlp], dim=2))

    @torch.no_grad()
    def forward(self, latents, text_states, pooled, timestep, img_ids, txt_ids, guidance=None, cache=None, step: int = 0):
        """latents [B, N_img, in_channels] (packed), text_states [B, N_txt, joint_attention_dim], pooled
        [B, pooled_projection_dim], timestep [B] in [0, 1], ids [N, 3] -> velocity [B, N_img, in_channels].
        `cache` (dit/cache.py, with the sampling step index `step`) may skip the blocks after the first."""
        a = self.args
        img = self._lin("x_embedder", latents.to(self.dtype))
        txt = self._lin("context_embedder", text_states.to(self.dtype))
        temb = self.conditioning(timestep, guidance, pooled)
        cos, sin = rope_cos_sin(torch.cat([txt_ids, img_ids], 0).to(self.device), a.axes_dims_rope)
        cos, sin = cos[None, None], sin[None, None]

        nt = txt.shape[1]

        def first(h):
            i_, t_ = self.double_block(0, h[:, nt:], h[:, :nt], temb, cos, sin)
            return torch.cat([t_, i_], dim=1)

        def rest(h, start=1):
            img_, txt_ = h[:, nt:], h[:, :nt]
            for i in range(start, a.num_layers):
                img_, txt_ = self.double_block(i, img_, txt_, temb, cos, sin)
            x = torch.cat([txt_, img_], dim=1)
            for i in range(a.num_single_layers):
                x = self.single_block(i, x, temb, cos, sin)
            return x

        h = torch.cat([txt, img], dim=1)
        if cache is not None and a.num_layers > 0:
            h = cache.run(step, h, first, rest)            # step caches: skip `rest` when the first block barely moved
        else:
            h = rest(h, 0)
        img = h[:, nt:]
        scale, shift = self._lin("norm_out.linear", F.silu(temb)).chunk(2, dim=1)
        return self._lin("proj_out", _ln(img) * (1 + scale[:, None]) + shift[:, None])


# ------------------------------------------------------------------------------------------ scheduler
class FlowMatchEulerScheduler:
    """sigma runs from 1 (noise) to 0 (image); x <- x + (sigma_next - sigma) * v.  The schedule is shifted
    towards the noisy end for large images: sigma' = e^mu / (e^mu + (1 / sigma - 1)), mu linear in the number
    of image tokens between (256 tokens, 0.5) and (4096 tokens, 1.15)."""

    def __init__(self, base_seq_len=256, max_seq_len=4096, base_shift=0.5, max_shift=1.15):
        self.base_seq_len, self.max_seq_len, self.base_shift, self.max_shift = base_seq_len, max_seq_len, base_shift, max_shift
        self.sigmas: List[float] = []

    def mu(self, image_seq_len: int) -> float:
        m = (self.max_shift - self.base_shift) / (self.max_seq_len - self.base_seq_len)
        return image_seq_len * m + (self.base_shift - m * self.base_seq_len)

    def set_timesteps(self, n: int, image_seq_len: int = 0, shift: bool = True) -> List[float]:
        sig = [1.0 - i * (1.0 - 1.0 / n) / max(n - 1, 1) for i in range(n)]            # linspace(1, 1/n, n)
        if shift:
            e = math.exp(self.mu(image_seq_len))
            sig = [e / (e + (1.0 / s - 1.0)) for s in sig]
        self.sigmas = sig + [0.0]
        return self.sigmas[:-1]

    def step(self, velocity: torch.Tensor, i: int, sample: torch.Tensor) -> torch.Tensor:
        return (sample.float() + (self.sigmas[i + 1] - self.sigmas[i]) * velocity.float()).to(sample.dtype)


# ------------------------------------------------------------------------------------------ latent packing
def pack_latents(x: torch.Tensor) -> torch.Tensor:
    """[B, C, H, W] -> [B, (H/2)(W/2), 4C]: every 2 x 2 patch of the latent image is one token."""
    B, C, H, W = x.shape
    return x.view(B, C, H // 2, 2, W // 2, 2).permute(0, 2, 4, 1, 3, 5).reshape(B, (H // 2) * (W // 2), C * 4)


def unpack_latents(x: torch.Tensor, H: int, W: int) -> torch.Tensor:
    B, N, D = x.shape
    return x.view(B, H // 2, W // 2, D // 4, 2, 2).permute(0, 3, 1, 4, 2, 5).reshape(B, D // 4, H, W)


def image_ids(H: int, W: int, device="cpu") -> torch.Tensor:
    """Position ids [(H/2)(W/2), 3] = (0, row, column) of the packed latent tokens."""
    ids = torch.zeros(H // 2, W // 2, 3, device=device)
    ids[..., 1] = torch.arange(H // 2, device=device)[:, None]
    ids[..., 2] = torch.arange(W // 2, device=device)[None, :]
    return ids.view(-1, 3)


# ------------------------------------------------------------------------------------------ pipeline
class FluxPipeline:
    """Prompt token ids -> image: CLIP pooled state and T5 states, `steps` Euler steps of the transformer over
    packed latents (guidance-distilled checkpoints take the guidance scale as an input; no second pass), VAE
    decode.  Tokenisation is the caller's (the two tokenizers ship with the checkpoint)."""

    def __init__(self, transformer: FluxTransformer, vae, clip, t5, latent_channels: int = 16):
        self.transformer, self.vae, self.clip, self.t5 = transformer, vae, clip, t5
        self.latent_channels = latent_channels
        self.scheduler = FlowMatchEulerScheduler()

    @torch.no_grad()
    def __call__(self, clip_ids: torch.Tensor, t5_ids: torch.Tensor, height: int = 1024, width: int = 1024, steps: int = 28,
                 guidance_scale: float = 3.5, seed: int = 0, cache=None, latents: Optional[torch.Tensor] = None) -> torch.Tensor:
        if height % 16 or width % 16:
            raise ValueError("height and width must be multiples of 16")
        tr = self.transformer
        dev, B = tr.device, clip_ids.shape[0]
        _, pooled = self.clip(clip_ids.to(dev))
        text = self.t5(t5_ids.to(dev))
        h, w = height // 8, width // 8
        if latents is None:
            g = torch.Generator().manual_seed(seed)
            latents = torch.randn(B, self.latent_channels, h, w, generator=g)
        x = pack_latents(latents.to(dev).to(tr.dtype))
        img_ids, txt_ids = image_ids(h, w, dev), torch.zeros(text.shape[1], 3, device=dev)
        sigmas = self.scheduler.set_timesteps(steps, x.shape[1])
        guidance = torch.full((B,), float(guidance_scale), device=dev) if tr.args.guidance_embeds else None
        if cache is not None:
            cache.reset()
        for i, s in enumerate(sigmas):
            t = torch.full((B,), float(s), device=dev)
            v = tr.forward(x, text, pooled, t, img_ids, txt_ids, guidance, cache=cache, step=i)
            x = self.scheduler.step(v, i, x)
        return self.vae.decode(unpack_latents(x, h, w)).clamp(-1, 1)
