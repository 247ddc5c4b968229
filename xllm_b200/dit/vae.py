"""Latent decoder of the image pipelines: a convolutional decoder with residual blocks, one single-head attention
block in the middle and nearest-neighbour upsampling (the `AutoencoderKL` decoder layout of the public
checkpoints: `decoder.conv_in`, `decoder.mid_block.{resnets,attentions}`, `decoder.up_blocks.N.{resnets,upsamplers}`,
`decoder.conv_norm_out`, `decoder.conv_out`).  Parity: xllm/models/dit/autoencoders/autoencoder_kl.h."""
from __future__ import annotations

from typing import Dict, Sequence

import torch
import torch.nn.functional as F


class VaeDecoder:
    def __init__(self, latent_channels=16, out_channels=3, block_out_channels: Sequence[int] = (128, 256, 512, 512),
                 layers_per_block=2, norm_groups=32, scaling_factor=0.3611, shift_factor=0.1159, dtype=torch.float32,
                 device="cpu"):
        self.dtype, self.device, self.groups = dtype, torch.device(device), norm_groups
        self.scaling_factor, self.shift_factor = scaling_factor, shift_factor
        self.layers = layers_per_block + 1
        rev = list(reversed(block_out_channels))
        self.rev = rev
        z = lambda *s: torch.zeros(*s, dtype=dtype, device=self.device)
        p: Dict[str, torch.Tensor] = {}

        def conv(name, o, i, k):
            p[name + ".weight"], p[name + ".bias"] = z(o, i, k, k), z(o)

        def norm(name, c):
            p[name + ".weight"], p[name + ".bias"] = torch.ones(c, dtype=dtype, device=self.device), z(c)

        def resnet(name, i, o):
            norm(name + ".norm1", i)
            conv(name + ".conv1", o, i, 3)
            norm(name + ".norm2", o)
            conv(name + ".conv2", o, o, 3)
            if i != o:
                conv(name + ".conv_shortcut", o, i, 1)

        top = rev[0]
        conv("decoder.conv_in", top, latent_channels, 3)
        resnet("decoder.mid_block.resnets.0", top, top)
        resnet("decoder.mid_block.resnets.1", top, top)
        norm("decoder.mid_block.attentions.0.group_norm", top)
        for n in ("to_q", "to_k", "to_v", "to_out.0"):
            p[f"decoder.mid_block.attentions.0.{n}.weight"], p[f"decoder.mid_block.attentions.0.{n}.bias"] = z(top, top), z(top)
        prev = top
        for b, ch in enumerate(rev):
            for j in range(self.layers):
                resnet(f"decoder.up_blocks.{b}.resnets.{j}", prev if j == 0 else ch, ch)
            if b < len(rev) - 1:
                conv(f"decoder.up_blocks.{b}.upsamplers.0.conv", ch, ch, 3)
            prev = ch
        norm("decoder.conv_norm_out", rev[-1])
        conv("decoder.conv_out", out_channels, rev[-1], 3)
        self.p = p

    def init_random(self, std=0.05, seed=0):
        g = torch.Generator().manual_seed(seed)
        for k, t in self.p.items():
            if "norm" in k and k.endswith(".weight"):
                t.fill_(1.0)
            elif k.endswith(".bias"):
                t.zero_()
            else:
                t.copy_((torch.randn(t.shape, generator=g) * std).to(t.dtype))

    def load_weights(self, weights):
        seen = set()
        for name, w in weights:
            if name in self.p:
                self.p[name].copy_(w.reshape(self.p[name].shape).to(self.dtype))   # older files keep the attention as 1 x 1 convs
                seen.add(name)
        return seen

    def _gn(self, name, x):
        return F.group_norm(x, self.groups, self.p[name + ".weight"], self.p[name + ".bias"], 1e-6)

    def _conv(self, name, x, pad):
        return F.conv2d(x, self.p[name + ".weight"], self.p[name + ".bias"], padding=pad)

    def _resnet(self, name, x):
        h = self._conv(name + ".conv1", F.silu(self._gn(name + ".norm1", x)), 1)
        h = self._conv(name + ".conv2", F.silu(self._gn(name + ".norm2", h)), 1)
        if name + ".conv_shortcut.weight" in self.p:
            x = self._conv(name + ".conv_shortcut", x, 0)
        return x + h

    def _attention(self, name, x):
        B, C, H, W = x.shape
        h = self._gn(name + ".group_norm", x).view(B, C, H * W).transpose(1, 2)
        lin = lambda n: F.linear(h, self.p[f"{name}.{n}.weight"], self.p[f"{name}.{n}.bias"])
        o = F.scaled_dot_product_attention(lin("to_q")[:, None], lin("to_k")[:, None], lin("to_v")[:, None])[:, 0]
        o = F.linear(o, self.p[name + ".to_out.0.weight"], self.p[name + ".to_out.0.bias"])
        return x + o.transpose(1, 2).reshape(B, C, H, W)

    @torch.no_grad()
    def decode(self, latents: torch.Tensor) -> torch.Tensor:
        """latents [B, C, h, w] as the transformer leaves them -> images [B, 3, 8h, 8w] in [-1, 1]."""
        x = latents.to(self.dtype) / self.scaling_factor + self.shift_factor
        x = self._conv("decoder.conv_in", x, 1)
        x = self._resnet("decoder.mid_block.resnets.0", x)
        x = self._attention("decoder.mid_block.attentions.0", x)
        x = self._resnet("decoder.mid_block.resnets.1", x)
        for b in range(len(self.rev)):
            for j in range(self.layers):
                x = self._resnet(f"decoder.up_blocks.{b}.resnets.{j}", x)
            if b < len(self.rev) - 1:
                x = self._conv(f"decoder.up_blocks.{b}.upsamplers.0.conv", F.interpolate(x, scale_factor=2.0, mode="nearest"), 1)
        return self._conv("decoder.conv_out", F.silu(self._gn("decoder.conv_norm_out", x)), 1)
