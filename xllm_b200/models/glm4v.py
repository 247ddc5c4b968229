"""GLM-4V family: a vision tower with learned, bicubically resampled position embeddings, RMSNorm /
SwiGLU blocks with 2-D rotary attention, a strided-convolution downsample and a gated merger; in front of
the GLM-4 decoder (sandwich norms, half of each head rotated in interleaved pairs) driven by 3-axis rotary
positions.  The same tower in front of a Qwen3 decoder is the reference's `oxygenvlm`.

Parity: xllm/models/vlm/oxygen_vlm.h (OxygenVisionPatchEmbed / Embeddings / PatchMerger /
VisionTransformer, `oxygenvlm`), models/llm/oxygen.h (`oxygenvlm_text`), processors/glm4v_*; checked
against HuggingFace's Glm4vForConditionalGeneration.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..parallel.state import single
from .families import Glm4CausalLM
from .layers import Module
from .qwen import DenseCausalLM
from .qwen_vl import Qwen2VLForConditionalGeneration, _linear, _rms, _rot_half
from .registry import register_model


class Glm4vVisionTower(Module):
    def __init__(self, vc: dict, dtype, device):
        super().__init__()
        self.dim = int(vc.get("hidden_size", 1536))
        self.out = int(vc.get("out_hidden_size", 4096))
        self.heads = int(vc.get("num_heads", 12))
        self.patch = int(vc.get("patch_size", 14))
        self.merge = int(vc.get("spatial_merge_size", 2))
        self.tp = int(vc.get("temporal_patch_size", 2))
        self.eps = float(vc.get("rms_norm_eps", 1e-5))
        self.act = vc.get("hidden_act", "silu")
        self.bias = bool(vc.get("attention_bias", False))
        inter = int(vc.get("intermediate_size", 13696))
        depth = int(vc.get("depth", 24))
        in_ch = int(vc.get("in_channels", vc.get("in_chans", 3)))
        side = int(vc.get("image_size", 336)) // self.patch
        self.depth = depth
        mk = lambda *s: torch.zeros(*s, dtype=dtype, device=device)
        D, O, m = self.dim, self.out, self.merge
        flat = lambda name, shape: {name: lambda w, n=name, sh=shape: self._params[n].copy_(w.reshape(sh).to(dtype))}
        # Conv3d / Conv2d with kernel = stride are linear maps of the (flattened) patch
        self.add_param("patch_embed.proj.weight", mk(D, in_ch * self.tp * self.patch * self.patch),
                       flat("patch_embed.proj.weight", (D, -1)))
        self.add_param("patch_embed.proj.bias", mk(D))
        self.add_param("post_conv_layernorm.weight", mk(D))
        self.add_param("embeddings.position_embedding.weight", mk(side * side, D))
        for i in range(depth):
            b = f"blocks.{i}."
            self.add_param(b + "norm1.weight", mk(D))
            self.add_param(b + "norm2.weight", mk(D))
            self.add_param(b + "attn.qkv.weight", mk(3 * D, D))
            if self.bias:
                self.add_param(b + "attn.qkv.bias", mk(3 * D))
            self.add_param(b + "attn.proj.weight", mk(D, D))
            self.add_param(b + "mlp.gate_proj.weight", mk(O, D))
            self.add_param(b + "mlp.up_proj.weight", mk(O, D))
            self.add_param(b + "mlp.down_proj.weight", mk(D, O))
        self.add_param("post_layernorm.weight", mk(D))
        self.add_param("downsample.weight", mk(O, D * m * m), flat("downsample.weight", (O, -1)))
        self.add_param("downsample.bias", mk(O))
        self.add_param("merger.proj.weight", mk(O, O))
        self.add_param("merger.post_projection_norm.weight", mk(O))
        self.add_param("merger.post_projection_norm.bias", mk(O))
        self.add_param("merger.gate_proj.weight", mk(inter, O))
        self.add_param("merger.up_proj.weight", mk(inter, O))
        self.add_param("merger.down_proj.weight", mk(O, inter))

    def _coords(self, grid_thw, device):
        """Row / column of every patch, in the merge-window order the processor emits patches in."""
        m, hs, ws = self.merge, [], []
        for t, h, w in grid_thw.tolist():
            hp = torch.arange(h, device=device).view(h, 1).expand(h, w)
            wp = torch.arange(w, device=device).view(1, w).expand(h, w)
            order = lambda z: z.reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            hs.append(order(hp).repeat(t))
            ws.append(order(wp).repeat(t))
        return torch.cat(hs), torch.cat(ws)

    def _position_embedding(self, grid_thw, hc, wc, device):
        """The learned side x side table sampled bicubically at every patch centre of an h x w grid."""
        p = self._params["embeddings.position_embedding.weight"]
        side = int(round(p.shape[0] ** 0.5))
        table = p.view(side, side, -1).permute(2, 0, 1)[None].float()
        th = torch.cat([torch.full((int(t * h * w),), float(h)) for t, h, w in grid_thw.tolist()]).to(device)
        tw = torch.cat([torch.full((int(t * h * w),), float(w)) for t, h, w in grid_thw.tolist()]).to(device)
        grid = torch.stack([(wc.float() + 0.5) / tw * 2 - 1, (hc.float() + 0.5) / th * 2 - 1], dim=-1)[None, :, None, :]
        out = F.grid_sample(table, grid, mode="bicubic", align_corners=False, padding_mode="border")
        return out[0, :, :, 0].T.to(p.dtype)

    def forward(self, pixel_values, grid_thw):
        """pixel_values [N_patches, C*tp*p*p] -> image token embeddings [N_patches / merge^2, out_hidden]."""
        p = self._params
        dt = p["patch_embed.proj.weight"].dtype
        x = _linear(pixel_values.to(dt), p["patch_embed.proj.weight"], p["patch_embed.proj.bias"])
        x = _rms(x, p["post_conv_layernorm.weight"], self.eps)
        hc, wc = self._coords(grid_thw, x.device)
        hd = self.dim // self.heads
        inv = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float32, device=x.device) / (hd // 2)))
        ang = torch.cat([hc.float()[:, None] * inv[None], wc.float()[:, None] * inv[None]], dim=-1)      # [N, hd/2]
        emb = torch.cat([ang, ang], dim=-1)
        cos, sin = emb.cos()[:, None, :], emb.sin()[:, None, :]
        x = x + self._position_embedding(grid_thw, hc, wc, x.device)
        cu = [0]
        for t, h, w in grid_thw.tolist():
            for _ in range(int(t)):                                     # attention stays inside a frame
                cu.append(cu[-1] + int(h * w))
        T, D = x.shape
        act = F.silu if self.act == "silu" else F.gelu
        for i in range(self.depth):
            b = f"blocks.{i}."
            h_ = _rms(x, p[b + "norm1.weight"], self.eps)
            q, k, v = _linear(h_, p[b + "attn.qkv.weight"], p.get(b + "attn.qkv.bias")).view(T, 3, self.heads, hd).unbind(1)
            qf, kf = q.float(), k.float()
            q = (qf * cos + _rot_half(qf) * sin).to(x.dtype)
            k = (kf * cos + _rot_half(kf) * sin).to(x.dtype)
            outs = []
            for a, e in zip(cu[:-1], cu[1:]):
                o = F.scaled_dot_product_attention(q[a:e].transpose(0, 1)[None], k[a:e].transpose(0, 1)[None],
                                                   v[a:e].transpose(0, 1)[None])[0]
                outs.append(o.transpose(0, 1).reshape(e - a, D))
            x = x + _linear(torch.cat(outs), p[b + "attn.proj.weight"])
            h_ = _rms(x, p[b + "norm2.weight"], self.eps)
            x = x + _linear(act(_linear(h_, p[b + "mlp.gate_proj.weight"])) * _linear(h_, p[b + "mlp.up_proj.weight"]),
                             p[b + "mlp.down_proj.weight"])
        x = _rms(x, p["post_layernorm.weight"], self.eps)
        m = self.merge
        # each group of m*m consecutive patches is one window [m, m, D]; the convolution sees it as [D, m, m]
        x = x.view(-1, m, m, D).permute(0, 3, 1, 2).reshape(-1, D * m * m)
        x = _linear(x, p["downsample.weight"], p["downsample.bias"])
        y = _linear(x, p["merger.proj.weight"])
        y = F.gelu(F.layer_norm(y, (self.out,), p["merger.post_projection_norm.weight"], p["merger.post_projection_norm.bias"], 1e-5))
        return _linear(act(_linear(y, p["merger.gate_proj.weight"])) * _linear(y, p["merger.up_proj.weight"]),
                        p["merger.down_proj.weight"])

    __call__ = forward


def _sections(args):
    half = args.rotary_dim // 2
    return list(args.mrope_section) or [half - 2 * (half * 3 // 8), half * 3 // 8, half * 3 // 8]


class Glm4vForConditionalGeneration(Glm4CausalLM):
    """GLM-4 decoder + the tower; rotary sections are contiguous ([8, 12, 12] pairs of the rotated half)."""

    def __init__(self, args, dtype=torch.bfloat16, device="cpu", ps=None):
        super().__init__(args, dtype, device, ps or single())
        self.visual = self.add_module("visual", Glm4vVisionTower(args.vision_config or {}, dtype, device))
        self.mrope_section = _sections(args)

    encode_images = Qwen2VLForConditionalGeneration.encode_images

    @staticmethod
    def remap_weight(name, w):
        if name.startswith("model.visual."):
            name = name[len("model."):]
        elif name.startswith("model.language_model."):
            name = "model." + name[len("model.language_model."):]
        return Glm4CausalLM.remap_weight(name, w)


@register_model("glm4v", "Glm4vForConditionalGeneration")
def build_glm4v(args, dtype, device, ps):
    return Glm4vForConditionalGeneration(args, dtype, device, ps)


class OxygenVLForConditionalGeneration(DenseCausalLM):
    """The reference's `oxygenvlm`: the same tower in front of a Qwen3 decoder with 3-axis rotary positions."""

    def __init__(self, args, dtype=torch.bfloat16, device="cpu", ps=None):
        super().__init__(args, dtype, device, ps or single())
        self.visual = self.add_module("visual", Glm4vVisionTower(args.vision_config or {}, dtype, device))
        self.mrope_section = _sections(args)

    encode_images = Qwen2VLForConditionalGeneration.encode_images
    remap_weight = staticmethod(Qwen2VLForConditionalGeneration.remap_weight)


@register_model("oxygenvlm", "OxygenvlmForConditionalGeneration")
def build_oxygenvlm(args, dtype, device, ps):
    return OxygenVLForConditionalGeneration(args, dtype, device, ps)


@register_model("oxygenvlm_text")
def build_oxygenvlm_text(args, dtype, device, ps):
    """The decoder alone (xllm/models/llm/oxygen.h): Qwen3 that accepts 3-axis positions and deep-stack
    features through the engine's embedding inputs."""
    m = DenseCausalLM(args, dtype, device, ps or single())
    m.mrope_section = _sections(args)
    return m
