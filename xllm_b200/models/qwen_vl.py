"""Qwen2-VL / Qwen2.5-VL: vision transformer + patch merger in front of the dense decoder, with
multimodal rotary position ids.

Parity: xllm/models/vlm/qwen2_vl.h, qwen2_5_vl.h (vision blocks, `Qwen2VisionPatchMerger`, merging
of image embeddings into the input embeddings, M-RoPE sections).  The language model is the shared
`DenseCausalLM`: image tokens enter through its `embeds` override, and the 3-axis rotary positions
through a per-row cos|sin table in the attention metadata, so the fused rope/KV-write kernel and the
paged attention kernels run unchanged.  The vision tower runs once per image at admission; it uses
torch's attention (one call per image, full attention inside an image).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .layers import Module
from .qwen import DenseCausalLM
from .registry import register_model
from ..parallel.state import single


def _linear(x, w, b=None):
    """Linear layer of a vision tower: the tcgen05 GEMM (with its bias epilogue) for bf16 on the device, the tensor
    library otherwise (shapes the kernel cannot take are counted as fallbacks by ops/gemm.py)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        from ..ops import gemm
        return gemm.linear(x.reshape(-1, x.shape[-1]), w, b).view(*x.shape[:-1], w.shape[0])
    return F.linear(x, w, b)


def _rot_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat([-x2, x1], dim=-1)


def _rms(x, w, eps=1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class VisionBlock(Module):
    """`gated` selects the Qwen2.5-VL block: RMSNorm without bias and a SwiGLU MLP (gate/up/down with
    biases) instead of LayerNorm and fc1 / quick-GELU / fc2."""

    def __init__(self, dim, heads, mlp_dim, dtype, device, act="quick_gelu", gated=False):
        super().__init__()
        self.heads, self.act, self.gated = heads, act, gated
        mk = lambda *s: torch.zeros(*s, dtype=dtype, device=device)
        shapes = [("norm1.weight", (dim,)), ("norm2.weight", (dim,)),
                  ("attn.qkv.weight", (3 * dim, dim)), ("attn.qkv.bias", (3 * dim,)),
                  ("attn.proj.weight", (dim, dim)), ("attn.proj.bias", (dim,))]
        if gated:
            shapes += [("mlp.gate_proj.weight", (mlp_dim, dim)), ("mlp.gate_proj.bias", (mlp_dim,)),
                       ("mlp.up_proj.weight", (mlp_dim, dim)), ("mlp.up_proj.bias", (mlp_dim,)),
                       ("mlp.down_proj.weight", (dim, mlp_dim)), ("mlp.down_proj.bias", (dim,))]
        else:
            shapes += [("norm1.bias", (dim,)), ("norm2.bias", (dim,)),
                       ("mlp.fc1.weight", (mlp_dim, dim)), ("mlp.fc1.bias", (mlp_dim,)),
                       ("mlp.fc2.weight", (dim, mlp_dim)), ("mlp.fc2.bias", (dim,))]
        for name, shape in shapes:
            self.add_param(name, mk(*shape))
        self.p = self._params

    def forward(self, x, cos, sin, cu):
        p = self.p
        if self.gated:
            h = _rms(x, p["norm1.weight"])
        else:
            h = F.layer_norm(x, x.shape[-1:], p["norm1.weight"], p["norm1.bias"], 1e-6)
        T, D = h.shape
        q, k, v = _linear(h, p["attn.qkv.weight"], p["attn.qkv.bias"]).view(T, 3, self.heads, D // self.heads).unbind(1)
        q = q * cos + _rot_half(q) * sin
        k = k * cos + _rot_half(k) * sin
        outs = []
        for a, b in zip(cu[:-1], cu[1:]):          # full attention inside each image
            o = F.scaled_dot_product_attention(q[a:b].transpose(0, 1)[None], k[a:b].transpose(0, 1)[None],
                                               v[a:b].transpose(0, 1)[None])[0]
            outs.append(o.transpose(0, 1).reshape(b - a, D))
        x = x + _linear(torch.cat(outs), p["attn.proj.weight"], p["attn.proj.bias"])
        if self.gated:
            h = _rms(x, p["norm2.weight"])
            g = F.silu(_linear(h, p["mlp.gate_proj.weight"], p["mlp.gate_proj.bias"]))
            u = _linear(h, p["mlp.up_proj.weight"], p["mlp.up_proj.bias"])
            return x + _linear(g * u, p["mlp.down_proj.weight"], p["mlp.down_proj.bias"])
        h = F.layer_norm(x, x.shape[-1:], p["norm2.weight"], p["norm2.bias"], 1e-6)
        h = _linear(h, p["mlp.fc1.weight"], p["mlp.fc1.bias"])
        h = h * torch.sigmoid(1.702 * h) if self.act == "quick_gelu" else F.gelu(h)
        return x + _linear(h, p["mlp.fc2.weight"], p["mlp.fc2.bias"])

    __call__ = forward


class VisionTower(Module):
    def __init__(self, vc: dict, out_hidden: int, dtype, device):
        super().__init__()
        # Qwen2.5-VL: gated blocks, windowed attention except in `fullatt_block_indexes`, `hidden_size` is the
        # tower width and `out_hidden_size` the decoder width (Qwen2-VL: `embed_dim` and `hidden_size`)
        self.v25 = "fullatt_block_indexes" in vc or "out_hidden_size" in vc
        self.dim = vc.get("hidden_size", 1280) if self.v25 else vc.get("embed_dim", vc.get("hidden_size", 1280))
        self.full_blocks = set(vc.get("fullatt_block_indexes") or [])
        self.window = int(vc.get("window_size", 112))
        self.heads = vc.get("num_heads", 16)
        self.patch = vc.get("patch_size", 14)
        self.merge = vc.get("spatial_merge_size", 2)
        self.tp = vc.get("temporal_patch_size", 2)
        in_ch = vc.get("in_chans", vc.get("in_channels", 3))
        depth = vc.get("depth", 32)
        mlp_dim = int(vc["intermediate_size"]) if self.v25 else int(self.dim * vc.get("mlp_ratio", 4))
        mk = lambda *s: torch.zeros(*s, dtype=dtype, device=device)
        # Conv3d(kernel = stride = patch) over non-overlapping patches is a linear map of the patch
        self.add_param("patch_embed.proj.weight", mk(self.dim, in_ch * self.tp * self.patch * self.patch),
                       {"patch_embed.proj.weight": lambda w, t=None: self._params["patch_embed.proj.weight"].copy_(
                           w.reshape(self.dim, -1).to(dtype))})
        blocks = Module()
        self.add_module("blocks", blocks)
        self.blocks = [blocks.add_module(str(i), VisionBlock(self.dim, self.heads, mlp_dim, dtype, device,
                                                             vc.get("hidden_act", "quick_gelu"), gated=self.v25))
                       for i in range(depth)]
        m2 = self.merge * self.merge
        for name, shape in (("merger.ln_q.weight", (self.dim,)),) + ((() if self.v25 else (("merger.ln_q.bias", (self.dim,)),)) + (
                            ("merger.mlp.0.weight", (self.dim * m2, self.dim * m2)), ("merger.mlp.0.bias", (self.dim * m2,)),
                            ("merger.mlp.2.weight", (out_hidden, self.dim * m2)), ("merger.mlp.2.bias", (out_hidden,)))):
            self.add_param(name, mk(*shape))

    def window_index(self, grid_thw):
        """Order of the merged units grouped by attention window, and the window boundaries in
        patches (Qwen2.5-VL): windows of `window_size` pixels tile each frame, ragged at the edges."""
        m = self.merge
        ws = max(1, self.window // m // self.patch)
        order, cu, base = [], [0], 0
        for t, h, w in grid_thw.tolist():
            gh, gw = h // m, w // m
            idx = torch.arange(t * gh * gw).reshape(t, gh, gw)
            ph, pw = ws - gh % ws, ws - gw % ws
            nh, nw = (gh + ph) // ws, (gw + pw) // ws
            pad = F.pad(idx, (0, pw, 0, ph), value=-100).reshape(t, nh, ws, nw, ws).permute(0, 1, 3, 2, 4)
            pad = pad.reshape(t, nh * nw, ws, ws)
            lens = (pad != -100).sum([2, 3]).reshape(-1)
            flat = pad.reshape(-1)
            order.append(flat[flat != -100] + base)
            for n in lens.tolist():
                if n:
                    cu.append(cu[-1] + n * m * m)
            base += t * gh * gw
        return torch.cat(order), cu

    def rot_pos_emb(self, grid_thw, device):
        """2-D rotary angles per patch, in the merge-window order the processor emits patches in."""
        hd = self.dim // self.heads
        inv = 1.0 / (10000.0 ** (torch.arange(0, hd // 2, 2, dtype=torch.float32, device=device) / (hd // 2)))
        out = []
        m = self.merge
        for t, h, w in grid_thw.tolist():
            hp = torch.arange(h, device=device).view(h, 1).expand(h, w)
            wp = torch.arange(w, device=device).view(1, w).expand(h, w)
            order = lambda z: z.reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            ids = torch.stack([order(hp), order(wp)], dim=-1).repeat(t, 1).float()       # [t*h*w, 2]
            ang = (ids[:, :, None] * inv[None, None, :]).reshape(ids.shape[0], -1)        # [N, hd/2]
            out.append(ang)
        ang = torch.cat(out)
        emb = torch.cat([ang, ang], dim=-1)                                             # [N, hd]
        return emb.cos()[:, None, :], emb.sin()[:, None, :]

    def forward(self, pixel_values, grid_thw):
        """pixel_values [N_patches, C*tp*p*p] -> image token embeddings [N_patches / merge^2, hidden]."""
        p = self._params
        x = _linear(pixel_values.to(p["patch_embed.proj.weight"].dtype), p["patch_embed.proj.weight"])
        cos, sin = self.rot_pos_emb(grid_thw, x.device)
        cos, sin = cos.to(x.dtype), sin.to(x.dtype)
        sizes = [int(t * h * w) for t, h, w in grid_thw.tolist()]
        cu = [0]
        for s in sizes:
            cu.append(cu[-1] + s)
        m2 = self.merge * self.merge
        if self.v25:
            order, cu_win = self.window_index(grid_thw)
            order = order.to(x.device)
            regroup = lambda z: z.reshape(z.shape[0] // m2, m2, *z.shape[1:])[order].reshape(z.shape)
            x, cos, sin = regroup(x), regroup(cos), regroup(sin)
            for i, blk in enumerate(self.blocks):
                x = blk(x, cos, sin, cu if i in self.full_blocks else cu_win)
            x = _rms(x, p["merger.ln_q.weight"])
        else:
            for blk in self.blocks:
                x = blk(x, cos, sin, cu)
            x = F.layer_norm(x, x.shape[-1:], p["merger.ln_q.weight"], p["merger.ln_q.bias"], 1e-6)
        x = x.view(-1, self.dim * m2)
        x = F.gelu(_linear(x, p["merger.mlp.0.weight"], p["merger.mlp.0.bias"]))
        x = _linear(x, p["merger.mlp.2.weight"], p["merger.mlp.2.bias"])
        return x[torch.argsort(order)] if self.v25 else x

    __call__ = forward


class Qwen2VLForConditionalGeneration(DenseCausalLM):
    def __init__(self, args, dtype=torch.bfloat16, device="cpu", ps=None):
        super().__init__(args, dtype, device, ps or single())
        self.visual = self.add_module("visual", VisionTower(args.vision_config or {}, args.hidden_size, dtype, device))
        half = args.rotary_dim // 2
        self.mrope_section = list(args.mrope_section) or [half - 2 * (half * 3 // 8), half * 3 // 8, half * 3 // 8]

    def encode_images(self, pixel_values, grid_thw):
        return self.visual(pixel_values.to(self.device), grid_thw)

    @staticmethod
    def remap_weight(name, w):
        # checkpoints name the tower `visual.*` or `model.visual.*`, the decoder `model.layers.*` or
        # `model.language_model.layers.*`, depending on the library version that wrote them
        if name.startswith("model.visual."):
            name = name[len("model."):]
        elif name.startswith("model.language_model."):
            name = "model." + name[len("model.language_model."):]
        return [(name, w)]


@register_model("qwen2_vl", "qwen2_5_vl", "Qwen2VLForConditionalGeneration", "Qwen2_5_VLForConditionalGeneration")
def build_qwen2_vl(args, dtype, device, ps):
    return Qwen2VLForConditionalGeneration(args, dtype, device, ps)


# ----------------------------------------------------------------------------------------- Qwen3-VL
class VisionTowerV3(Module):
    """Qwen3-VL tower: LayerNorm blocks with a tanh-GELU MLP, a learned position table interpolated
    bilinearly to the image grid, 2-D rotary attention inside each frame, a merger, and "deepstack"
    mergers that read the states after chosen blocks; their outputs are added to the decoder's
    hidden states at the image rows after its first layers.  forward returns
    [N / merge^2, out * (1 + n_deepstack)]: the image embeddings followed by the deepstack features."""

    def __init__(self, vc: dict, dtype, device):
        super().__init__()
        self.dim, self.heads = vc["hidden_size"], vc["num_heads"]
        self.out = vc["out_hidden_size"]
        self.patch, self.merge, self.tp = vc.get("patch_size", 16), vc.get("spatial_merge_size", 2), vc.get("temporal_patch_size", 2)
        self.deep_idx = list(vc.get("deepstack_visual_indexes") or [])
        self.side = int(round(vc.get("num_position_embeddings", 2304) ** 0.5))
        self.act = vc.get("hidden_act", "gelu_pytorch_tanh")
        in_ch, inter, m2 = vc.get("in_channels", 3), vc["intermediate_size"], self.merge ** 2
        mk = lambda *s: torch.zeros(*s, dtype=dtype, device=device)
        D = self.dim
        shapes = [("patch_embed.proj.bias", (D,)), ("pos_embed.weight", (self.side ** 2, D))]
        for i in range(vc["depth"]):
            b = f"blocks.{i}."
            shapes += [(b + "norm1.weight", (D,)), (b + "norm1.bias", (D,)), (b + "norm2.weight", (D,)), (b + "norm2.bias", (D,)),
                       (b + "attn.qkv.weight", (3 * D, D)), (b + "attn.qkv.bias", (3 * D,)),
                       (b + "attn.proj.weight", (D, D)), (b + "attn.proj.bias", (D,)),
                       (b + "mlp.linear_fc1.weight", (inter, D)), (b + "mlp.linear_fc1.bias", (inter,)),
                       (b + "mlp.linear_fc2.weight", (D, inter)), (b + "mlp.linear_fc2.bias", (D,))]
        for pre, nd in [("merger.", D)] + [(f"deepstack_merger_list.{k}.", D * m2) for k in range(len(self.deep_idx))]:
            shapes += [(pre + "norm.weight", (nd,)), (pre + "norm.bias", (nd,)),
                       (pre + "linear_fc1.weight", (D * m2, D * m2)), (pre + "linear_fc1.bias", (D * m2,)),
                       (pre + "linear_fc2.weight", (self.out, D * m2)), (pre + "linear_fc2.bias", (self.out,))]
        self.depth = vc["depth"]
        w = mk(D, in_ch * self.tp * self.patch * self.patch)
        self.add_param("patch_embed.proj.weight", w, {"patch_embed.proj.weight": lambda x, t=w: t.copy_(x.reshape(t.shape).to(t.dtype))})
        for name, shape in shapes:
            self.add_param(name, mk(*shape))

    def _pos_embed(self, grid_thw, device):
        p, m, n = self._params["pos_embed.weight"], self.merge, self.side
        outs = []
        for t, h, w in grid_thw.tolist():
            hi, wi = torch.linspace(0, n - 1, h), torch.linspace(0, n - 1, w)
            h0, w0 = hi.int(), wi.int()
            h1, w1 = (h0 + 1).clip(max=n - 1), (w0 + 1).clip(max=n - 1)
            dh, dw = (hi - h0)[:, None], (wi - w0)[None, :]
            emb = 0
            for hh, ww, wt in ((h0, w0, (1 - dh) * (1 - dw)), (h0, w1, (1 - dh) * dw), (h1, w0, dh * (1 - dw)), (h1, w1, dh * dw)):
                idx = (hh.long()[:, None] * n + ww.long()[None, :]).flatten().to(device)
                emb = emb + p[idx] * wt.flatten().to(device=device, dtype=p.dtype)[:, None]
            emb = emb.repeat(t, 1).view(t, h // m, m, w // m, m, -1).permute(0, 1, 3, 2, 4, 5).flatten(0, 4)
            outs.append(emb)
        return torch.cat(outs)

    def _merge(self, pre, x, post_norm):
        p, D, m2 = self._params, self.dim, self.merge ** 2
        if post_norm:
            x = F.layer_norm(x.view(-1, D * m2), (D * m2,), p[pre + "norm.weight"], p[pre + "norm.bias"], 1e-6)
        else:
            x = F.layer_norm(x, (D,), p[pre + "norm.weight"], p[pre + "norm.bias"], 1e-6).view(-1, D * m2)
        x = F.gelu(_linear(x, p[pre + "linear_fc1.weight"], p[pre + "linear_fc1.bias"]))
        return _linear(x, p[pre + "linear_fc2.weight"], p[pre + "linear_fc2.bias"])

    rot_pos_emb = VisionTower.rot_pos_emb

    def forward(self, pixel_values, grid_thw):
        p, D = self._params, self.dim
        x = _linear(pixel_values.to(p["patch_embed.proj.weight"].dtype), p["patch_embed.proj.weight"], p["patch_embed.proj.bias"])
        x = x + self._pos_embed(grid_thw, x.device)
        cos, sin = self.rot_pos_emb(grid_thw, x.device)
        cos, sin = cos.to(x.dtype), sin.to(x.dtype)
        cu = [0]
        for t, h, w in grid_thw.tolist():                  # attention stays inside a frame
            for _ in range(t):
                cu.append(cu[-1] + h * w)
        deep = []
        for i in range(self.depth):
            b = f"blocks.{i}."
            h_ = F.layer_norm(x, (D,), p[b + "norm1.weight"], p[b + "norm1.bias"], 1e-6)
            T = h_.shape[0]
            q, k, v = _linear(h_, p[b + "attn.qkv.weight"], p[b + "attn.qkv.bias"]).view(T, 3, self.heads, D // self.heads).unbind(1)
            q = q * cos + _rot_half(q) * sin
            k = k * cos + _rot_half(k) * sin
            outs = []
            for a0, b0 in zip(cu[:-1], cu[1:]):
                o = F.scaled_dot_product_attention(q[a0:b0].transpose(0, 1)[None], k[a0:b0].transpose(0, 1)[None],
                                                   v[a0:b0].transpose(0, 1)[None])[0]
                outs.append(o.transpose(0, 1).reshape(b0 - a0, D))
            x = x + _linear(torch.cat(outs), p[b + "attn.proj.weight"], p[b + "attn.proj.bias"])
            h_ = F.layer_norm(x, (D,), p[b + "norm2.weight"], p[b + "norm2.bias"], 1e-6)
            h_ = F.gelu(_linear(h_, p[b + "mlp.linear_fc1.weight"], p[b + "mlp.linear_fc1.bias"]),
                        approximate="tanh" if "tanh" in self.act else "none")
            x = x + _linear(h_, p[b + "mlp.linear_fc2.weight"], p[b + "mlp.linear_fc2.bias"])
            if i in self.deep_idx:
                deep.append(self._merge(f"deepstack_merger_list.{self.deep_idx.index(i)}.", x, True))
        return torch.cat([self._merge("merger.", x, False)] + deep, dim=-1)

    __call__ = forward


class Qwen3VLForConditionalGeneration(Qwen2VLForConditionalGeneration):
    mrope_interleaved = True

    def __init__(self, args, dtype=torch.bfloat16, device="cpu", ps=None):
        DenseCausalLM.__init__(self, args, dtype, device, ps or single())
        self.visual = self.add_module("visual", VisionTowerV3(args.vision_config or {}, dtype, device))
        half = args.rotary_dim // 2
        self.mrope_section = list(args.mrope_section) or [half - 2 * (half * 3 // 8), half * 3 // 8, half * 3 // 8]


@register_model("qwen3_vl", "Qwen3VLForConditionalGeneration")
def build_qwen3_vl(args, dtype, device, ps):
    return Qwen3VLForConditionalGeneration(args, dtype, device, ps)


class Qwen3VLMoeForConditionalGeneration(Qwen3VLForConditionalGeneration):
    """Qwen3-VL with the Qwen3-MoE decoder.  Its checkpoints keep the experts of a layer in two fused
    tensors, `experts.gate_up_proj` [E, 2I, H] (or [E, H, 2I] in the original release) and
    `experts.down_proj` [E, H, I] (or [E, I, H]); they are split into per-expert tensors on load."""

    def __init__(self, args, dtype=torch.bfloat16, device="cpu", ps=None):
        from .qwen_moe import _make_mlp
        DenseCausalLM.__init__(self, args, dtype, device, ps or single(), make_mlp=_make_mlp(args, dtype, device, ps or single()))
        self.visual = self.add_module("visual", VisionTowerV3(args.vision_config or {}, dtype, device))
        half = args.rotary_dim // 2
        self.mrope_section = list(args.mrope_section) or [half - 2 * (half * 3 // 8), half * 3 // 8, half * 3 // 8]

    def remap_weight(self, name, w):
        out = []
        for n, t in Qwen2VLForConditionalGeneration.remap_weight(name, w):
            H, I = self.args.hidden_size, self.args.moe_intermediate_size
            if n.endswith(".mlp.experts.gate_up_proj"):
                base = n[: -len("gate_up_proj")]
                if t.shape[1] != 2 * I:
                    t = t.transpose(1, 2)                  # [E, H, 2I] -> [E, 2I, H]
                for e in range(t.shape[0]):
                    out += [(f"{base}{e}.gate_proj.weight", t[e, :I]), (f"{base}{e}.up_proj.weight", t[e, I:])]
            elif n.endswith(".mlp.experts.down_proj"):
                base = n[: -len("down_proj")]
                if t.shape[1] != H:
                    t = t.transpose(1, 2)                  # [E, I, H] -> [E, H, I]
                for e in range(t.shape[0]):
                    out.append((f"{base}{e}.down_proj.weight", t[e]))
            else:
                out.append((n, t))
        return out


@register_model("qwen3_vl_moe", "Qwen3VLMoeForConditionalGeneration")
def build_qwen3_vl_moe(args, dtype, device, ps):
    return Qwen3VLMoeForConditionalGeneration(args, dtype, device, ps)
