"""Image preprocessing for Qwen2-VL-style models and the bookkeeping that ties image tokens to a
prompt.

Parity: the image processors and prompt/position builders of xllm/processors/* (Qwen2-VL /
Qwen2.5-VL: `smart_resize`, normalise, patchify with temporal duplication, `get_rope_index`) and
`MMData / MMInput` (xllm/core/framework/multimodal/*).  Decoding of PNG/JPEG goes through Pillow;
everything after that is torch on the CPU.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280):
    """Round both sides to multiples of `factor` keeping the aspect ratio and the pixel budget."""
    if max(height, width) / min(height, width) > 200:
        raise ValueError("aspect ratio above 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def _to_chw_float(img) -> torch.Tensor:
    """PIL image, HWC uint8 array or CHW float tensor -> CHW float32 in [0, 1]."""
    if isinstance(img, torch.Tensor):
        t = img.float()
        return t / 255.0 if t.max() > 1.5 else t
    if isinstance(img, np.ndarray):
        return torch.from_numpy(img).permute(2, 0, 1).float() / 255.0
    arr = np.asarray(img.convert("RGB"))
    return torch.from_numpy(arr.copy()).permute(2, 0, 1).float() / 255.0


class Qwen2VLImageProcessor:
    def __init__(self, patch_size=14, merge_size=2, temporal_patch_size=2, min_pixels=56 * 56,
                 max_pixels=14 * 14 * 4 * 1280, mean=CLIP_MEAN, std=CLIP_STD):
        self.p, self.m, self.tp = patch_size, merge_size, temporal_patch_size
        self.min_pixels, self.max_pixels = min_pixels, max_pixels
        self.mean = torch.tensor(mean).view(3, 1, 1)
        self.std = torch.tensor(std).view(3, 1, 1)

    def one(self, img) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
        x = _to_chw_float(img)
        C, H, W = x.shape
        h, w = smart_resize(H, W, self.p * self.m, self.min_pixels, self.max_pixels)
        if (h, w) != (H, W):
            x = torch.nn.functional.interpolate(x[None], size=(h, w), mode="bicubic", align_corners=False,
                                                antialias=True)[0].clamp(0, 1)
        x = (x - self.mean) / self.std
        frames = x[None].repeat(self.tp, 1, 1, 1)                       # a still image fills the temporal patch
        gh, gw, p, m = h // self.p, w // self.p, self.p, self.m
        # [T, C, gh/m, m, p, gw/m, m, p] -> patches ordered so that each m x m window is contiguous
        y = frames.view(1, self.tp, C, gh // m, m, p, gw // m, m, p)
        y = y.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(gh * gw, C * self.tp * p * p)
        return y, (1, gh, gw)

    def __call__(self, images: Sequence):
        outs = [self.one(im) for im in images]
        pixel_values = torch.cat([o[0] for o in outs]) if outs else torch.zeros(0, 3 * self.tp * self.p * self.p)
        grid = torch.tensor([o[1] for o in outs], dtype=torch.int64).view(-1, 3)
        return pixel_values, grid

    def tokens_per_image(self, grid_thw) -> List[int]:
        return [int(t * h * w) // (self.m * self.m) for t, h, w in grid_thw.tolist()]


def expand_image_tokens(token_ids: Sequence[int], image_pad_id: int, counts: Sequence[int]) -> List[int]:
    """Every single `image_pad_id` in the prompt stands for one image: repeat it `counts[i]` times."""
    out, i = [], 0
    for t in token_ids:
        if t == image_pad_id:
            if i >= len(counts):
                raise ValueError("more image placeholders than images")
            out.extend([image_pad_id] * counts[i])
            i += 1
        else:
            out.append(int(t))
    if i != len(counts):
        raise ValueError("more images than image placeholders")
    return out


def mrope_positions(token_ids: Sequence[int], image_pad_id: int, grid_thw, merge_size: int = 2):
    """3-D rotary position ids (temporal, height, width) of an expanded prompt; text tokens advance
    all three together, the tokens of an image share a temporal position and carry their row / column.
    Returns (positions [3, L] int64, delta) where a decoded token at sequence index i sits at
    position i + delta on all three axes."""
    L = len(token_ids)
    pos = torch.zeros(3, L, dtype=torch.int64)
    nxt, i, img = 0, 0, 0
    grid = grid_thw.tolist() if hasattr(grid_thw, "tolist") else list(grid_thw)
    while i < L:
        if token_ids[i] == image_pad_id:
            t, h, w = grid[img]
            gh, gw = h // merge_size, w // merge_size
            n = t * gh * gw
            tt = torch.arange(t).view(t, 1, 1).expand(t, gh, gw).reshape(-1)
            hh = torch.arange(gh).view(1, gh, 1).expand(t, gh, gw).reshape(-1)
            ww = torch.arange(gw).view(1, 1, gw).expand(t, gh, gw).reshape(-1)
            pos[:, i:i + n] = torch.stack([tt, hh, ww]) + nxt
            nxt = int(pos[:, i:i + n].max()) + 1
            i += n
            img += 1
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    return pos, nxt - L


@dataclass
class MMInput:
    """What a multimodal request carries next to its (expanded) token ids."""
    embeds: torch.Tensor                       # [n_mm_tokens, hidden] output of the vision tower
    positions: List[int] = field(default_factory=list)   # prompt indices of the placeholder tokens, ascending
    mrope: Optional[torch.Tensor] = None       # [3, L] position ids of the prompt
    delta: int = 0
    hash_key: int = 0                          # discriminator for the prefix cache (content hash of the images)


def mrope_table(pos3: torch.Tensor, rot_dim: int, theta: float, sections: Sequence[int],
                interleaved: bool = False) -> torch.Tensor:
    """cos|sin rows [T, rot_dim] for 3-D positions pos3 [3, T]: frequency j uses the axis whose
    section contains j (sections count rotary pairs: sum = rot_dim / 2).  `interleaved` (Qwen3-VL)
    deals the axes out in turn instead, t h w t h w ..., the temporal axis keeping what is left."""
    half = rot_dim // 2
    assert sum(sections) == half
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64, device=pos3.device) * 2.0 / rot_dim))
    if interleaved:
        axis = torch.zeros(half, dtype=torch.long, device=pos3.device)
        for ax, off in ((1, 1), (2, 2)):
            axis[off:sections[ax] * 3:3] = ax
    else:
        axis = torch.repeat_interleave(torch.arange(3, device=pos3.device),
                                       torch.tensor(list(sections), device=pos3.device))
    p = pos3.to(torch.float64)[axis]                      # [half, T]
    ang = (p * inv[:, None]).T                            # [T, half]
    return torch.cat([ang.cos(), ang.sin()], dim=-1).float()
