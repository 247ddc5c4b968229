"""Text-to-image pipeline behind `/v1/images/generations`.

Parity: the reference's DiT master / engine / worker and image generation service
(xllm/core/distributed_runtime/dit_master.cpp, api_service image generation handlers): a request
carries a prompt, a size, a step count and a seed; the worker runs the denoising loop of a diffusion
transformer (with a step cache: FBCache / TaylorSeer / residual) and a decoder turns the latent into
pixels; the response carries base64 images.

The denoiser here is the compact DiT of `dit/model.py` (random weights unless a state dict is
given) and the "VAE" a fixed linear map from 4 latent channels to RGB with nearest-neighbour
upsampling: the route, the request / response format, the sampling loop and the step caches are the
product; Flux / Qwen-Image / Wan checkpoints (text encoders, VAEs, 3-D rope) are not supported.
"""
from __future__ import annotations

import base64
import hashlib
import struct
import time
import zlib
from typing import List, Optional

import numpy as np
import torch

from .cache import make_cache
from .model import TinyDiT


def encode_png(img: np.ndarray) -> bytes:
    """Minimal PNG writer for an [H, W, 3] uint8 array (no external imaging library)."""
    h, w, c = img.shape
    assert c == 3 and img.dtype == np.uint8
    raw = b"".join(b"\x00" + img[y].tobytes() for y in range(h))

    def chunk(tag, data):
        return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)

    return (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0))
            + chunk(b"IDAT", zlib.compress(raw, 6)) + chunk(b"IEND", b""))


class ImagePipeline:
    def __init__(self, model: Optional[TinyDiT] = None, latent_size: int = 8, steps: int = 20, cache: str = "fbcache",
                 device: str = "cpu", seed: int = 0):
        torch.manual_seed(seed)
        self.model = (model or TinyDiT(size=latent_size)).to(device).eval()
        self.latent_size = self.model.size
        self.steps = steps
        self.cache_kind = cache
        self.device = device
        g = torch.Generator().manual_seed(seed + 1)
        self.to_rgb = torch.randn(3, self.model.in_ch, generator=g) * 0.5          # latent channels -> RGB

    def prompt_embedding(self, prompt: str, n: int) -> torch.Tensor:
        """A fixed pseudo-embedding of the prompt (this build has no text encoder): the conditioning
        vector of the guided branch."""
        seed = int.from_bytes(hashlib.blake2b(("cond:" + prompt).encode(), digest_size=4).digest(), "little")
        g = torch.Generator().manual_seed(seed)
        return torch.randn(1, self.model.dim, generator=g).expand(n, -1).to(self.device)

    @torch.no_grad()
    def generate(self, prompt: str, n: int = 1, size: str = "64x64", steps: Optional[int] = None,
                 seed: Optional[int] = None, guidance_scale: float = 1.0, parallel=None) -> List[np.ndarray]:
        w, h = (int(v) for v in size.lower().split("x"))
        if seed is None:                       # the same prompt gives the same image
            seed = int.from_bytes(hashlib.blake2b(prompt.encode(), digest_size=4).digest(), "little")
        g = torch.Generator().manual_seed(int(seed))
        noise = torch.randn(n, self.model.in_ch, self.latent_size, self.latent_size, generator=g).to(self.device)
        cache = make_cache(self.cache_kind) if self.cache_kind and self.cache_kind != "none" else None
        cond = self.prompt_embedding(prompt, n) if guidance_scale != 1.0 else None
        lat = self.model.sample(noise, steps=steps or self.steps, cache=cache, cond=cond, guidance_scale=guidance_scale,
                                st=parallel).float().cpu()
        rgb = torch.einsum("oc,bchw->bohw", self.to_rgb, lat)
        rgb = torch.nn.functional.interpolate(rgb, size=(h, w), mode="nearest")
        rgb = ((rgb.tanh() * 0.5 + 0.5) * 255).round().clamp(0, 255).to(torch.uint8)
        self.last_cache = cache
        return [im.permute(1, 2, 0).contiguous().numpy() for im in rgb]

    def openai_response(self, body: dict) -> dict:
        """`POST /v1/images/generations` body -> response ({created, data: [{b64_json}, ...]})."""
        prompt = body.get("prompt")
        if not isinstance(prompt, str) or not prompt:
            raise ValueError("`prompt` is required")
        n = int(body.get("n") or 1)
        if not 1 <= n <= 8:
            raise ValueError("`n` must be between 1 and 8")
        size = str(body.get("size") or "64x64")
        try:
            w, h = (int(v) for v in size.lower().split("x"))
        except ValueError:
            raise ValueError("`size` must look like 256x256")
        if not (8 <= w <= 1024 and 8 <= h <= 1024):
            raise ValueError("`size` out of range")
        imgs = self.generate(prompt, n, size, body.get("num_inference_steps") or body.get("steps"), body.get("seed"),
                             guidance_scale=float(body.get("guidance_scale") or 1.0), parallel=getattr(self, "parallel", None))
        return {"created": int(time.time()),
                "data": [{"b64_json": base64.b64encode(encode_png(im)).decode()} for im in imgs]}
