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


class FluxImagePipeline:
    """The Flux-family pipeline (`dit/flux.py`) loaded from a checkpoint directory in the layout the public
    releases use — `transformer/`, `vae/`, `text_encoder/` (CLIP), `text_encoder_2/` (T5), `tokenizer/`,
    `tokenizer_2/`, each with its `config.json` and safetensors — behind the same `openai_response` interface as
    `ImagePipeline` (the reference's DiT master + image generation service for `--backend dit`)."""

    def __init__(self, pipe, clip_tokenizer, t5_tokenizer, clip_len: int = 77, t5_len: int = 512, steps: int = 28,
                 guidance_scale: float = 3.5, cache: str = "none"):
        self.pipe, self.clip_tok, self.t5_tok = pipe, clip_tokenizer, t5_tokenizer
        self.clip_len, self.t5_len, self.steps, self.guidance_scale, self.cache_kind = clip_len, t5_len, steps, guidance_scale, cache

    @staticmethod
    def from_pretrained(model_dir: str, dtype=torch.float32, device: str = "cpu", **kw) -> "FluxImagePipeline":
        import json
        import os

        from ..utils.loader import iterate_weights
        from ..utils.tokenizer import load_tokenizer
        from .flux import FluxArgs, FluxPipeline, FluxTransformer
        from .text_encoders import ClipTextEncoder, T5TextEncoder
        from .vae import VaeDecoder

        def cfg(sub):
            with open(os.path.join(model_dir, sub, "config.json")) as f:
                return json.load(f)

        tr = FluxTransformer(FluxArgs.from_config(cfg("transformer")), dtype, device)
        tr.load_weights(iterate_weights(os.path.join(model_dir, "transformer")))
        vc = cfg("vae")
        vae = VaeDecoder(latent_channels=vc.get("latent_channels", 16), out_channels=vc.get("out_channels", 3),
                         block_out_channels=tuple(vc.get("block_out_channels", (128, 256, 512, 512))),
                         layers_per_block=vc.get("layers_per_block", 2), norm_groups=vc.get("norm_num_groups", 32),
                         scaling_factor=vc.get("scaling_factor", 0.3611), shift_factor=vc.get("shift_factor", 0.1159) or 0.0,
                         dtype=dtype, device=device)
        vae.load_weights(iterate_weights(os.path.join(model_dir, "vae")))
        clip = ClipTextEncoder.from_pretrained(os.path.join(model_dir, "text_encoder"), dtype, device)
        t5 = T5TextEncoder.from_pretrained(os.path.join(model_dir, "text_encoder_2"), dtype, device)
        pipe = FluxPipeline(tr, vae, clip, t5, latent_channels=vc.get("latent_channels", 16))
        return FluxImagePipeline(pipe, load_tokenizer(os.path.join(model_dir, "tokenizer")),
                                 load_tokenizer(os.path.join(model_dir, "tokenizer_2")),
                                 clip_len=int(clip.cfg.get("max_position_embeddings", 77)), **kw)

    def _ids(self, tok, prompt: str, length: int, pad: int, eos: Optional[int], bos: Optional[int] = None) -> torch.Tensor:
        ids = list(tok.encode(prompt))
        if bos is not None:
            ids = [bos] + ids
        ids = ids[: length - (1 if eos is not None else 0)]
        if eos is not None:
            ids.append(eos)
        return torch.tensor([ids + [pad] * (length - len(ids))], dtype=torch.long)

    @torch.no_grad()
    def generate(self, prompt: str, n: int = 1, size: str = "1024x1024", steps: Optional[int] = None, seed: Optional[int] = None,
                 guidance_scale: Optional[float] = None) -> List[np.ndarray]:
        w, h = (int(v) for v in size.lower().split("x"))
        if seed is None:
            seed = int.from_bytes(hashlib.blake2b(prompt.encode(), digest_size=4).digest(), "little")
        ccfg = self.pipe.clip.cfg
        eos, bos = int(ccfg.get("eos_token_id", 2)), ccfg.get("bos_token_id")
        clip_ids = self._ids(self.clip_tok, prompt, self.clip_len, eos, eos, bos)       # CLIP pads with its end-of-text token
        t5_eos = int(getattr(self.pipe.t5.model.args, "eos_token_id", 1))
        t5_ids = self._ids(self.t5_tok, prompt, min(self.t5_len, 512), int(self.pipe.t5.model.args.pad_token_id), t5_eos)
        cache = make_cache(self.cache_kind) if self.cache_kind and self.cache_kind != "none" else None
        img = self.pipe(clip_ids.expand(n, -1), t5_ids.expand(n, -1), height=h, width=w, steps=int(steps or self.steps),
                        guidance_scale=float(self.guidance_scale if guidance_scale is None else guidance_scale), seed=int(seed),
                        cache=cache)
        rgb = ((img.float().cpu() * 0.5 + 0.5) * 255).round().clamp(0, 255).to(torch.uint8)
        return [im.permute(1, 2, 0).contiguous().numpy() for im in rgb]

    def openai_response(self, body: dict) -> dict:
        prompt = body.get("prompt")
        if not isinstance(prompt, str) or not prompt:
            raise ValueError("`prompt` is required")
        n = int(body.get("n") or 1)
        if not 1 <= n <= 8:
            raise ValueError("`n` must be between 1 and 8")
        size = str(body.get("size") or "1024x1024")
        try:
            w, h = (int(v) for v in size.lower().split("x"))
        except ValueError:
            raise ValueError("`size` must look like 1024x1024")
        if w % 16 or h % 16 or not (16 <= w <= 2048 and 16 <= h <= 2048):
            raise ValueError("`size`: both sides must be multiples of 16 between 16 and 2048")
        imgs = self.generate(prompt, n, size, body.get("num_inference_steps") or body.get("steps"), body.get("seed"),
                             body.get("guidance_scale"))
        return {"created": int(time.time()), "data": [{"b64_json": base64.b64encode(encode_png(im)).decode()} for im in imgs]}
