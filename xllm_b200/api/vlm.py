"""Offline API for vision-language models.

Parity: `VLM` / `VLMMaster` of the reference (xllm/pybind/vlm.py, core/distributed_runtime/
vlm_master.cpp): a request is text (or token ids) with image placeholders plus the images; the master
preprocesses the images, runs the vision encoder, expands the placeholders and hands the scheduler a
token sequence whose image positions are filled from the encoder output.
"""
from __future__ import annotations

import hashlib
from typing import List, Optional, Sequence

import torch

from ..multimodal.image import MMInput, Qwen2VLImageProcessor, expand_image_tokens, mrope_positions
from .llm import LLM, SamplingParams


class VLM(LLM):
    def __init__(self, *args, processor: Optional[Qwen2VLImageProcessor] = None, **kw):
        super().__init__(*args, **kw)
        model = self.engine.model
        if not hasattr(model, "visual"):
            raise ValueError("VLM needs a model with a vision tower")
        v = model.visual
        self.processor = processor or Qwen2VLImageProcessor(v.patch, v.merge, v.tp)
        self.image_token_id = self.engine.args.image_token_id

    @torch.no_grad()
    def prepare(self, token_ids: Sequence[int], images: Sequence) -> tuple:
        """(expanded token ids, MMInput) for one request."""
        model = self.engine.model
        pixel_values, grid = self.processor(images)
        counts = self.processor.tokens_per_image(grid)
        ids = expand_image_tokens(token_ids, self.image_token_id, counts)
        embeds = model.encode_images(pixel_values, grid) if len(images) else torch.zeros(0, self.engine.args.hidden_size)
        pos3, delta = mrope_positions(ids, self.image_token_id, grid, self.processor.m)
        where = [i for i, t in enumerate(ids) if t == self.image_token_id]
        assert len(where) == embeds.shape[0]
        digest = hashlib.blake2b(pixel_values.numpy().tobytes(), digest_size=8).digest() if len(images) else b"\0" * 8
        return ids, MMInput(embeds, where, pos3, delta, int.from_bytes(digest, "little"))

    def generate_mm(self, requests: List[dict], sampling_params: Optional[SamplingParams] = None):
        """requests: [{"prompt_token_ids": [...] | "prompt": str, "images": [PIL | array | tensor, ...]}].
        Returns one list of generated token ids per request (and texts when a tokenizer is loaded)."""
        sp = sampling_params or SamplingParams()
        eng = self.engine
        out = {}
        for i, r in enumerate(requests):
            ids = r.get("prompt_token_ids")
            if ids is None:
                ids = self._encode(r["prompt"])
            ids, mm = self.prepare(ids, r.get("images") or [])
            eng.add_request(f"vlm-{i}", ids, temperature=sp.temperature, top_p=sp.top_p, top_k=sp.top_k,
                            max_tokens=sp.max_tokens, ignore_eos=sp.ignore_eos, mm=mm if r.get("images") else None)
            out[f"vlm-{i}"] = []
        while eng.has_unfinished():
            for ev in eng.step():
                if ev.token >= 0 and ev.request_id in out:
                    out[ev.request_id].append(int(ev.token))
        for ev in eng.drain():
            if ev.token >= 0 and ev.request_id in out:
                out[ev.request_id].append(int(ev.token))
        return [out[f"vlm-{i}"] for i in range(len(requests))]
