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
from ..multimodal.media import decode_video
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
    def prepare(self, token_ids: Sequence[int], images: Sequence, videos: Sequence = (),
                second_per_grid: Optional[Sequence[float]] = None) -> tuple:
        """(expanded token ids, MMInput) for one request.  `videos`: frame stacks [T, 3, H, W] (or lists of
        frames), one per video placeholder; `second_per_grid` (Qwen2.5-VL) is the time one temporal patch of
        each video spans, which scales the videos' temporal rotary positions."""
        from ..multimodal.media import Qwen2VLVideoProcessor, video_mrope_positions
        model = self.engine.model
        args = self.engine.args
        pixel_values, grid = self.processor(images)
        counts = self.processor.tokens_per_image(grid)
        ids = expand_image_tokens(token_ids, self.image_token_id, counts) if (len(images) or self.image_token_id in token_ids) \
            else [int(t) for t in token_ids]
        embeds = model.encode_images(pixel_values, grid) if len(images) else torch.zeros(0, args.hidden_size)
        hashed = [pixel_values]
        if len(videos):
            if args.video_token_id < 0:
                raise ValueError("this model has no video placeholder token")
            if getattr(self, "video_processor", None) is None:
                self.video_processor = Qwen2VLVideoProcessor(self.processor.p, self.processor.m, self.processor.tp)
            v_pixels, v_grid = self.video_processor(videos)
            ids = expand_image_tokens(ids, args.video_token_id, self.video_processor.tokens_per_video(v_grid))
            v_embeds = model.encode_images(v_pixels, v_grid)
            hashed.append(v_pixels)
            # one embedding row per placeholder, in prompt order: images and videos may interleave
            kinds = torch.tensor([1 if t == self.image_token_id else 2 if t == args.video_token_id else 0 for t in ids])
            rows = torch.empty((int((kinds > 0).sum()), embeds.shape[1] if embeds.numel() else v_embeds.shape[1]),
                               dtype=v_embeds.dtype, device=v_embeds.device)
            order = kinds[kinds > 0]
            rows[order == 1] = embeds.to(rows.dtype).to(rows.device)
            rows[order == 2] = v_embeds
            embeds = rows
            tps = float(getattr(args, "tokens_per_second", 0.0) or 0.0)
            pos3, delta = video_mrope_positions(ids, {"image": self.image_token_id, "video": args.video_token_id},
                                                {"image": grid.tolist(), "video": v_grid.tolist()}, self.processor.m,
                                                second_per_grid, tps)
            where = [i for i, k in enumerate(kinds.tolist()) if k]
        else:
            pos3, delta = mrope_positions(ids, self.image_token_id, grid, self.processor.m)
            where = [i for i, t in enumerate(ids) if t == self.image_token_id]
        assert len(where) == embeds.shape[0]
        h = hashlib.blake2b(digest_size=8)
        for t in hashed:
            h.update(t.numpy().tobytes())
        digest = h.digest() if (len(images) or len(videos)) else b"\0" * 8
        return ids, MMInput(embeds, where, pos3, delta, int.from_bytes(digest, "little"))

    def generate_mm(self, requests: List[dict], sampling_params: Optional[SamplingParams] = None):
        """requests: [{"prompt_token_ids": [...] | "prompt": str, "images": [PIL | array | tensor, ...],
        "videos": [frames [T, 3, H, W] | path | bytes, ...]}].
        Returns one list of generated token ids per request (and texts when a tokenizer is loaded)."""
        sp = sampling_params or SamplingParams()
        eng = self.engine
        out = {}
        for i, r in enumerate(requests):
            ids = r.get("prompt_token_ids")
            if ids is None:
                ids = self._encode(r["prompt"])
            videos = [decode_video(v)[0] if isinstance(v, (str, bytes, bytearray)) else v for v in (r.get("videos") or [])]
            ids, mm = self.prepare(ids, r.get("images") or [], videos, r.get("second_per_grid"))
            eng.add_request(f"vlm-{i}", ids, temperature=sp.temperature, top_p=sp.top_p, top_k=sp.top_k,
                            max_tokens=sp.max_tokens, ignore_eos=sp.ignore_eos,
                            mm=mm if (r.get("images") or videos) else None)
            out[f"vlm-{i}"] = []
        while eng.has_unfinished():
            for ev in eng.step():
                if ev.token >= 0 and ev.request_id in out:
                    out[ev.request_id].append(int(ev.token))
        for ev in eng.drain():
            if ev.token >= 0 and ev.request_id in out:
                out[ev.request_id].append(int(ev.token))
        return [out[f"vlm-{i}"] for i in range(len(requests))]
