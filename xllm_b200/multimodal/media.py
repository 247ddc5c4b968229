"""Video, audio and further image preprocessing.

Parity: xllm/processors/{qwen2_vl_video_processor,glm4v_image_processor,glm4v_video_processor,
clip_image_processor,minicpmv_image_processor,audio_processor}.* and the frame sampling of the reference's
multimodal input path (core/framework/multimodal/*).  Everything is torch on the CPU after decoding
(OpenCV for video containers, the standard library for PCM wav); outputs have the layouts the vision /
audio towers take: patch rows [n, C * temporal * p * p] with a (t, h, w) grid per item, CHW crops, or
log-mel frames.
"""
from __future__ import annotations

import io
import math
import wave
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .image import CLIP_MEAN, CLIP_STD, _to_chw_float, smart_resize


# ------------------------------------------------------------------------------------------ video
def sample_frame_indices(total_frames: int, video_fps: float, target_fps: float = 2.0, min_frames: int = 4,
                         max_frames: int = 768, multiple: int = 2) -> List[int]:
    """Uniform sampling at `target_fps`, clamped to [min_frames, max_frames] and rounded down to a multiple of
    the temporal patch (Qwen2-VL's rule): indices into the decoded frame sequence."""
    if total_frames <= 0:
        return []
    want = total_frames / max(video_fps, 1e-6) * target_fps
    lo = math.ceil(min_frames / multiple) * multiple
    hi = math.floor(min(max_frames, total_frames) / multiple) * multiple
    n = min(max(want, lo), max(hi, lo))
    n = max(multiple, math.floor(n / multiple) * multiple)
    n = min(n, max(total_frames, 1))
    return torch.linspace(0, total_frames - 1, int(n)).round().long().tolist()


def decode_video(source, target_fps: float = 2.0, **sampling) -> Tuple[torch.Tensor, float]:
    """File path or bytes of a container OpenCV can read -> (frames [T, 3, H, W] uint8 RGB, sampled fps)."""
    import os
    import tempfile

    import cv2
    tmp = None
    if isinstance(source, (bytes, bytearray)):
        tmp = tempfile.NamedTemporaryFile(suffix=".mp4", delete=False)
        tmp.write(source)
        tmp.close()
        source = tmp.name
    try:
        cap = cv2.VideoCapture(source)
        if not cap.isOpened():
            raise ValueError("cannot open video")
        fps = cap.get(cv2.CAP_PROP_FPS) or 25.0
        frames = []
        while True:
            ok, f = cap.read()
            if not ok:
                break
            frames.append(cv2.cvtColor(f, cv2.COLOR_BGR2RGB))
        cap.release()
    finally:
        if tmp is not None:
            os.unlink(tmp.name)
    if not frames:
        raise ValueError("video has no frames")
    idx = sample_frame_indices(len(frames), fps, target_fps, **sampling)
    picked = torch.from_numpy(np.stack([frames[i] for i in idx])).permute(0, 3, 1, 2).contiguous()
    return picked, len(idx) / max(len(frames) / fps, 1e-6)


class Qwen2VLVideoProcessor:
    """Frames [T, 3, H, W] -> patch rows and a (T / temporal_patch, gh, gw) grid.  The pixel budget applies
    per frame (`min_pixels` / `max_pixels` are the reference's shortest_edge / longest_edge of a video)."""

    def __init__(self, patch_size=14, merge_size=2, temporal_patch_size=2, min_pixels=128 * 28 * 28,
                 max_pixels=768 * 28 * 28, mean=CLIP_MEAN, std=CLIP_STD):
        self.p, self.m, self.tp = patch_size, merge_size, temporal_patch_size
        self.min_pixels, self.max_pixels = min_pixels, max_pixels
        self.mean = torch.tensor(mean).view(1, 3, 1, 1)
        self.std = torch.tensor(std).view(1, 3, 1, 1)

    def one(self, frames) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
        x = frames if isinstance(frames, torch.Tensor) else torch.stack([_to_chw_float(f) for f in frames])
        x = x.float()
        if x.max() > 1.5:
            x = x / 255.0
        T, C, H, W = x.shape
        h, w = smart_resize(H, W, self.p * self.m, self.min_pixels, self.max_pixels)
        if (h, w) != (H, W):
            x = torch.nn.functional.interpolate(x, size=(h, w), mode="bicubic", align_corners=False,
                                                antialias=True).clamp(0, 1)
        x = (x - self.mean) / self.std
        if T % self.tp:
            x = torch.cat([x, x[-1:].expand(self.tp - T % self.tp, -1, -1, -1)])
        gt, gh, gw, p, m = x.shape[0] // self.tp, h // self.p, w // self.p, self.p, self.m
        y = x.view(gt, self.tp, C, gh // m, m, p, gw // m, m, p)
        y = y.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(gt * gh * gw, C * self.tp * p * p)
        return y, (gt, gh, gw)

    def __call__(self, videos: Sequence):
        outs = [self.one(v) for v in videos]
        pixels = torch.cat([o[0] for o in outs]) if outs else torch.zeros(0, 3 * self.tp * self.p * self.p)
        return pixels, torch.tensor([o[1] for o in outs], dtype=torch.int64).view(-1, 3)

    def tokens_per_video(self, grid_thw) -> List[int]:
        return [int(t * h * w) // (self.m * self.m) for t, h, w in grid_thw.tolist()]


def video_mrope_positions(token_ids: Sequence[int], pad_ids: dict, grids: dict, merge_size: int = 2,
                          second_per_grid: Optional[Sequence[float]] = None, tokens_per_second: float = 0.0):
    """3-D rotary positions of a prompt with image AND video placeholders (already expanded).
    `pad_ids` = {"image": id, "video": id}; `grids` = {"image": [[t,h,w],...], "video": [...]}.
    With `tokens_per_second` > 0 (Qwen2.5-VL) the temporal index of video frame group k is
    floor(k * second_per_grid * tokens_per_second) instead of k.  Returns (positions [3, L], delta)."""
    L = len(token_ids)
    pos = torch.zeros(3, L, dtype=torch.int64)
    nxt, i = 0, 0
    seen = {"image": 0, "video": 0}
    kinds = {int(v): k for k, v in pad_ids.items()}
    while i < L:
        kind = kinds.get(int(token_ids[i]))
        if kind is None:
            pos[:, i] = nxt
            nxt += 1
            i += 1
            continue
        g = grids[kind][seen[kind]]
        t, h, w = (int(v) for v in g)
        gh, gw = h // merge_size, w // merge_size
        n = t * gh * gw
        tt = torch.arange(t)
        if kind == "video" and tokens_per_second > 0:
            spg = float(second_per_grid[seen[kind]]) if second_per_grid is not None else 1.0
            tt = (tt.double() * spg * tokens_per_second).long()
        tt = tt.view(t, 1, 1).expand(t, gh, gw).reshape(-1)
        hh = torch.arange(gh).view(1, gh, 1).expand(t, gh, gw).reshape(-1)
        ww = torch.arange(gw).view(1, 1, gw).expand(t, gh, gw).reshape(-1)
        pos[:, i:i + n] = torch.stack([tt, hh, ww]) + nxt
        nxt = int(pos[:, i:i + n].max()) + 1
        i += n
        seen[kind] += 1
    return pos, nxt - L


# ------------------------------------------------------------------------------------------ more image processors
class Glm4vImageProcessor:
    """GLM-4V family: the Qwen2-VL patch layout with GLM's pixel budget (shortest_edge 112 x 112,
    longest_edge 14 x 14 x 2 x 2 x 2 x 6144) — the budget counts the temporal patch too."""

    def __init__(self, patch_size=14, merge_size=2, temporal_patch_size=2, min_pixels=112 * 112,
                 max_pixels=14 * 14 * 2 * 2 * 2 * 6144, mean=CLIP_MEAN, std=CLIP_STD):
        self.p, self.m, self.tp = patch_size, merge_size, temporal_patch_size
        self.min_pixels, self.max_pixels = min_pixels, max_pixels
        self.mean = torch.tensor(mean).view(3, 1, 1)
        self.std = torch.tensor(std).view(3, 1, 1)

    def resize_target(self, T: int, H: int, W: int) -> Tuple[int, int]:
        """GLM's variant of smart_resize: sides to multiples of patch * merge under a budget of
        t * h * w pixels, short sides first scaled up to one factor."""
        f = self.p * self.m
        if T < self.tp:
            raise ValueError("fewer frames than the temporal patch")
        if H < f or W < f:
            s = max(f / H, f / W)
            H, W = int(H * s), int(W * s)
        if max(H, W) / min(H, W) > 200:
            raise ValueError("aspect ratio above 200")
        h, w = round(H / f) * f, round(W / f) * f
        t = round(T / self.tp) * self.tp
        if t * h * w > self.max_pixels:
            beta = math.sqrt(T * H * W / self.max_pixels)
            h = max(f, math.floor(H / beta / f) * f)
            w = max(f, math.floor(W / beta / f) * f)
        elif t * h * w < self.min_pixels:
            beta = math.sqrt(self.min_pixels / (T * H * W))
            h, w = math.ceil(H * beta / f) * f, math.ceil(W * beta / f) * f
        return h, w

    def one(self, img):
        x = _to_chw_float(img)
        C, H, W = x.shape
        h, w = self.resize_target(self.tp, H, W)
        if (h, w) != (H, W):
            x = torch.nn.functional.interpolate(x[None], size=(h, w), mode="bicubic", align_corners=False,
                                                antialias=True)[0].clamp(0, 1)
        x = (x - self.mean) / self.std
        frames = x[None].repeat(self.tp, 1, 1, 1)
        gh, gw, p, m = h // self.p, w // self.p, self.p, self.m
        y = frames.view(1, self.tp, C, gh // m, m, p, gw // m, m, p)
        y = y.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(gh * gw, C * self.tp * p * p)
        return y, (1, gh, gw)

    def __call__(self, images: Sequence):
        outs = [self.one(im) for im in images]
        pixels = torch.cat([o[0] for o in outs]) if outs else torch.zeros(0, 3 * self.tp * self.p * self.p)
        return pixels, torch.tensor([o[1] for o in outs], dtype=torch.int64).view(-1, 3)


Glm4vImageProcessor.tokens_per_image = lambda self, grid_thw: [int(t * h * w) // (self.m * self.m) for t, h, w in grid_thw.tolist()]


class ClipImageProcessor:
    """Shortest side to `size` (bicubic), centre crop `crop` x `crop`, CLIP normalisation -> [N, 3, crop, crop]."""

    def __init__(self, size=224, crop=224, mean=CLIP_MEAN, std=CLIP_STD):
        self.size, self.crop = size, crop
        self.mean = torch.tensor(mean).view(3, 1, 1)
        self.std = torch.tensor(std).view(3, 1, 1)

    def one(self, img) -> torch.Tensor:
        x = _to_chw_float(img)
        C, H, W = x.shape
        s = self.size / min(H, W)
        h, w = (self.size, int(W * s)) if H <= W else (int(H * s), self.size)
        x = torch.nn.functional.interpolate(x[None], size=(h, w), mode="bicubic", align_corners=False,
                                            antialias=True)[0].clamp(0, 1)
        top, left = (h - self.crop) // 2, (w - self.crop) // 2
        if top < 0 or left < 0:                              # smaller than the crop: pad with zeros around
            canvas = torch.zeros(C, max(h, self.crop), max(w, self.crop))
            canvas[:, max(0, -top): max(0, -top) + h, max(0, -left): max(0, -left) + w] = x
            x, top, left = canvas, max(0, top), max(0, left)
        x = x[:, top: top + self.crop, left: left + self.crop]
        return (x - self.mean) / self.std

    def __call__(self, images: Sequence) -> torch.Tensor:
        return torch.stack([self.one(im) for im in images]) if images else torch.zeros(0, 3, self.crop, self.crop)


class MiniCPMVImageProcessor:
    """MiniCPM-V's adaptive slicing: an overview image plus up to `max_slices` crops on the grid whose aspect
    ratio is closest (in log scale) to the image's; every piece is resized so that both sides are multiples
    of the patch and its area is about scale_resolution^2.  Returns (pieces [3, h, w] normalised, grid (cols,
    rows) or None without slices, per-piece (h, w) in patches)."""

    def __init__(self, max_slices=9, scale_resolution=448, patch_size=14, mean=(0.5, 0.5, 0.5), std=(0.5, 0.5, 0.5)):
        self.max_slices, self.res, self.p = max_slices, scale_resolution, patch_size
        self.mean = torch.tensor(mean).view(3, 1, 1)
        self.std = torch.tensor(std).view(3, 1, 1)

    def best_grid(self, W: int, H: int) -> Optional[Tuple[int, int]]:
        ratio = W * H / (self.res * self.res)
        n = min(math.ceil(ratio), self.max_slices)
        if n <= 1:
            return None
        log_ratio = math.log(W / H)
        best, err = None, float("inf")
        for cand in (n - 1, n, n + 1):
            if cand == 1 or cand > self.max_slices:
                continue
            for cols in range(1, cand + 1):
                if cand % cols == 0:
                    e = abs(log_ratio - math.log(cols / (cand // cols)))
                    if e < err:
                        best, err = (cols, cand // cols), e
        return best

    def _fit(self, W: int, H: int, upscale: bool) -> Tuple[int, int]:
        if W * H > self.res * self.res or upscale:
            r = W / H
            H = int(self.res / math.sqrt(r))
            W = int(H * r)
        return max(round(W / self.p) * self.p, self.p), max(round(H / self.p) * self.p, self.p)

    def _resize(self, x, w, h):
        return torch.nn.functional.interpolate(x[None], size=(h, w), mode="bicubic", align_corners=False,
                                               antialias=True)[0].clamp(0, 1)

    def __call__(self, img):
        x = _to_chw_float(img)
        _, H, W = x.shape
        grid = self.best_grid(W, H)
        pieces = []
        if grid is None:
            w, h = self._fit(W, H, upscale=True)
            pieces.append(self._resize(x, w, h))
        else:
            w, h = self._fit(W, H, upscale=False)
            pieces.append(self._resize(x, w, h))
            cols, rows = grid
            cw, ch = self._fit(max(1, W // cols), max(1, H // rows), upscale=True)
            whole = self._resize(x, cw * cols, ch * rows)
            for r in range(rows):
                for c in range(cols):
                    pieces.append(whole[:, r * ch:(r + 1) * ch, c * cw:(c + 1) * cw])
        sizes = [(pc.shape[1] // self.p, pc.shape[2] // self.p) for pc in pieces]
        return [(pc - self.mean) / self.std for pc in pieces], grid, sizes


# ------------------------------------------------------------------------------------------ audio
def decode_wav(source) -> Tuple[torch.Tensor, int]:
    """PCM wav (path or bytes; 8 / 16 / 32-bit) -> (mono float32 samples in [-1, 1], sample rate)."""
    f = wave.open(io.BytesIO(source) if isinstance(source, (bytes, bytearray)) else source, "rb")
    try:
        n, ch, width, rate = f.getnframes(), f.getnchannels(), f.getsampwidth(), f.getframerate()
        raw = f.readframes(n)
    finally:
        f.close()
    if width == 1:
        x = (torch.frombuffer(bytearray(raw), dtype=torch.uint8).float() - 128.0) / 128.0
    elif width == 2:
        x = torch.frombuffer(bytearray(raw), dtype=torch.int16).float() / 32768.0
    elif width == 4:
        x = torch.frombuffer(bytearray(raw), dtype=torch.int32).float() / 2147483648.0
    else:
        raise ValueError(f"unsupported sample width {width}")
    return x.view(-1, ch).mean(dim=1), rate


def resample_linear(x: torch.Tensor, rate: int, target: int) -> torch.Tensor:
    if rate == target or x.numel() == 0:
        return x
    n = int(round(x.numel() * target / rate))
    return torch.nn.functional.interpolate(x.view(1, 1, -1), size=n, mode="linear", align_corners=False).view(-1)


def mel_filterbank(n_mels: int, n_fft: int, rate: int) -> torch.Tensor:
    """Slaney-scale triangular filters with Slaney normalisation [n_mels, n_fft / 2 + 1] (Whisper's bank)."""
    def hz_to_mel(f):
        f = np.asarray(f, dtype=np.float64)
        lin = f / (200.0 / 3)
        log = 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (np.log(6.4) / 27.0)
        return np.where(f >= 1000.0, log, lin)

    def mel_to_hz(m):
        m = np.asarray(m, dtype=np.float64)
        lin = m * (200.0 / 3)
        log = 1000.0 * np.exp((np.log(6.4) / 27.0) * (m - 15.0))
        return np.where(m >= 15.0, log, lin)

    freqs = np.linspace(0, rate / 2, n_fft // 2 + 1)
    pts = mel_to_hz(np.linspace(hz_to_mel(0.0), hz_to_mel(rate / 2), n_mels + 2))
    diff = np.diff(pts)
    ramps = pts[:, None] - freqs[None, :]
    lower, upper = -ramps[:-2] / diff[:-1, None], ramps[2:] / diff[1:, None]
    fb = np.maximum(0, np.minimum(lower, upper))
    fb *= (2.0 / (pts[2:] - pts[:-2]))[:, None]
    return torch.from_numpy(fb).float()


class LogMelExtractor:
    """Whisper-style features: 16 kHz, 25 ms Hann window, 10 ms hop, `n_mels` Slaney filters, log10 clipped
    to 8 decades below the maximum and mapped to about [-1, 1]; audio padded / cut to `chunk_seconds`."""

    def __init__(self, n_mels=128, n_fft=400, hop=160, rate=16000, chunk_seconds=30):
        self.n_mels, self.n_fft, self.hop, self.rate, self.chunk = n_mels, n_fft, hop, rate, chunk_seconds
        self.filters = mel_filterbank(n_mels, n_fft, rate)
        self.window = torch.hann_window(n_fft, periodic=True)

    def __call__(self, samples: torch.Tensor, rate: Optional[int] = None, pad: bool = True) -> torch.Tensor:
        x = resample_linear(samples.float(), rate or self.rate, self.rate)
        if pad:
            n = self.chunk * self.rate
            x = torch.nn.functional.pad(x, (0, max(0, n - x.numel())))[:n]
        spec = torch.stft(x, self.n_fft, self.hop, window=self.window, return_complex=True)   # centred, reflect padding
        power = spec[..., :-1].abs() ** 2
        mel = self.filters @ power
        log = torch.clamp(mel, min=1e-10).log10()
        log = torch.maximum(log, log.max() - 8.0)
        return (log + 4.0) / 4.0                                  # [n_mels, frames]
