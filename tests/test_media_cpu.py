"""Video / audio / further image processors against the HuggingFace processors of the same families."""
import io
import wave

import numpy as np
import pytest
import torch

from xllm_b200.multimodal import (ClipImageProcessor, Glm4vImageProcessor, LogMelExtractor, MiniCPMVImageProcessor,
                                  Qwen2VLVideoProcessor, decode_video, decode_wav, sample_frame_indices,
                                  video_mrope_positions)


def _frames(T, H, W, seed=0):
    g = torch.Generator().manual_seed(seed)
    # smooth content, so that resampling differences between implementations stay small
    base = torch.rand(T, 3, H // 8 + 1, W // 8 + 1, generator=g)
    x = torch.nn.functional.interpolate(base, size=(H, W), mode="bilinear", align_corners=False)
    return (x * 255).round().to(torch.uint8)


def test_qwen2vl_video_processor_matches_huggingface():
    from transformers import Qwen2VLVideoProcessor as HF
    hf = HF()
    mine = Qwen2VLVideoProcessor()
    for T, H, W in ((4, 224, 336), (5, 280, 280), (6, 500, 700)):
        v = _frames(T, H, W, seed=T)
        want = hf(videos=[v], return_tensors="pt", do_sample_frames=False)
        got, grid = mine([v])
        assert grid.tolist() == want["video_grid_thw"].tolist()
        assert got.shape == want["pixel_values_videos"].shape
        err = (got - want["pixel_values_videos"]).abs()
        assert err.max() < 0.08 and err.mean() < 8e-3, (T, H, W, float(err.max()), float(err.mean()))
    assert mine.tokens_per_video(grid) == [int(grid[0].prod()) // 4]


def test_glm4v_image_processor_matches_huggingface():
    from transformers import Glm4vImageProcessor as HF
    hf, mine = HF(), Glm4vImageProcessor()
    for H, W in ((224, 224), (300, 500), (60, 90)):
        img = _frames(1, H, W, seed=H)[0]
        want = hf(images=[img.permute(1, 2, 0).numpy()], return_tensors="pt")
        got, grid = mine([img])
        assert grid.tolist() == want["image_grid_thw"].tolist(), (H, W)
        err = (got - want["pixel_values"]).abs()
        assert err.max() < 0.1 and err.mean() < 6e-3, (H, W, float(err.max()), float(err.mean()))


def test_clip_image_processor_matches_huggingface():
    from transformers import CLIPImageProcessor as HF
    hf, mine = HF(), ClipImageProcessor()
    for H, W in ((224, 224), (300, 500), (640, 480)):
        img = _frames(1, H, W, seed=W)[0]
        want = hf(images=[img.permute(1, 2, 0).numpy()], return_tensors="pt")["pixel_values"]
        got = mine([img])
        assert got.shape == want.shape == (1, 3, 224, 224)
        err = (got - want).abs()
        assert err.mean() < 0.02, (H, W, float(err.max()), float(err.mean()))


def test_log_mel_matches_whisper_feature_extractor():
    from transformers import WhisperFeatureExtractor
    t = torch.arange(16000 * 3) / 16000.0
    x = 0.4 * torch.sin(2 * torch.pi * 440 * t) + 0.2 * torch.sin(2 * torch.pi * 1234 * t) + 0.01 * torch.randn(t.numel())
    for n_mels in (80, 128):
        hf = WhisperFeatureExtractor(feature_size=n_mels)
        want = torch.from_numpy(hf(x.numpy(), sampling_rate=16000, return_tensors="np")["input_features"][0])
        got = LogMelExtractor(n_mels=n_mels)(x)
        assert got.shape == want.shape == (n_mels, 3000)
        assert (got - want).abs().max() < 2e-3
    # wav container round trip, stereo 16-bit at 8 kHz -> mono, resampled
    buf = io.BytesIO()
    w = wave.open(buf, "wb")
    w.setnchannels(2)
    w.setsampwidth(2)
    w.setframerate(8000)
    pcm = (np.stack([np.sin(np.arange(8000) * 0.1), np.sin(np.arange(8000) * 0.1)], 1) * 20000).astype(np.int16)
    w.writeframes(pcm.tobytes())
    w.close()
    samples, rate = decode_wav(buf.getvalue())
    assert rate == 8000 and samples.shape == (8000,) and abs(float(samples.max()) - 20000 / 32768) < 1e-3
    feats = LogMelExtractor(n_mels=80)(samples, rate)
    assert feats.shape == (80, 3000) and torch.isfinite(feats).all()


def test_frame_sampling_and_video_positions(tmp_path):
    assert sample_frame_indices(100, 25.0, target_fps=2.0) == torch.linspace(0, 99, 8).round().long().tolist()
    assert len(sample_frame_indices(10, 25.0)) == 4                      # min_frames
    assert len(sample_frame_indices(100000, 25.0, max_frames=768)) == 768
    assert len(sample_frame_indices(3, 30.0)) in (2, 3)
    # text, video of 2 frame groups on a 2 x 2 merged grid, text; Qwen2.5-VL temporal scaling
    V, I = 900, 901
    toks = [1, 2] + [V] * 8 + [3]
    pos, delta = video_mrope_positions(toks, {"image": I, "video": V}, {"image": [], "video": [[2, 4, 4]]})
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:10].tolist() == [2] * 4 + [3] * 4 and pos[1, 2:6].tolist() == [2, 2, 3, 3] and pos[2, 2:6].tolist() == [2, 3, 2, 3]
    assert pos[:, 10].tolist() == [4, 4, 4] and delta == 5 - 11
    pos2, _ = video_mrope_positions(toks, {"image": I, "video": V}, {"image": [], "video": [[2, 4, 4]]},
                                    second_per_grid=[1.5], tokens_per_second=2.0)
    assert pos2[0, 2:10].tolist() == [2] * 4 + [5] * 4 and pos2[:, 10].tolist() == [6, 6, 6]
    # a real container through OpenCV
    cv2 = pytest.importorskip("cv2")
    path = str(tmp_path / "clip.avi")
    wr = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"MJPG"), 10.0, (64, 48))
    if not wr.isOpened():
        pytest.skip("no MJPG encoder in this OpenCV build")
    for i in range(30):
        wr.write(np.full((48, 64, 3), i * 8, dtype=np.uint8))
    wr.release()
    frames, fps = decode_video(path, target_fps=2.0)
    assert frames.shape == (6, 3, 48, 64) and abs(fps - 2.0) < 0.05
    assert int(frames[0].float().mean()) < int(frames[-1].float().mean())


def test_minicpmv_slicing():
    p = MiniCPMVImageProcessor(max_slices=9, scale_resolution=448)
    assert p.best_grid(400, 400) is None
    assert p.best_grid(1344, 448) == (3, 1) and p.best_grid(896, 896) == (2, 2)
    pieces, grid, sizes = p(_frames(1, 896, 1344)[0])
    assert grid == (3, 2) and len(pieces) == 1 + 6
    assert all(pc.shape[1] % 14 == 0 and pc.shape[2] % 14 == 0 for pc in pieces)
    assert all(abs(pc.shape[1] * pc.shape[2] - 448 * 448) / (448 * 448) < 0.15 for pc in pieces)
    assert sizes[0] == (pieces[0].shape[1] // 14, pieces[0].shape[2] // 14)
    small, grid, _ = p(_frames(1, 100, 150)[0])
    assert grid is None and len(small) == 1 and abs(small[0].shape[1] * small[0].shape[2] - 448 * 448) / (448 * 448) < 0.15
