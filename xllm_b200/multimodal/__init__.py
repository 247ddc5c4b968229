"""Multimodal inputs: image preprocessing, prompt expansion, M-RoPE position ids."""
from .image import MMInput, Qwen2VLImageProcessor, expand_image_tokens, mrope_positions, smart_resize  # noqa: F401
from .media import (ClipImageProcessor, Glm4vImageProcessor, LogMelExtractor, MiniCPMVImageProcessor,  # noqa: F401
                    Qwen2VLVideoProcessor, decode_video, decode_wav, sample_frame_indices, video_mrope_positions)
