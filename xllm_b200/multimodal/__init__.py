"""Multimodal inputs: image preprocessing, prompt expansion, M-RoPE position ids."""
from .image import MMInput, Qwen2VLImageProcessor, expand_image_tokens, mrope_positions, smart_resize  # noqa: F401
