"""xllm_b200 — a Blackwell (sm_100a) native LLM serving engine.

The names exported here are those of the reference's Python package (xllm/__init__.py:144-161):
LLM, VLM, Embedding, SamplingParams, BeamSearchParams, PoolingParams, RequestParams, RequestOutput,
Usage, SequenceOutput, plus the engine classes of this implementation.
"""
__version__ = "0.2.0"

from .api.llm import (LLM, BeamSearchParams, EmbeddingOutput, PoolingParams, RequestOutput, RequestParams,  # noqa: E402,F401
                      SamplingParams, SequenceOutput, Usage)
from .engine.llm_engine import EngineConfig, LLMEngine  # noqa: E402,F401

Options = EngineConfig      # the reference's option bag (xllm_export.Options)


def __getattr__(name):
    # heavier front ends are imported on first use
    if name == "VLM":
        from .api.vlm import VLM
        return VLM
    if name == "Embedding":
        from .api.embedding import Embedding
        return Embedding
    raise AttributeError(name)
