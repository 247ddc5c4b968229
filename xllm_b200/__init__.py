"""xllm_b200 — a Blackwell (sm_100a) native LLM serving engine."""
__version__ = "0.1.0"

from .api.llm import LLM, BeamSearchParams, RequestOutput, SamplingParams, SequenceOutput  # noqa: E402,F401
from .engine.llm_engine import EngineConfig, LLMEngine  # noqa: E402,F401
