"""Model registry: model_type / architecture name -> factory(args, dtype, device, parallel_state).

Counterpart of the reference's ModelRegistry and REGISTER_CAUSAL_MODEL macros
(xllm/models/model_registry.cpp, xllm/models/llm/qwen3.h:256-286).
"""
from __future__ import annotations

from typing import Callable, Dict

_FACTORIES: Dict[str, Callable] = {}


def register_model(*names):
    def deco(fn):
        for n in names:
            _FACTORIES[n.lower()] = fn
        return fn
    return deco


def supported_models():
    _import_all()
    return sorted(_FACTORIES)


def _import_all():
    from . import qwen  # noqa: F401
    for mod in ("qwen_moe", "deepseek", "qwen_vl", "families", "qwen3_next", "rwkv7", "glm4v"):
        try:
            __import__(f"{__package__}.{mod}")
        except ModuleNotFoundError as e:
            if e.name != f"{__package__}.{mod}":
                raise


def create_model(args, dtype, device, ps=None):
    _import_all()
    keys = [args.model_type.lower()] + [a.lower() for a in args.architectures]
    for k in keys:
        if k in _FACTORIES:
            return _FACTORIES[k](args, dtype, device, ps)
    raise KeyError(f"no model registered for {keys}; supported: {supported_models()}")
