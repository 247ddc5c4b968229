"""Python side of the C API (`csrc/c_api/xllm.h`): JSON in, JSON out."""
from __future__ import annotations

import json

from .llm import LLM, SamplingParams


def create(model: str, options_json: str):
    return LLM(model, **json.loads(options_json or "{}"))


def generate(llm: LLM, prompts_json: str, sampling_json: str) -> str:
    prompts = json.loads(prompts_json)
    sp = SamplingParams(**json.loads(sampling_json or "{}"))
    outs = llm.generate(prompts, sp)
    res = []
    for o in outs:
        so = o.outputs[0]
        res.append({"token_ids": list(so.token_ids), "text": so.text or "", "finish_reason": so.finish_reason or "",
                    "prompt_tokens": o.usage.num_prompt_tokens})
    return json.dumps(res)


def stats(llm: LLM) -> str:
    return json.dumps({k: float(v) for k, v in llm.engine.stats().items()})
