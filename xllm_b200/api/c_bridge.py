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


def call(llm: LLM, method: str, args_json: str) -> str:
    """Dispatcher of `xllm_llm_call`."""
    a = json.loads(args_json or "{}")
    if method == "chat":
        tok = llm.tokenizer
        if tok is None:
            raise ValueError("chat needs a tokenizer with a chat template")
        text = tok.apply_chat_template(a["messages"], tools=a.get("tools"), add_generation_prompt=True,
                                       enable_thinking=bool(a.get("enable_thinking", True)))
        return generate(llm, json.dumps([text]), json.dumps(a.get("sampling") or {}))
    if method == "embed":
        outs = llm.embed(a["prompts"])
        return json.dumps([[float(x) for x in o.outputs.embedding] if hasattr(o, "outputs") else [float(x) for x in o]
                           for o in outs])
    if method == "beam_search":
        res = llm.beam_search(a["prompt"], beam_width=int(a.get("beam_width", 4)), max_tokens=int(a.get("max_tokens", 16)),
                              ignore_eos=bool(a.get("ignore_eos", False)))[0]     # one prompt -> its beams
        return json.dumps([{"token_ids": list(r.token_ids), "score": float(r.score),
                            "cumulative_logprob": float(r.cumulative_logprob)} for r in res])
    if method == "recommend":
        # the rec entry points of the reference's C API (c_api/rec.h): histories in, items with scores out
        res = llm.recommend(a["prompts"], beam_width=int(a.get("beam_width", 32)), num_steps=int(a.get("num_steps", 3)),
                            num_return=a.get("num_return"), valid_items=a.get("valid_items"))
        return json.dumps([[{"token_ids": list(it.token_ids), "logprob": float(it.logprob)} for it in items] for items in res])
    if method == "sleep":
        llm.sleep(int(a.get("level", 1)))
        return json.dumps({"ok": True})
    if method == "wake_up":
        llm.wake_up()
        return json.dumps({"ok": True})
    if method == "stats":
        return stats(llm)
    raise ValueError(f"unknown method {method!r}")
