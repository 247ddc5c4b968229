"""Worker for test_dp_attention_cpu.py: two data-parallel ranks (gloo, CPU), experts split over both,
different requests on each rank; rank 1 runs out of work early and must keep pairing collectives."""
import json
import os
import sys

import torch
import torch.distributed as dist

from xllm_b200.api.llm import LLM, SamplingParams
from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
from xllm_b200.models import ModelArgs
from xllm_b200.parallel.state import init_parallel


def args():
    return ModelArgs(model_type="qwen3_moe", vocab_size=500, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=16, intermediate_size=128, num_experts=8, num_experts_per_tok=2,
                     moe_intermediate_size=32, norm_topk_prob=True, tie_word_embeddings=False, max_position_embeddings=256)


def main():
    ps = init_parallel(dp_size=2, ep_size=2, backend="gloo")
    assert ps.tp_size == 1 and ps.dp_rank == ps.rank
    from mp_tp_engine import hf_names
    from xllm_b200.models import create_model
    from xllm_b200.parallel.state import single
    a = args()
    full = create_model(a, torch.float32, "cpu", single())     # the same full model on every rank
    full.init_random(seed=7)
    model = create_model(a, torch.float32, "cpu", ps)           # this rank's share of the experts
    model.load_weights(list(hf_names(full)), strict=True)
    cfg = dict(model="m", device="cpu", dtype="float32", num_blocks=64, enable_graph=False, max_tokens_per_batch=32,
               enable_schedule_overlap=False)
    eng = LLMEngine(EngineConfig(**cfg), ps=ps, model=model, model_args=a)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (9, 40, 17, 5)]
    ref = LLM.__new__(LLM)
    ref.engine = LLMEngine(EngineConfig(**cfg), ps=single(), model=full, model_args=a)
    ref.tokenizer = None
    mine = {0: [0, 1, 2], 1: [3]}[ps.rank]          # rank 1 gets one short request
    for i in mine:
        eng.add_request(f"r{i}", prompts[i], temperature=0.0, max_tokens=12 if ps.rank == 0 else 3, ignore_eos=True)
    out = {f"r{i}": [] for i in mine}
    while eng.dp_has_unfinished():
        for ev in eng.step():
            if ev.token >= 0:
                out[ev.request_id].append(int(ev.token))
    want = {}
    for i in mine:
        sp = SamplingParams(max_tokens=12 if ps.rank == 0 else 3, temperature=0.0, ignore_eos=True)
        want[f"r{i}"] = ref.generate([prompts[i]], sp)[0].outputs[0].token_ids
    print("RESULT", ps.rank, json.dumps({"out": out, "want": want, "fake": eng.fake_steps, "dp_steps": eng.dp_steps}),
          flush=True)
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
