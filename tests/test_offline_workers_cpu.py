"""`LLM(devices="a,b")` starts its own worker ranks: two CPU ranks over gloo give the tokens of one rank."""
import os

import torch

from xllm_b200 import LLM, SamplingParams
from xllm_b200.engine.offline_worker import device_indices, parse_devices


def test_parse_devices():
    assert parse_devices(None) == ["auto"] and parse_devices("cuda") == ["cuda:0"]
    assert parse_devices("cuda:2, cuda:5") == ["cuda:2", "cuda:5"] and device_indices(["cuda:2", "cuda:5"]) == [2, 5]


def _write_checkpoint(tmp_path):
    """A small Qwen3 checkpoint in the HuggingFace layout, so that every rank loads the same weights."""
    import json

    from xllm_b200.utils.loader import save_file
    cfg = {"model_type": "qwen3", "vocab_size": 512, "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
           "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
           "tie_word_embeddings": False, "max_position_embeddings": 512, "torch_dtype": "float32"}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    g = torch.Generator().manual_seed(0)
    t = {"model.embed_tokens.weight": torch.randn(512, 64, generator=g) * 0.5, "model.norm.weight": torch.ones(64),
         "lm_head.weight": torch.randn(512, 64, generator=g) * 0.5}
    for i in range(2):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"] = torch.ones(64)
        t[p + "post_attention_layernorm.weight"] = torch.ones(64)
        t[p + "self_attn.q_norm.weight"] = torch.ones(16)
        t[p + "self_attn.k_norm.weight"] = torch.ones(16)
        for n, shape in (("self_attn.q_proj", (64, 64)), ("self_attn.k_proj", (32, 64)), ("self_attn.v_proj", (32, 64)),
                         ("self_attn.o_proj", (64, 64)), ("mlp.gate_proj", (128, 64)), ("mlp.up_proj", (128, 64)),
                         ("mlp.down_proj", (64, 128))):
            t[p + n + ".weight"] = torch.randn(*shape, generator=g) * 0.2
    save_file(t, str(tmp_path / "model.safetensors"), {"format": "pt"})
    return str(tmp_path)


def test_two_spawned_ranks_match_one(monkeypatch, tmp_path):
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        monkeypatch.delenv(k, raising=False)
    model = _write_checkpoint(tmp_path)
    kw = dict(dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=4, max_tokens_per_batch=128,
              enable_graph=False)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (21, 9)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    one = [o.outputs[0].token_ids for o in LLM(model, devices="cpu", **kw).generate(prompts, sp)]
    llm = LLM(model, devices="cpu,cpu", **kw)
    try:
        assert llm.engine.ps.world_size == 2 and llm._workers is not None and llm._workers.alive()
        assert llm.engine.ps.ctl is not None          # control events travel through shared memory
        two = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        again = [o.outputs[0].token_ids for o in llm.generate(prompts[:1], sp)]
    finally:
        llm.close()
    assert two == one and again == one[:1]
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        os.environ.pop(k, None)


def test_eagle3_head_runs_replicated_under_tensor_parallelism(monkeypatch, tmp_path):
    """Two ranks, the target sharded, the EAGLE-3 head whole on each: greedy output equals the unspeculated
    single-rank run, and drafts are proposed and verified."""
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        monkeypatch.delenv(k, raising=False)
    model = _write_checkpoint(tmp_path)
    kw = dict(dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=4, max_tokens_per_batch=128,
              enable_graph=False)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (17, 30)]
    sp = SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True)
    plain = [o.outputs[0].token_ids for o in LLM(model, devices="cpu", **kw).generate(prompts, sp)]
    llm = LLM(model, devices="cpu,cpu", num_speculative_tokens=2, speculative_method="eagle3", **kw)
    try:
        eng = llm.engine
        assert eng.ps.tp_size == 2 and eng.eagle3.ps.tp_size == 1 and eng.eagle3.kv_heads_full == 2
        assert eng.spec.drafter.kv[0].shape[1] == 2 and eng.runner.kv_caches[0][0].shape[1] == 1
        spec = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        stats = eng.spec.stats() if hasattr(eng.spec, "stats") else {}
    finally:
        llm.close()
    assert spec == plain, (spec, plain, stats)
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        os.environ.pop(k, None)
