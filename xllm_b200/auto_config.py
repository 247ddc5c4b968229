"""Hardware-aware launch configuration: looks at the model and at the GPUs of this host and writes the
JSON that `python -m xllm_b200.serve --config_json_file ...` takes.

    python -m xllm_b200.auto_config --model /path/to/Qwen3-8B --out launch.json [--tpot_slo_ms 50]

Parity: the reference's `xllm/auto_config` (a per-model-type tuner that adjusts a base config to
the detected platform and device count: auto_config/utils.py `BaseTuner`, `detect_hardware`;
auto_config/qwen3.py).  The policy here is written for B200 boxes: it sizes tensor parallelism from
the weight bytes against HBM, the prefill chunk from the compute/bandwidth ridge of the part and the
running-sequence cap from the KV bytes that are left.
"""
from __future__ import annotations

import argparse
import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

from .models.config import ModelArgs, load_model_args, preset


@dataclass
class Hardware:
    n_gpus: int = 1
    hbm_bytes: int = 180 * 10 ** 9
    name: str = "NVIDIA B200"
    nvlink: bool = True


def detect_hardware(probe: Optional[Callable[[], List[dict]]] = None) -> Hardware:
    """`probe` returns one dict per visible GPU ({"name", "memory_bytes"}); the default asks torch.
    A host without GPUs reports one nominal B200, so that a config can be prepared elsewhere."""
    gpus = []
    if probe is not None:
        gpus = probe()
    else:
        try:
            import torch
            if torch.cuda.is_available():
                for i in range(torch.cuda.device_count()):
                    p = torch.cuda.get_device_properties(i)
                    gpus.append({"name": p.name, "memory_bytes": int(p.total_memory)})
        except Exception:      # no usable torch / driver: fall through to the nominal part
            gpus = []
    if not gpus:
        return Hardware()
    return Hardware(n_gpus=len(gpus), hbm_bytes=min(g["memory_bytes"] for g in gpus), name=gpus[0]["name"],
                    nvlink=len(gpus) > 1)


def weight_bytes(a: ModelArgs, bytes_per_param: float = 2.0) -> int:
    H, L = a.hidden_size, a.num_hidden_layers
    if a.kv_lora_rank:
        qk = a.qk_nope_head_dim + a.qk_rope_head_dim
        attn = (H * a.q_lora_rank + a.q_lora_rank * a.num_attention_heads * qk if a.q_lora_rank
                else H * a.num_attention_heads * qk)
        attn += H * (a.kv_lora_rank + a.qk_rope_head_dim) + a.kv_lora_rank * a.num_attention_heads * (a.qk_nope_head_dim + a.v_head_dim)
        attn += a.num_attention_heads * a.v_head_dim * H
    else:
        attn = H * a.head_dim * (2 * a.num_attention_heads + 2 * a.num_key_value_heads)
    dense = 3 * H * a.intermediate_size
    moe = a.num_experts * 3 * H * a.moe_intermediate_size + H * a.num_experts
    moe += 3 * H * (a.shared_expert_intermediate_size or a.moe_intermediate_size * a.n_shared_experts)
    total = 0
    for i in range(L):
        total += attn + (moe if a.is_moe_layer(i) else dense)
    total += a.vocab_size * H * (1 if a.tie_word_embeddings else 2)
    return int(total * bytes_per_param)


def kv_bytes_per_token(a: ModelArgs, tp: int, latent: bool) -> int:
    if a.kv_lora_rank and latent:
        return a.num_hidden_layers * (a.kv_lora_rank + a.qk_rope_head_dim) * 2
    if a.kv_lora_rank:
        return a.num_hidden_layers * 2 * (a.num_attention_heads // tp) * 256 * 2
    return a.num_hidden_layers * 2 * max(1, a.num_key_value_heads // tp) * a.head_dim * 2


def tune(a: ModelArgs, hw: Hardware, tpot_slo_ms: float = 0.0, max_model_len: int = 0) -> Dict:
    cfg: Dict = {"block_size": 16, "enable_prefix_cache": True, "enable_chunked_prefill": True,
                 "enable_schedule_overlap": True, "enable_graph": True, "max_memory_utilization": 0.9}
    wb = weight_bytes(a)
    # smallest power-of-two tensor-parallel degree whose weight shard leaves at least 30 % of HBM for the KV cache
    tp = 1
    while tp < hw.n_gpus and wb / tp > 0.6 * hw.hbm_bytes:
        tp *= 2
    heads = a.num_key_value_heads if not a.kv_lora_rank else a.num_attention_heads
    while tp > 1 and (a.num_attention_heads % tp or (heads % tp and tp % heads)):
        tp //= 2
    cfg["nnodes"] = tp
    cfg["dp_size"] = max(1, hw.n_gpus // tp) if a.num_experts == 0 else 1
    if a.num_experts > 0 and tp > 1:
        cfg["ep_size"] = tp                       # experts sharded over the same ranks, all-to-all dispatch
    latent = bool(a.kv_lora_rank)
    if latent:
        cfg["mla_latent_cache"] = True
    # prefill chunk: a B200 reaches its GEMM plateau from ~4k tokens per step; 8k keeps the step under ~100 ms for 8B-class models
    flops_per_token = 2.0 * wb / 2 / max(tp, 1)
    step_ms_at_8k = 8192 * flops_per_token / 1.4e15 * 1e3
    cfg["max_tokens_per_batch"] = 8192 if step_ms_at_8k <= 150 else 4096
    if tpot_slo_ms > 0:                           # a decode token waits for at most one prefill chunk
        while cfg["max_tokens_per_batch"] > 1024 and \
                cfg["max_tokens_per_batch"] * flops_per_token / 1.4e15 * 1e3 > tpot_slo_ms:
            cfg["max_tokens_per_batch"] //= 2
    free = hw.hbm_bytes * cfg["max_memory_utilization"] - wb / tp - 6 * 10 ** 9
    per_tok = kv_bytes_per_token(a, tp, latent)
    kv_tokens = max(0, int(free // per_tok))
    mml = max_model_len or min(a.max_position_embeddings, 32768)
    cfg["max_model_len"] = mml
    cfg["max_seqs_per_batch"] = int(max(8, min(512, kv_tokens // max(1, mml // 4))))
    cfg["kv_tokens_estimate"] = kv_tokens
    if a.num_nextn_predict_layers > 0:
        cfg["num_speculative_tokens"] = 1
        cfg["speculative_method"] = "mtp"
        cfg["enable_schedule_overlap"] = False
    if "linear_num_value_heads" in a.extra:
        cfg["enable_prefix_cache"] = False
        cfg["enable_graph"] = False
    return cfg


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="model directory or preset name")
    ap.add_argument("--out", default="")
    ap.add_argument("--tpot_slo_ms", type=float, default=0.0)
    ap.add_argument("--max_model_len", type=int, default=0)
    ns = ap.parse_args(argv)
    a = load_model_args(ns.model) if os.path.isdir(ns.model) else preset(ns.model)
    cfg = tune(a, detect_hardware(), ns.tpot_slo_ms, ns.max_model_len)
    text = json.dumps(cfg, indent=1, sort_keys=True)
    if ns.out:
        with open(ns.out, "w") as f:
            f.write(text + "\n")
    print(text)
    return cfg


if __name__ == "__main__":
    main()
