"""Library arm of the benchmark: the same workload through vLLM from the image (cuBLAS GEMMs, NCCL
collectives, FlashAttention / FlashInfer attention, CUDA graphs), random weights of the same
architecture.  This is NOT the reference arm: it is the strongest all-library engine on the box and
gives the product's end-to-end number a denominator measured on the same GPU.

The reference's CUDA build is the same kind of stack (cuBLAS: xllm/core/kernels/cuda/matmul.cpp:21-25,
FlashInfer attention: xllm/core/layers/cuda/flashinfer_attention.cpp:224-304, NCCL process groups).
"""
from __future__ import annotations

import json
import os
import tempfile
import time

HF_CONFIGS = {
    "qwen3-8b": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096,
                     num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                     intermediate_size=12288, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960,
                     hidden_act="silu", tie_word_embeddings=False, attention_bias=False, torch_dtype="bfloat16",
                     bos_token_id=151643, eos_token_id=151645, use_sliding_window=False, sliding_window=None,
                     max_window_layers=36, attention_dropout=0.0, initializer_range=0.02, use_cache=True),
    "qwen3-32b": dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=5120,
                      num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                      intermediate_size=25600, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960,
                      hidden_act="silu", tie_word_embeddings=False, attention_bias=False, torch_dtype="bfloat16",
                      bos_token_id=151643, eos_token_id=151645, use_sliding_window=False, sliding_window=None,
                      max_window_layers=64, attention_dropout=0.0, initializer_range=0.02, use_cache=True),
    "qwen3-30b-a3b": dict(architectures=["Qwen3MoeForCausalLM"], model_type="qwen3_moe", vocab_size=151936,
                          hidden_size=2048, num_hidden_layers=48, num_attention_heads=32, num_key_value_heads=4,
                          head_dim=128, intermediate_size=6144, moe_intermediate_size=768, num_experts=128,
                          num_experts_per_tok=8, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[],
                          rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960, hidden_act="silu",
                          tie_word_embeddings=False, attention_bias=False, torch_dtype="bfloat16",
                          bos_token_id=151643, eos_token_id=151645, use_sliding_window=False, sliding_window=None,
                          router_aux_loss_coef=0.001, output_router_logits=False, use_cache=True),
}


def run(model: str, n_gpus: int, input_len: int, output_len: int, concurrency: int, requests: int, chunk: int,
        warmup_requests: int = 0, expert_parallel: bool = False, attention_backend: str = "") -> dict:
    """Whole-workload output tokens/s through vLLM's offline API.  Raises on any failure."""
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
    os.environ.setdefault("VLLM_DO_NOT_TRACK", "1")
    os.environ.setdefault("VLLM_WORKER_MULTIPROC_METHOD", "spawn")
    os.environ.setdefault("VLLM_HOST_IP", "127.0.0.1")
    if attention_backend:
        os.environ["VLLM_ATTENTION_BACKEND"] = attention_backend
    import numpy as np
    from vllm import LLM, SamplingParams

    d = tempfile.mkdtemp(prefix="libarm_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(HF_CONFIGS[model], f)
    kw = dict(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", seed=0,
              max_model_len=input_len + output_len + 16, max_num_seqs=concurrency,
              max_num_batched_tokens=concurrency + chunk, enable_prefix_caching=False, enable_chunked_prefill=True,
              gpu_memory_utilization=0.9, tensor_parallel_size=n_gpus, generation_config="vllm",
              disable_log_stats=True)
    if expert_parallel and n_gpus > 1:
        kw["enable_expert_parallel"] = True
    t0 = time.time()
    llm = LLM(**kw)
    init_s = time.time() - t0
    vocab = HF_CONFIGS[model]["vocab_size"]
    rng = np.random.default_rng(0)
    sp = SamplingParams(max_tokens=output_len, temperature=0.0, ignore_eos=True, detokenize=False)

    def prompts(n):
        return [{"prompt_token_ids": rng.integers(0, vocab - 1000, size=input_len).tolist()} for _ in range(n)]

    if warmup_requests:
        llm.generate(prompts(warmup_requests), SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True,
                                                              detokenize=False), use_tqdm=False)
    batch = prompts(requests)
    t0 = time.perf_counter()
    outs = llm.generate(batch, sp, use_tqdm=False)
    dt = time.perf_counter() - t0
    n_out = sum(len(o.outputs[0].token_ids) for o in outs)
    import vllm
    return {"value": n_out / dt, "seconds": dt, "output_tokens": n_out, "init_seconds": init_s,
            "library": f"vllm {vllm.__version__}", "attention_backend": os.environ.get("VLLM_ATTENTION_BACKEND", "default")}
