"""State slots of the linear-attention family under scheduling pressure: a run with so few KV blocks
that sequences are preempted and recomputed must give the same tokens as an unconstrained run, and
every slot must be returned."""
import torch

from xllm_b200 import LLM, SamplingParams
from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
from xllm_b200.models import ModelArgs


def _args():
    return ModelArgs(model_type="qwen3_next", vocab_size=600, hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=32, intermediate_size=128, qk_norm=True, partial_rotary_factor=0.25,
                     rope_theta=10000.0, max_position_embeddings=512, tie_word_embeddings=False,
                     extra=dict(linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16,
                                linear_value_head_dim=16, linear_conv_kernel_dim=4, full_attention_interval=4))


def _make(**kw):
    llm = LLM.__new__(LLM)
    llm.engine = LLMEngine(EngineConfig(model="n", device="cpu", dtype="float32", enable_graph=False, block_size=16,
                                        max_seqs_per_batch=6, **kw), model_args=_args())
    llm.tokenizer = None
    llm.engine.model.init_random(std=0.08, seed=3)
    return llm


def test_preemption_and_chunking_do_not_change_the_stream():
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 600, (n,), generator=g).tolist() for n in (30, 45, 18, 60, 25)]
    sp = SamplingParams(max_tokens=24, temperature=0.0, ignore_eos=True)
    roomy = _make(num_blocks=128, max_tokens_per_batch=256)
    want = [o.outputs[0].token_ids for o in roomy.generate(prompts, sp)]
    tight = _make(num_blocks=14, max_tokens_per_batch=32)          # 13 usable blocks for ~340 tokens of context
    got = [o.outputs[0].token_ids for o in tight.generate(prompts, sp)]
    assert got == want
    assert tight.engine.scheduler.num_preemptions > 0
    assert not tight.engine.model.state.owner and len(tight.engine.model.state.free) == 7
