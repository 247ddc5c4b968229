"""MLA kernels against the PyTorch fp32 reference of the same math, and a DeepSeek-shaped engine on the
latent cache (eager and CUDA-graph decode)."""
import math

import pytest
import torch

from xllm_b200.ops import mla as mla_ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
L, R = 512, 64


def _cache(nblocks, page, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(nblocks, 1, page, L + R, device=DEV, dtype=torch.bfloat16, generator=g) * 0.5).contiguous()


@pytest.mark.parametrize("nh,page,lens,splits", [(16, 16, [1, 17, 300, 1024], 1), (128, 16, [700, 33], 4),
                                                 (5, 64, [129, 2000, 64], 3), (16, 16, [5000], 16)])
def test_mla_decode_matches_reference(nh, page, lens, splits):
    torch.manual_seed(1)
    N = len(lens)
    max_blocks = max((n + page - 1) // page for n in lens) + 1
    nb = N * max_blocks + 1
    cache = _cache(nb, page)
    bt = (torch.randperm(nb - 1, device=DEV)[: N * max_blocks] + 1).view(N, max_blocks).to(torch.int32)
    q = torch.randn(N, nh, L + R, device=DEV, dtype=torch.bfloat16) * 0.3
    sl = torch.tensor(lens, device=DEV, dtype=torch.int32)
    scale = 1.0 / math.sqrt(192)
    canary = torch.full((N + 2, nh, L), 3.0, device=DEV, dtype=torch.bfloat16)
    got = mla_ops.decode(q, cache, bt, scale, seq_lens=sl, splits=splits, out=canary[1:-1])
    want = mla_ops.decode_reference(q, cache, bt, sl, None, scale)
    err = (got.float() - want.float()).abs()
    assert bool((err <= 2e-2 + 2e-2 * want.float().abs()).all()), err.max().item()
    assert bool((canary[0] == 3).all()) and bool((canary[-1] == 3).all())


def test_mla_prompt_rows_see_their_own_prefix():
    """Rows of a prompt chunk: visible length from the position, block-table row from bt_rows."""
    torch.manual_seed(2)
    page, nh = 16, 16
    cache = _cache(64, page, seed=3)
    bt = (torch.randperm(63, device=DEV)[:40] + 1).view(2, 20).to(torch.int32)
    pos = torch.tensor([0, 1, 2, 100, 101, 299], device=DEV, dtype=torch.int64)
    rows = torch.tensor([0, 0, 0, 1, 1, 1], device=DEV, dtype=torch.int32)
    q = torch.randn(6, nh, L + R, device=DEV, dtype=torch.bfloat16) * 0.3
    got = mla_ops.decode(q, cache, bt, 0.07, positions=pos, bt_rows=rows, splits=2)
    want = mla_ops.decode_reference(q, cache, bt, pos + 1, rows, 0.07)
    err = (got.float() - want.float()).abs()
    assert bool((err <= 2e-2 + 2e-2 * want.float().abs()).all()), err.max().item()


def test_mla_cache_write_matches_reference():
    from xllm_b200.ops import reference as ref
    torch.manual_seed(3)
    T, nh, page, nope = 37, 16, 16, 128
    kv_a_full = torch.randn(T, L + R + 8, device=DEV, dtype=torch.bfloat16)
    kv_a = kv_a_full[:, : L + R]                                  # row stride != 576
    w = (torch.randn(L, device=DEV) * 0.1 + 1).to(torch.bfloat16)
    cs = ref.build_cos_sin_cache(R, 512, 10000.0, None, DEV)
    pos = torch.randint(0, 500, (T,), device=DEV)
    slots = torch.randperm(8 * page, device=DEV)[:T].to(torch.int32)
    slots[5] = -1
    q = torch.randn(T, nh, nope + R, device=DEV, dtype=torch.bfloat16)
    cache = torch.zeros(8, 1, page, L + R, device=DEV, dtype=torch.bfloat16)
    q_cat = torch.zeros(T, nh, L + R, device=DEV, dtype=torch.bfloat16)
    mla_ops.cache_write(kv_a, w, 1e-6, cs, pos, slots, cache, q[..., nope:], q_cat)
    cache_r = torch.zeros_like(cache).cpu()
    q_cat_r = torch.zeros_like(q_cat).cpu()
    mla_ops.cache_write(kv_a.cpu().contiguous(), w.cpu(), 1e-6, cs.cpu(), pos.cpu(), slots.cpu(), cache_r, q[..., nope:].cpu(),
                        q_cat_r)
    assert torch.allclose(cache.float().cpu(), cache_r.float(), atol=3e-2, rtol=2e-2)
    assert torch.allclose(q_cat.float().cpu(), q_cat_r.float(), atol=2e-2, rtol=2e-2)
    assert bool((q_cat[..., :L] == 0).all())                      # only the rotary columns were written


def test_deepseek_latent_engine_graph_equals_eager():
    from xllm_b200 import LLM, SamplingParams
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
    from xllm_b200.models import ModelArgs
    args = ModelArgs(model_type="deepseek_v3", vocab_size=8000, hidden_size=512, num_hidden_layers=2,
                     num_attention_heads=16, num_key_value_heads=16, head_dim=192, intermediate_size=1024, num_experts=8,
                     num_experts_per_tok=2, moe_intermediate_size=256, n_shared_experts=1, first_k_dense_replace=1,
                     scoring_func="sigmoid", n_group=2, topk_group=1, routed_scaling_factor=2.5, router_bias=True,
                     q_lora_rank=256, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                     qk_norm=False, rope_theta=10000.0, max_position_embeddings=4096)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 8000, (int(n),), generator=g).tolist() for n in (33, 70, 128, 5)]
    sp = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    outs = {}
    for name, kw in (("latent_eager", dict(mla_latent_cache=True, enable_graph=False)),
                     ("latent_graph", dict(mla_latent_cache=True, enable_graph=True)),
                     ("materialised", dict(mla_latent_cache=False, enable_graph=False))):
        llm = LLM.__new__(LLM)
        llm.engine = LLMEngine(EngineConfig(model="t", device="cuda:0", dtype="bfloat16", block_size=16, num_blocks=256,
                                            max_seqs_per_batch=8, max_tokens_per_batch=512, max_model_len=512,
                                            random_weights=True, **kw), model_args=args)
        llm.tokenizer = None
        outs[name] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        if name == "latent_graph":
            assert llm.engine.runner.graph_replays > 0
    agree = sum(a == b for a, b in zip(outs["latent_eager"], outs["latent_graph"]))
    assert agree >= 3, outs
    first = sum(a[0] == b[0] for a, b in zip(outs["latent_eager"], outs["materialised"]))
    assert first >= 3, outs
