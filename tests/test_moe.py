"""Mixture-of-experts: routing / fused layer against the PyTorch reference (GPU), the MoE model end
to end on CPU (expert-sliced weights reproduce the full model), checkpoint-name loading."""
import pytest
import torch

from xllm_b200.models import ModelArgs, create_model
from xllm_b200.ops import moe as M


def _args(**kw):
    base = dict(model_type="qwen3_moe", vocab_size=1000, hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=64, intermediate_size=512, num_experts=8, num_experts_per_tok=2,
                moe_intermediate_size=128, norm_topk_prob=True, max_position_embeddings=512, tie_word_embeddings=False)
    base.update(kw)
    return ModelArgs(**base)


def test_route_reference_group_limited():
    torch.manual_seed(0)
    logits = torch.randn(16, 32)
    ids, w = M.route_reference(logits, 4, "sigmoid", torch.randn(32) * 0.1, n_group=4, topk_group=2, renorm=True, scale=2.5)
    assert ids.shape == (16, 4) and torch.allclose(w.sum(-1), torch.full((16,), 2.5))
    assert bool(((ids // 8).unique(dim=1).shape[1] <= 4))
    for t in range(16):
        assert len(set((ids[t] // 8).tolist())) <= 2  # at most topk_group groups are used


def test_moe_model_cpu_runs_and_loads_expert_names():
    from xllm_b200 import LLM, SamplingParams
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
    args = _args()
    m = create_model(args, torch.float32, "cpu")
    names = [n for n, _ in m.named_loaders()]
    assert "model.layers.0.mlp.experts.3.gate_proj.weight" in names and "model.layers.1.mlp.gate.weight" in names
    llm = LLM.__new__(LLM)
    llm.engine = LLMEngine(EngineConfig(model="m", device="cpu", dtype="float32", num_blocks=64, enable_graph=False),
                           model_args=args)
    llm.tokenizer = None
    out = llm.generate([[1, 2, 3, 4, 5, 6, 7]], SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True))
    assert len(out[0].outputs[0].token_ids) == 5


@pytest.mark.gpu
@pytest.mark.parametrize("scoring,n_group,topk_group,bias,E,K", [("softmax", 1, 1, False, 128, 8), ("sigmoid", 8, 4, True, 256, 8),
                                                                ("softmax", 1, 1, False, 8, 2)])
def test_route_kernel_matches_reference(scoring, n_group, topk_group, bias, E, K):
    from xllm_b200.ops import _lib
    from xllm_b200.ops._lib import ptr, stream
    torch.manual_seed(1)
    T = 77
    logits = torch.randn(T, E, device="cuda")
    b = (torch.randn(E, device="cuda") * 0.2) if bias else None
    ws = M.MoeWorkspace(T, K, E, E, 64, 64, "cuda")
    lib = _lib.load()
    assert lib.xllm_moe_route(ptr(logits), 1, ptr(b), ptr(ws.topk_ids), ptr(ws.topk_w), ptr(ws.counts), ptr(ws.slot), T, E,
                              K, n_group, topk_group, 0 if scoring == "softmax" else 1, 1, 2.0, 0, E, stream()) == 0
    ids, w = M.route_reference(logits, K, scoring, b, n_group, topk_group, True, 2.0)
    got_ids = ws.topk_ids.view(T, K).long()
    assert torch.equal(got_ids.sort(-1).values, ids.sort(-1).values)
    assert torch.allclose(ws.topk_w.view(T, K).sort(-1).values, w.sort(-1).values, atol=1e-5, rtol=1e-4)
    assert int(ws.counts.sum()) == T * K
    assert torch.equal(ws.counts.long(), torch.bincount(ids.flatten(), minlength=E))


@pytest.mark.gpu
@pytest.mark.parametrize("T,E,K,H,I,e_begin,e_local", [(64, 8, 2, 256, 128, 0, 8), (300, 128, 8, 2048, 768, 0, 128),
                                                      (5, 128, 8, 2048, 768, 32, 32), (1, 8, 2, 256, 128, 0, 8)])
def test_fused_moe_matches_reference(T, E, K, H, I, e_begin, e_local):
    torch.manual_seed(2)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    logits = torch.randn(T, E, device="cuda")
    w1 = torch.randn(e_local, 2 * I, H, device="cuda", dtype=torch.bfloat16) * 0.05
    w2 = torch.randn(e_local, H, I, device="cuda", dtype=torch.bfloat16) * 0.05
    shared = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    for sh in (None, shared):
        y = M.fused_moe(x, logits, w1, w2, K, expert_begin=e_begin, shared_out=sh)
        ref = M.fused_moe_reference(x, logits, w1, w2, K, expert_begin=e_begin, shared_out=sh)
        err = (y.float() - ref.float()).abs()
        assert bool((err <= 3e-2 + 3e-2 * ref.float().abs()).all()), err.max().item()
    # same workspace reused by a second call (counts are re-zeroed by the offsets kernel)
    ws = M.MoeWorkspace(T, K, E, e_local, H, I, "cuda")
    a = M.fused_moe(x, logits, w1, w2, K, expert_begin=e_begin, ws=ws)
    b = M.fused_moe(x, logits, w1, w2, K, expert_begin=e_begin, ws=ws)
    assert torch.allclose(a.float(), b.float(), atol=2e-2, rtol=2e-2)
