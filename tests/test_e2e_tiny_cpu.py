"""Tiny Qwen3-style decoder on CPU (fp32) through the whole stack, checked against a plain
PyTorch forward that recomputes the full sequence with dense causal attention at every step."""
import math

import torch

from xllm_b200 import LLM, SamplingParams
from xllm_b200.models import preset


def _ref_forward(model, ids):
    """Dense reference: no paging, no KV cache, textbook ops."""
    a = model.args
    sd = dict(model.named_params())
    x = sd["model.embed_tokens.weight"][ids]
    T = ids.shape[0]
    d, nq, nkv = a.head_dim, a.num_attention_heads, a.num_key_value_heads
    pos = torch.arange(T)
    inv = 1.0 / (a.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
    fr = torch.outer(pos.double(), inv)
    cos, sin = fr.cos().float()[:, None, :], fr.sin().float()[:, None, :]

    def norm(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + a.rms_norm_eps) * w

    def rope(v):
        v1, v2 = v[..., : d // 2], v[..., d // 2:]
        return torch.cat([v1 * cos - v2 * sin, v2 * cos + v1 * sin], -1)

    for i in range(a.num_hidden_layers):
        p = f"model.layers.{i}."
        h = norm(x, sd[p + "input_layernorm.weight"])
        qkv = h @ sd[p + "self_attn.qkv_proj.weight"].T
        q, k, v = qkv.split([nq * d, nkv * d, nkv * d], -1)
        q = rope(norm(q.view(T, nq, d), sd[p + "self_attn.q_norm.weight"]))
        k = rope(norm(k.view(T, nkv, d), sd[p + "self_attn.k_norm.weight"]))
        v = v.view(T, nkv, d)
        k = k.repeat_interleave(nq // nkv, 1)
        v = v.repeat_interleave(nq // nkv, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(d)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(T, nq * d)
        x = x + o @ sd[p + "self_attn.o_proj.weight"].T
        h = norm(x, sd[p + "post_attention_layernorm.weight"])
        gu = h @ sd[p + "mlp.gate_up_proj.weight"].T
        g, u = gu.chunk(2, -1)
        x = x + (torch.nn.functional.silu(g) * u) @ sd[p + "mlp.down_proj.weight"].T
    x = norm(x, sd["model.norm.weight"])
    return x @ sd["model.embed_tokens.weight"].T


def _make_prompts(seed=0, n=4):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(16, 65, (n,), generator=g).tolist()
    return [torch.randint(0, 32000, (L,), generator=g).tolist() for L in lens]


def test_tiny_greedy_matches_dense_reference():
    llm = LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
              max_tokens_per_batch=256, enable_graph=False)
    prompts = _make_prompts()
    outs = llm.generate(prompts, SamplingParams(max_tokens=32, temperature=0.0, ignore_eos=True))
    model = llm.engine.model
    for p, o in zip(prompts, outs):
        ids = list(p)
        for _ in range(32):
            logits = _ref_forward(model, torch.tensor(ids))
            ids.append(int(logits[-1].argmax()))
        assert o.outputs[0].token_ids == ids[len(p):]
        assert o.outputs[0].finish_reason == "length"
        assert o.finished


def test_tiny_chunked_prefill_and_overlap_match_plain():
    prompts = _make_prompts(seed=3, n=5)
    sp = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    base = LLM("tiny", devices="cpu", dtype="float32", num_blocks=128, enable_graph=False,
               enable_prefix_cache=False).generate(prompts, sp)
    for kw in (dict(max_tokens_per_batch=24, policy="decode_first"),
               dict(enable_schedule_overlap=True),
               dict(max_tokens_per_batch=40, enable_schedule_overlap=True, policy="decode_first"),
               dict(enable_prefix_cache=True)):
        args = dict(num_blocks=128, enable_graph=False, enable_prefix_cache=False)
        args.update(kw)
        got = LLM("tiny", devices="cpu", dtype="float32", **args).generate(prompts, sp)
        for a, b in zip(base, got):
            assert a.outputs[0].token_ids == b.outputs[0].token_ids, kw


def test_prefix_cache_hit_and_n_samples():
    llm = LLM("tiny", devices="cpu", dtype="float32", num_blocks=128, enable_graph=False)
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, 32000, (48,), generator=g).tolist()
    sp = SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True)
    first = llm.generate([shared + [5, 6, 7]], sp)[0]
    second = llm.generate([shared + [9, 10]], sp)[0]
    assert first.usage.num_cached_tokens == 0
    assert second.usage.num_cached_tokens == 48
    # n = 3 greedy samples of one prompt are identical and share the prompt blocks
    o = llm.generate([shared], SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True, n=3))[0]
    assert len(o.outputs) == 3
    assert o.outputs[0].token_ids == o.outputs[1].token_ids == o.outputs[2].token_ids
    assert llm.stats()["kv_utilization"] == 0.0
