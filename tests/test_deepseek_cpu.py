"""DeepSeek-style MLA + MoE model on CPU against a dense textbook forward (no paging, no padding)."""
import math

import torch

from xllm_b200 import LLM, SamplingParams
from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
from xllm_b200.models import ModelArgs
from xllm_b200.ops import moe as M


def _args():
    return ModelArgs(model_type="deepseek_v3", vocab_size=500, hidden_size=128, num_hidden_layers=3, num_attention_heads=4,
                     num_key_value_heads=4, head_dim=48, intermediate_size=256, num_experts=8, num_experts_per_tok=2,
                     moe_intermediate_size=64, n_shared_experts=1, first_k_dense_replace=1, scoring_func="sigmoid",
                     n_group=4, topk_group=2, routed_scaling_factor=2.5, router_bias=True, q_lora_rank=64, kv_lora_rank=32,
                     qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=24, qk_norm=False, rope_theta=10000.0,
                     max_position_embeddings=256, norm_topk_prob=True, tie_word_embeddings=False)


def _ref_logits(model, ids):
    a = model.args
    sd = dict(model.named_params())
    T = ids.shape[0]
    x = sd["model.embed_tokens.weight"][ids]
    nh, nope, rd, vd = a.num_attention_heads, a.qk_nope_head_dim, a.qk_rope_head_dim, a.v_head_dim
    inv = 1.0 / (a.rope_theta ** (torch.arange(0, rd, 2, dtype=torch.float64) / rd))
    fr = torch.outer(torch.arange(T).double(), inv)
    cos, sin = fr.cos().float(), fr.sin().float()

    def norm(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + a.rms_norm_eps) * w

    def rope(v):  # complex pairs (x0, x1), (x2, x3), ...
        v1, v2 = v[..., 0::2], v[..., 1::2]
        c, s = cos[:, None, :], sin[:, None, :]
        return torch.stack([v1 * c - v2 * s, v2 * c + v1 * s], -1).flatten(-2)

    for i in range(a.num_hidden_layers):
        p = f"model.layers.{i}."
        h = norm(x, sd[p + "input_layernorm.weight"])
        q = norm(h @ sd[p + "self_attn.q_a_proj.weight"].T, sd[p + "self_attn.q_a_layernorm.weight"]) @ sd[p + "self_attn.q_b_proj.weight"].T
        q = q.view(T, nh, nope + rd)
        kva = h @ sd[p + "self_attn.kv_a_proj_with_mqa.weight"].T
        c_kv, k_pe = kva[:, :a.kv_lora_rank], kva[:, a.kv_lora_rank:]
        kv = (norm(c_kv, sd[p + "self_attn.kv_a_layernorm.weight"]) @ sd[p + "self_attn.kv_b_proj.weight"].T).view(T, nh, nope + vd)
        qf = torch.cat([q[..., :nope], rope(q[..., nope:])], -1)
        kf = torch.cat([kv[..., :nope], rope(k_pe[:, None, :]).expand(T, nh, rd)], -1)
        s = torch.einsum("qhd,khd->hqk", qf, kf) / math.sqrt(nope + rd)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), kv[..., nope:]).reshape(T, nh * vd)
        x = x + o @ sd[p + "self_attn.o_proj.weight"].T
        h = norm(x, sd[p + "post_attention_layernorm.weight"])
        if a.is_moe_layer(i):
            logits = h @ sd[p + "mlp.gate.weight"].T
            sh = h @ sd[p + "mlp.shared_experts.gate_up_proj.weight"].T
            g, u = sh.chunk(2, -1)
            shared = (torch.nn.functional.silu(g) * u) @ sd[p + "mlp.shared_experts.down_proj.weight"].T
            y = M.fused_moe_reference(h, logits, sd[p + "mlp.experts.gate_up"], sd[p + "mlp.experts.down"], a.num_experts_per_tok,
                                      "sigmoid", sd[p + "mlp.gate.e_score_correction_bias"], a.n_group, a.topk_group, True,
                                      a.routed_scaling_factor, 0, shared)
        else:
            gu = h @ sd[p + "mlp.gate_up_proj.weight"].T
            g, u = gu.chunk(2, -1)
            y = (torch.nn.functional.silu(g) * u) @ sd[p + "mlp.down_proj.weight"].T
        x = x + y
    return norm(x, sd["model.norm.weight"]) @ sd["lm_head.weight"].T


def test_deepseek_mla_moe_matches_dense_reference():
    args = _args()
    llm = LLM.__new__(LLM)
    llm.engine = LLMEngine(EngineConfig(model="d", device="cpu", dtype="float32", num_blocks=64, enable_graph=False,
                                        max_tokens_per_batch=20, policy="decode_first"), model_args=args)
    llm.tokenizer = None
    model = llm.engine.model
    with torch.no_grad():  # make the routing bias non-trivial
        for n, t in model.named_params():
            if n.endswith("e_score_correction_bias"):
                t.copy_(torch.randn_like(t) * 0.05)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (9, 33, 17)]
    outs = llm.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))
    for p, o in zip(prompts, outs):
        ids = list(p)
        for _ in range(6):
            ids.append(int(_ref_logits(model, torch.tensor(ids))[-1].argmax()))
        assert o.outputs[0].token_ids == ids[len(p):]


def test_fp8_block_checkpoint_stream_is_dequantised():
    from xllm_b200.ops import fp8
    from xllm_b200.utils.loader import dequant_fp8_stream
    w = torch.randn(200, 256) * 0.1
    q, s = fp8.quant_block128_ref(w)
    stream = [("a.weight", q), ("b.weight", torch.ones(3)), ("a.weight_scale_inv", s)]
    got = dict(dequant_fp8_stream(stream))
    assert set(got) == {"a.weight", "b.weight"} and got["a.weight"].dtype == torch.bfloat16
    assert (got["a.weight"].float() - w).abs().max() < 0.03


def test_latent_cache_form_matches_materialised_form():
    """The same weights through both MLA forms, with chunked prefill, a shared prompt prefix served
    from the prefix cache and several sequences decoding together: identical token streams, and a
    cache row of kv_lora_rank + rope values per token instead of per-head K and V."""
    args = _args()

    def make(**kw):
        llm = LLM.__new__(LLM)
        llm.engine = LLMEngine(EngineConfig(model="d", device="cpu", dtype="float32", num_blocks=96, enable_graph=False,
                                            max_tokens_per_batch=24, **kw), model_args=args)
        llm.tokenizer = None
        return llm

    g = torch.Generator().manual_seed(4)
    shared = torch.randint(0, 500, (32,), generator=g).tolist()
    prompts = [shared + torch.randint(0, 500, (n,), generator=g).tolist() for n in (5, 30)] + \
              [torch.randint(0, 500, (n,), generator=g).tolist() for n in (11, 50)]
    sp = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
    a = make()
    b = make(mla_latent_cache=True)
    for (n, t), (_, u) in zip(a.engine.model.named_params(), b.engine.model.named_params()):
        u.copy_(t)
    want = [o.outputs[0].token_ids for o in a.generate(prompts, sp)]
    got = [o.outputs[0].token_ids for o in b.generate(prompts, sp)]
    assert got == want
    again = [o.outputs[0].token_ids for o in b.generate(prompts[:2], sp)]       # now from the prefix cache
    assert again == want[:2]
    ka, kb = a.engine.runner.kv_caches[0][0], b.engine.runner.kv_caches[0][0]
    assert kb.shape[1] == 1 and kb.shape[3] == args.kv_lora_rank + args.qk_rope_head_dim
    assert kb[0].numel() * 1 < ka[0].numel() * 2


def test_fp8_checkpoint_runs_in_fp8_layers_and_matches_dequantised(tmp_path):
    """A block-scaled e4m3 checkpoint (128 x 128 weight blocks) loaded twice: into layers that keep the
    e4m3 weights and their scales (fp8 execution) and dequantised to the wide type at load.  Same
    tokens, logits equal up to rounding."""
    import dataclasses
    import json

    from xllm_b200 import LLM, SamplingParams
    from xllm_b200.models import ModelArgs, create_model
    from xllm_b200.ops import fp8
    from xllm_b200.utils.loader import save_file
    args = ModelArgs(model_type="deepseek_v3", vocab_size=512, hidden_size=256, num_hidden_layers=2,
                     num_attention_heads=4, num_key_value_heads=4, head_dim=48, intermediate_size=256, num_experts=4,
                     num_experts_per_tok=2, moe_intermediate_size=128, n_shared_experts=1, first_k_dense_replace=1,
                     scoring_func="sigmoid", n_group=2, topk_group=1, routed_scaling_factor=2.5, router_bias=True,
                     q_lora_rank=128, kv_lora_rank=128, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32,
                     qk_norm=False, rope_theta=10000.0, max_position_embeddings=512, dtype="float32")
    src = create_model(args, torch.float32, "cpu")
    src.init_random(seed=5)
    tensors = {}
    for name, t in _checkpoint_names(src):
        quantise = "proj" in name and name.endswith(".weight") and t.dim() == 2 and t.shape[1] % 128 == 0
        if quantise:
            q, sc = fp8.quant_block128_ref(t)
            tensors[name] = q
            tensors[name + "_scale_inv"] = sc
        else:
            tensors[name] = t
    d = tmp_path / "ckpt"
    d.mkdir()
    save_file(tensors, str(d / "model.safetensors"))
    cfg = {"model_type": "deepseek_v3", "architectures": ["DeepseekV3ForCausalLM"], "vocab_size": 512, "hidden_size": 256,
           "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 4, "intermediate_size": 256,
           "n_routed_experts": 4, "num_experts_per_tok": 2, "moe_intermediate_size": 128, "n_shared_experts": 1,
           "first_k_dense_replace": 1, "scoring_func": "sigmoid", "n_group": 2, "topk_group": 1,
           "routed_scaling_factor": 2.5, "topk_method": "noaux_tc", "norm_topk_prob": True, "q_lora_rank": 128,
           "kv_lora_rank": 128, "qk_nope_head_dim": 32, "qk_rope_head_dim": 16, "v_head_dim": 32, "rope_theta": 10000.0,
           "max_position_embeddings": 512, "rms_norm_eps": 1e-6, "torch_dtype": "float32", "eos_token_id": 1,
           "quantization_config": {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128]}}
    (d / "config.json").write_text(json.dumps(cfg))
    prompts = [[5, 9, 33, 120, 7, 7, 250], [400, 3, 18]]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    outs = {}
    for mode in (True, False):
        llm = LLM(str(d), devices="cpu", dtype="float32", enable_graph=False, num_blocks=64, max_seqs_per_batch=4,
                  max_tokens_per_batch=64, fp8_execution=mode, tokenizer=_NoTokenizer())
        kinds = {t.dtype for _, t in llm.engine.model.named_params()}
        assert (torch.float8_e4m3fn in kinds) == mode
        outs[mode] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert outs[True] == outs[False], outs


class _NoTokenizer:
    def decode(self, ids, skip_special=True):
        return ""


def _checkpoint_names(model):
    """Parameters under checkpoint names: fused projections and stacked experts split back."""
    a = model.args
    for n, t in model.named_params():
        if n.endswith("gate_up_proj.weight"):
            g, u = t.chunk(2)
            base = n[: -len("gate_up_proj.weight")]
            yield base + "gate_proj.weight", g
            yield base + "up_proj.weight", u
        elif n.endswith("experts.gate_up"):
            base = n[: -len("gate_up")]
            for e in range(t.shape[0]):
                g, u = t[e].chunk(2)
                yield f"{base}{e}.gate_proj.weight", g
                yield f"{base}{e}.up_proj.weight", u
        elif n.endswith("experts.down"):
            base = n[: -len("down")]
            for e in range(t.shape[0]):
                yield f"{base}{e}.down_proj.weight", t[e]
        else:
            yield n, t
