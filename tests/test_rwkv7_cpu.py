"""RWKV-7: the recurrence against an independent statement of its formulas, and the engine's state
handling (chunked prompts, batches, slot reuse) against token-by-token evaluation."""
import torch
import torch.nn.functional as F

from xllm_b200 import LLM, SamplingParams
from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
from xllm_b200.models import ModelArgs
from xllm_b200.models.config import model_args_from_dict
from xllm_b200.models.rwkv7 import Rwkv7CausalLM, TimeMix


def _args():
    return ModelArgs(model_type="rwkv7", vocab_size=512, hidden_size=64, num_hidden_layers=3, num_attention_heads=4,
                     num_key_value_heads=4, head_dim=16, intermediate_size=256, tie_word_embeddings=False,
                     max_position_embeddings=512,
                     extra={"decay_low_rank_dim": 8, "a_low_rank_dim": 8, "v_low_rank_dim": 6, "gate_low_rank_dim": 12})


def test_config_defaults():
    a = model_args_from_dict({"model_type": "rwkv7", "hidden_size": 768, "num_hidden_layers": 12, "vocab_size": 65536,
                              "head_size": 64})
    assert a.num_attention_heads == 12 and a.head_dim == 64 and a.intermediate_size == 3072


def test_time_mix_matches_the_formulas_written_out_per_head():
    torch.manual_seed(0)
    args = _args()
    tm = TimeMix(args, 1, torch.float32, "cpu")
    for _, p in tm.named_params():
        p.copy_(torch.randn_like(p) * 0.3)
    T, C, H, N = 7, 64, 4, 16
    x = torch.randn(T, C)
    shift = torch.randn(C)
    S0 = torch.randn(H, N, N) * 0.1
    v_first = torch.randn(T, C)
    out, last, S1, _ = tm.forward(x, shift, S0, v_first)
    # the same, scalar by scalar over heads
    P = {n: t for n, t in tm.named_params()}
    prev = torch.cat([shift[None], x[:-1]])
    mix = lambda n: x + (prev - x) * P[n].view(C)
    r = mix("x_r") @ P["receptance.weight"].T
    k = mix("x_k") @ P["key.weight"].T
    v = mix("x_v") @ P["value.weight"].T
    w = torch.exp(-torch.exp(F.logsigmoid(P["w0"].view(C) + torch.tanh(mix("x_w") @ P["w1"]) @ P["w2"]) - 0.5))
    a = torch.sigmoid(P["a0"].view(C) + mix("x_a") @ P["a1"] @ P["a2"])
    g = torch.sigmoid(mix("x_g") @ P["g1"]) @ P["g2"]
    v = v + (v_first - v) * torch.sigmoid(P["v0"].view(C) + mix("x_v") @ P["v1"] @ P["v2"])
    y = torch.zeros(T, C)
    S = S0.clone()
    rkv = torch.zeros(T, C)
    for t in range(T):
        for h in range(H):
            sl = slice(h * N, (h + 1) * N)
            kk = k[t, sl] * P["k_k"].view(C)[sl]
            kk = kk / kk.norm().clamp_min(1e-12)
            k2 = k[t, sl] * (1 + (a[t, sl] - 1) * P["k_a"].view(C)[sl])
            Sh = S[h]
            Sh = Sh * w[t, sl][None, :] - (Sh @ kk)[:, None] * (kk * a[t, sl])[None, :] + v[t, sl][:, None] * k2[None, :]
            S[h] = Sh
            y[t, sl] = Sh @ r[t, sl]
            rkv[t, sl] = (r[t, sl] * k2 * P["r_k"][h]).sum() * v[t, sl]
    yn = F.group_norm(y, H, P["ln_x.weight"], P["ln_x.bias"], tm.gn_eps)
    want = ((yn + rkv) * g) @ P["output.weight"].T
    assert torch.allclose(out, want, atol=2e-4, rtol=1e-4), float((out - want).abs().max())
    assert torch.allclose(S1, S, atol=1e-5) and torch.equal(last, x[-1])


def _engine(**kw):
    llm = LLM.__new__(LLM)
    llm.engine = LLMEngine(EngineConfig(model="r", device="cpu", dtype="float32", num_blocks=64, enable_graph=False,
                                        enable_prefix_cache=False, **kw), model_args=_args())
    llm.tokenizer = None
    return llm


def test_engine_state_handling_is_independent_of_chunking_and_batching():
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (5, 37, 18, 50)]
    sp = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
    one = _engine(max_seqs_per_batch=1, max_tokens_per_batch=256)
    want = [one.generate([p], sp)[0].outputs[0].token_ids for p in prompts]          # one sequence at a time, whole prompts
    assert isinstance(one.engine.model, Rwkv7CausalLM)
    batched = _engine(max_seqs_per_batch=8, max_tokens_per_batch=256)
    assert [o.outputs[0].token_ids for o in batched.generate(prompts, sp)] == want
    chunked = _engine(max_seqs_per_batch=3, max_tokens_per_batch=16)                  # prompts in 16-token chunks, slots reused
    assert [o.outputs[0].token_ids for o in chunked.generate(prompts, sp)] == want
    assert not chunked.engine.model.state.owner                                       # every slot came back
    # token by token through the model equals the whole prompt at once
    m = one.engine.model
    from xllm_b200.api.embedding import hidden_states
    seq = prompts[1] + want[1]
    h_all = hidden_states(one.engine, seq)
    assert h_all.shape == (len(seq), 64) and torch.isfinite(h_all).all()
    assert m.logits(h_all[len(prompts[1]) - 1:len(prompts[1])]).argmax(-1).item() == want[1][0]
