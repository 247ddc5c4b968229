"""Step-time predictor: exact recovery of a synthetic cost model, budgets, and a live profile of the
tiny CPU engine."""
from xllm_b200 import LLM
from xllm_b200.engine.profile_manager import ProfileManager


def test_fit_and_budgets_on_synthetic_costs():
    pf = lambda n, c: 1e-3 + 2e-6 * n + 1e-10 * (n * n + 2 * n * c)
    dc = lambda b, c: 5e-4 + 1e-5 * b + 2e-9 * b * c
    pm = ProfileManager(pf, dc).profile()
    assert abs(pm.predict_prefill(3000, 100) - pf(3000, 100)) < 1e-6
    assert abs(pm.predict_decode(64, 1000) - dc(64, 1000)) < 1e-7
    budget = pm.token_budget(0.020, decode_batch=64, context_per_seq=1000)
    assert dc(64, 1000) + pf(budget, 0) <= 0.020 < dc(64, 1000) + pf(budget + 64, 0)
    assert pm.token_budget(1e-4) == 0
    b = pm.max_decode_batch(0.002, 1000)
    assert dc(b, 1000) <= 0.002 < dc(b + 1, 1000)


def test_profile_of_a_live_engine():
    llm = LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=128, max_seqs_per_batch=8,
              max_tokens_per_batch=256, enable_graph=False)
    pm = ProfileManager.for_engine(llm.engine, repeats=1).profile(prefill_tokens=(16, 64, 128), decode_batches=(1, 4),
                                                                   contexts=(32, 64))
    assert pm.predict_prefill(128) > 0 and pm.predict_decode(4, 64) > 0
    assert len(pm.samples_prefill) == 6 and len(pm.samples_decode) == 4


def test_engine_applies_profiled_budgets():
    """With latency targets the engine profiles itself at start-up and caps the scheduler's per-step
    tokens and sequences; generation still works, in more (smaller) steps."""
    import torch
    from xllm_b200 import LLM, SamplingParams
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
    kw = dict(model="tiny", device="cpu", dtype="float32", num_blocks=128, enable_graph=False, max_seqs_per_batch=16,
              max_tokens_per_batch=512, max_model_len=512)
    base = LLMEngine(EngineConfig(**kw))
    assert base.profile_manager is None
    # time one 256-token prompt step to pick a target that only smaller steps meet
    from xllm_b200.engine.profile_manager import ProfileManager
    t256 = ProfileManager.for_engine(base, repeats=2).time_prefill(256, 0)
    eng = LLMEngine(EngineConfig(enable_profile_token_budget=True, max_global_ttft_ms=t256 * 1e3 * 0.35,       # far below what a 512-token step takes, whatever the host load
                                 max_global_tpot_ms=1e6, **kw))
    assert eng.profile_manager is not None and len(eng.profile_manager.samples_prefill) >= 6
    b = eng.profiled_budget
    assert eng.cfg.block_size <= b["max_tokens_per_batch"] < 512 and b["max_seqs_per_batch"] == 16
    llm = LLM.__new__(LLM)
    llm.engine, llm.tokenizer = eng, None
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 32000, (300,), generator=g).tolist() for _ in range(2)]
    sp = SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True)
    ref = LLM.__new__(LLM)
    ref.engine, ref.tokenizer = base, None
    want = [o.outputs[0].token_ids for o in ref.generate(prompts, sp)]
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == want
    assert eng.steps > base.steps                  # the capped engine needed more steps for the same prompts
