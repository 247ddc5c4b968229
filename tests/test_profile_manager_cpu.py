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
