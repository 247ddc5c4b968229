"""Prefill/decode disaggregation on the tiny CPU model: a prefill-only engine and a decode-only
engine with separate KV caches must reproduce the single-engine token stream."""
import torch

from xllm_b200 import LLM, SamplingParams
from xllm_b200.engine.disagg import PDCoordinator, make_pd_pair

KW = dict(device="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
          max_tokens_per_batch=128, enable_graph=False, enable_prefix_cache=False)


def test_pd_pair_matches_single_engine():
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (5, 16, 33, 70)]
    llm = LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
              max_tokens_per_batch=128, enable_graph=False)
    want = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0,
                                                                                   ignore_eos=True))]
    p, d = make_pd_pair("tiny", **KW)
    assert p.runner.kv_caches[0][0].data_ptr() != d.runner.kv_caches[0][0].data_ptr()
    pd = PDCoordinator(p, d)
    for i, pr in enumerate(prompts):
        assert pd.add_request(f"r{i}", pr, max_tokens=12, temperature=0.0, ignore_eos=True)
    got = {f"r{i}": [] for i in range(len(prompts))}
    fin = set()

    def on(ev):
        if ev.token >= 0:
            got[ev.request_id].append(ev.token)
        if ev.request_finished:
            fin.add(ev.request_id)

    pd.run_until_done(on)
    assert [got[f"r{i}"] for i in range(len(prompts))] == want
    assert fin == set(got)
    assert pd.transferred_blocks == sum((len(pr) + 15) // 16 for pr in prompts)
    # every block went back on both sides
    assert p.scheduler.block_stats(0).num_used == 0 and d.scheduler.block_stats(0).num_used == 0


def test_pd_decode_side_backpressure():
    """With too few decode blocks for all requests at once the hand-offs queue and drain."""
    p, d = make_pd_pair("tiny", decode_kw=dict(num_blocks=8), **KW)
    pd = PDCoordinator(p, d)
    g = torch.Generator().manual_seed(5)
    for i in range(4):
        pd.add_request(f"q{i}", torch.randint(0, 32000, (40,), generator=g).tolist(), max_tokens=6, temperature=0.0,
                       ignore_eos=True)
    n = {f"q{i}": 0 for i in range(4)}

    def on(ev):
        if ev.token >= 0:
            n[ev.request_id] += 1

    pd.run_until_done(on)
    assert all(v == 6 for v in n.values()), n
