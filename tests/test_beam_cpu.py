"""Beam search on the tiny CPU model: width 1 is greedy decoding; wider beams return distinct,
sorted hypotheses whose scores match a dense recomputation; no KV block is leaked."""
import torch

from xllm_b200 import LLM, SamplingParams
from test_e2e_tiny_cpu import _ref_forward


def _llm():
    return LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=96, max_seqs_per_batch=8,
               max_tokens_per_batch=256, enable_graph=False, enable_prefix_cache=False)


def test_beam_width_one_is_greedy_and_wide_beams_score_right():
    llm = _llm()
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, 32000, (37,), generator=g).tolist()
    greedy = llm.generate([prompt], SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True))[0].outputs[0].token_ids
    one = llm.beam_search([prompt], beam_width=1, max_tokens=10, ignore_eos=True)[0]
    assert one[0].token_ids == greedy
    wide = llm.beam_search([prompt], beam_width=4, max_tokens=10, ignore_eos=True)[0]
    assert len(wide) == 4 and len({tuple(b.token_ids) for b in wide}) == 4
    assert all(wide[i].score >= wide[i + 1].score for i in range(3))
    assert wide[0].cumulative_logprob >= one[0].cumulative_logprob - 1e-4
    model = llm.engine.model
    for b in wide[:2]:
        ids = torch.tensor(prompt + b.token_ids)
        lp = torch.log_softmax(_ref_forward(model, ids).float(), -1)
        want = sum(float(lp[len(prompt) - 1 + i, t]) for i, t in enumerate(b.token_ids))
        assert abs(want - b.cumulative_logprob) < 2e-2, (want, b.cumulative_logprob)
    assert llm.engine.scheduler.block_manager(0).num_used_blocks == 0
