"""Speculative decoding (n-gram drafter + one-pass verification) on the tiny CPU model: the token
stream must be identical to plain greedy decoding, and repetitive text must be accepted in bulk."""
import numpy as np
import torch

from xllm_b200 import LLM, SamplingParams
from xllm_b200.engine.speculative import NgramDrafter


def _llm(**kw):
    return LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=128, max_seqs_per_batch=8,
               max_tokens_per_batch=256, enable_graph=False, enable_schedule_overlap=False, **kw)


def test_ngram_drafter_finds_latest_match():
    d = NgramDrafter(3, max_ngram=3)
    toks = np.array([5, 6, 7, 8, 9, 1, 2, 6, 7, 3, 4, 6, 7], dtype=np.int32)
    assert d.propose_one(toks).tolist() == [3, 4, 6]       # latest "6 7" is followed by 3 4 6
    assert d.propose_one(np.array([1, 2, 3], dtype=np.int32)).tolist() == [3, 3, 3]  # no match: repeat


def test_speculative_greedy_equals_plain_greedy():
    g = torch.Generator().manual_seed(3)
    base = torch.randint(0, 32000, (12,), generator=g).tolist()
    prompts = [base * 3, torch.randint(0, 32000, (40,), generator=g).tolist(), (base[:5] * 6)[:29]]
    sp = SamplingParams(max_tokens=24, temperature=0.0, ignore_eos=True)
    plain = [o.outputs[0].token_ids for o in _llm().generate(prompts, sp)]
    for k in (1, 3):
        llm = _llm(num_speculative_tokens=k)
        outs = llm.generate(prompts, sp)
        assert [o.outputs[0].token_ids for o in outs] == plain
        assert all(len(o.outputs[0].token_ids) == 24 for o in outs)
        assert llm.engine.spec.steps > 0


def test_speculative_accepts_repetition_and_stops_mid_row():
    # a model-free check of the multi-token bookkeeping: a stop token inside an accepted run ends
    # the sequence there and drops the rest of the run
    llm = _llm(num_speculative_tokens=3)
    eng = llm.engine
    prompt = list(range(100, 120))
    eng.add_request("r", prompt, temperature=0.0, max_tokens=50, stop_token_ids=[777], eos_token_id=-1)
    got = []
    while eng.has_unfinished():
        batches = eng.scheduler.schedule()
        if not batches:
            break
        b = batches[0]
        if b.n_prefill > 0:
            evs = eng._finish(eng.runner.execute(b))
        else:
            evs = eng.scheduler.process_output_multi(b.batch_id, np.array([1, 2, 777, 4], dtype=np.int64),
                                                     np.array([4], dtype=np.int32))
        got += [e.token for e in evs if e.token >= 0]
    assert got[1:] == [1, 2, 777] and len(got) == 4


def test_mtp_drafter_on_deepseek_matches_plain_greedy():
    """DeepSeek-style model + its MTP layer as the drafter (own paged KV cache, hidden states of the
    verified rows): the token stream must not depend on whether drafts are accepted."""
    from test_deepseek_cpu import _args
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine

    def make(**kw):
        llm = LLM.__new__(LLM)
        llm.engine = LLMEngine(EngineConfig(model="d", device="cpu", dtype="float32", num_blocks=96, enable_graph=False,
                                            max_tokens_per_batch=24, enable_schedule_overlap=False, **kw), model_args=_args())
        llm.tokenizer = None
        return llm

    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (9, 40, 17)]   # 40 > 24: chunked prefill
    sp = SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True)
    plain = [o.outputs[0].token_ids for o in make().generate(prompts, sp)]
    llm = make(num_speculative_tokens=1, speculative_method="mtp")
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == plain
    spec = llm.engine.spec
    assert spec.steps > 0 and spec.proposed > 0
    assert len(spec.drafter.draft) > 0
    # a drafter that already knows the answer gets everything accepted, so two tokens per step
    llm2 = make(num_speculative_tokens=1, speculative_method="mtp")
    truth = {tuple(p): t for p, t in zip(prompts, plain)}

    class Oracle:
        k = 1
        def propose(self, batch, n, **_):
            out = np.zeros((n, 1), dtype=np.int64)
            for i in range(n):
                h = batch.history(i, 0).tolist()
                for p, t in truth.items():
                    if tuple(h[: len(p)]) == p:
                        j = len(h) - len(p)
                        out[i, 0] = t[j] if j < len(t) else 0
            return out
        def observe(self, *a, **kw): pass
        def after_execute(self, *a, **kw): pass

    llm2.engine.spec.drafter = Oracle()
    got2 = [o.outputs[0].token_ids for o in llm2.generate(prompts, sp)]
    assert got2 == plain and llm2.engine.spec.acceptance_rate > 0.9


def test_mtp_chained_drafts_match_plain_greedy():
    """Three draft tokens per step from one MTP layer chained on its own output: the stream is the
    plain greedy one, and every proposal is k tokens wide."""
    from test_deepseek_cpu import _args
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine

    def make(**kw):
        llm = LLM.__new__(LLM)
        llm.engine = LLMEngine(EngineConfig(model="d", device="cpu", dtype="float32", num_blocks=96, enable_graph=False,
                                            max_tokens_per_batch=24, enable_schedule_overlap=False, **kw), model_args=_args())
        llm.tokenizer = None
        return llm

    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (15, 16, 33)]   # 16: a block boundary
    sp = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    plain = [o.outputs[0].token_ids for o in make().generate(prompts, sp)]
    llm = make(num_speculative_tokens=3, speculative_method="mtp")
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == plain
    d = llm.engine.spec.drafter
    assert d.k == 3 and all(len(v) == 3 for v in d.draft.values())


def test_eagle3_head_drafts_and_stream_is_unchanged():
    """EAGLE-3 head on a tiny dense model: the target exposes three auxiliary hidden states, the head
    drafts two tokens per step over its draft vocabulary (mapped through d2t), and the verified stream
    equals plain greedy decoding."""
    def make(**kw):
        return LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=96, max_seqs_per_batch=8,
                   max_tokens_per_batch=64, enable_graph=False, enable_schedule_overlap=False, **kw)

    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (7, 30, 70)]
    sp = SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True)
    plain = [o.outputs[0].token_ids for o in make().generate(prompts, sp)]
    llm = make(num_speculative_tokens=2, speculative_method="eagle3")
    eng = llm.engine
    H = eng.args.hidden_size
    eng.eagle3.d2t.copy_(torch.full_like(eng.eagle3.d2t, 3))       # draft id d stands for target id d + 3
    eng.eagle3.d2t[-3:] = 0
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == plain
    assert eng.model.last_aux.shape[-1] == 3 * H
    assert eng.spec.steps > 0 and all(len(v) == 2 for v in eng.spec.drafter.draft.values())
    ids = torch.tensor([0, 5, 100])
    assert eng.eagle3.to_target_ids(ids).tolist() == [3, 8, 103]
