"""Admission rules and the sliding-window block release of the C++ scheduler, driven through the
engine on the tiny CPU model: zero-eviction admission never preempts, fixed-steps runs waves,
windowed models give dead KV blocks back while they run."""
import dataclasses

import torch

from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
from xllm_b200.models.config import preset

KW = dict(model="tiny", device="cpu", dtype="float32", block_size=16, max_seqs_per_batch=8, max_tokens_per_batch=128,
          enable_graph=False, enable_prefix_cache=False)


def _run(eng, prompts, max_tokens, arrivals=None):
    """Drive the engine by hand; `arrivals[i]` = step at which prompt i is added (default 0)."""
    arrivals = arrivals or [0] * len(prompts)
    got = {i: [] for i in range(len(prompts))}
    first_step = {}
    done_step = {}
    step = 0
    added = set()
    while len(done_step) < len(prompts) and step < 2000:
        for i, a in enumerate(arrivals):
            if a <= step and i not in added:
                assert eng.add_request(f"r{i}", prompts[i], max_tokens=max_tokens, temperature=0.0, ignore_eos=True)
                added.add(i)
        evs = eng.step() if eng.has_unfinished() else []
        if not eng.scheduler.has_unfinished():
            evs = evs + eng.drain()
        for ev in evs:
            i = int(ev.request_id[1:])
            if ev.token >= 0:
                got[i].append(int(ev.token))
                first_step.setdefault(i, step)
            if ev.request_finished:
                done_step[i] = step
        step += 1
    return [got[i] for i in range(len(prompts))], first_step, done_step


def _prompts(n, length, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 32000, (length,), generator=g).tolist() for _ in range(n)]


def test_zero_eviction_never_preempts_where_continuous_does():
    prompts = _prompts(6, 40)
    # 6 x (40 + 60) tokens = 42 blocks of 16 at the end; the pool has 23 usable ones
    base = LLMEngine(EngineConfig(num_blocks=24, **KW))
    want, _, _ = _run(base, prompts, 60)
    assert base.scheduler.num_preemptions > 0                       # the plain scheduler over-admits and evicts
    ze = LLMEngine(EngineConfig(num_blocks=24, scheduler_type="zero_eviction", **KW))
    got, _, _ = _run(ze, prompts, 60)
    assert ze.scheduler.num_preemptions == 0
    assert ze.scheduler.num_admission_refusals > 0                   # some requests had to wait their turn
    assert got == want
    assert ze.scheduler.block_stats(0).num_used == 0


def test_zero_eviction_rejects_what_can_never_fit():
    ze = LLMEngine(EngineConfig(num_blocks=4, scheduler_type="zero_eviction", **KW))
    got, _, done = _run(ze, _prompts(1, 40), 60)                     # needs 7 blocks, 3 exist
    assert got == [[]] and 0 in done


def test_fixed_steps_runs_waves():
    prompts = _prompts(4, 20, seed=3)
    eng = LLMEngine(EngineConfig(num_blocks=64, scheduler_type="fixed_steps", **KW))
    got, first, done = _run(eng, prompts, 3, arrivals=[0, 0, 1, 1])
    assert all(len(t) == 3 for t in got)
    # requests 2 and 3 arrived while the first wave ran: they start only after it has finished
    assert min(first[2], first[3]) > max(done[0], done[1])
    assert first[0] == first[1] and first[2] == first[3]
    ref = LLMEngine(EngineConfig(num_blocks=64, **KW))
    want, first_c, done_c = _run(ref, prompts, 3, arrivals=[0, 0, 1, 1])
    assert got == want
    assert min(first_c[2], first_c[3]) <= max(done_c[0], done_c[1])  # the continuous scheduler mixes them in


def test_sliding_window_gives_blocks_back_and_keeps_the_tokens():
    args = dataclasses.replace(preset("tiny"), sliding_window=40)
    prompts = _prompts(3, 90, seed=5)
    eng = LLMEngine(EngineConfig(num_blocks=64, **KW), model_args=args)
    assert eng.scheduler is not None
    got, _, _ = _run(eng, prompts, 40)
    assert eng.scheduler.num_window_released_blocks > 0
    assert eng.scheduler.block_stats(0).num_used == 0
    # the same model over a scheduler that keeps every block: identical tokens, more blocks in use
    keep = LLMEngine(EngineConfig(num_blocks=64, **KW), model=eng.model, model_args=dataclasses.replace(args))
    want, _, _ = _run(_without_release(keep), prompts, 40)
    assert got == want
    # 3 x 130 tokens need 27 blocks at the end, the prompts 18 at once; 19 usable blocks are enough
    # only because blocks behind the window come back
    peak = LLMEngine(EngineConfig(num_blocks=20, **KW), model=eng.model, model_args=args)
    got2, _, _ = _run(peak, prompts, 40)
    assert got2 == want and peak.scheduler.num_preemptions == 0
    tight = _without_release(LLMEngine(EngineConfig(num_blocks=20, **KW), model=eng.model, model_args=args))
    _run(tight, prompts, 40)
    assert tight.scheduler.num_preemptions > 0


def _without_release(engine):
    """Rebuild the engine's scheduler with sliding_window = 0 (blocks are kept; the attention
    kernels still apply the window)."""
    rt = engine.rt
    sc = rt.SchedulerConfig()
    cfg = engine.cfg
    sc.max_tokens_per_batch = cfg.max_tokens_per_batch
    sc.max_seqs_per_batch = cfg.max_seqs_per_batch
    sc.enable_chunked_prefill = True
    sc.enable_prefix_cache = False
    sc.block_size = cfg.block_size
    sc.num_blocks = engine.num_blocks
    sc.policy = cfg.policy
    sc.sliding_window = 0
    engine.scheduler = rt.Scheduler(sc)
    return engine
