"""sleep / wake_up: memory is released, and generation after wake-up (including a request that was
running when the instance went to sleep) gives the same tokens."""
import torch

from xllm_b200 import LLM, SamplingParams


def test_sleep_levels_and_resume():
    llm = LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=4,
              max_tokens_per_batch=128, enable_graph=False)
    eng = llm.engine
    g = torch.Generator().manual_seed(0)
    p = torch.randint(0, 32000, (30,), generator=g).tolist()
    sp = SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True)
    want = llm.generate([p], sp)[0].outputs[0].token_ids
    for level in (1, 2):
        eng.add_request(f"mid{level}", p, temperature=0.0, max_tokens=10, ignore_eos=True)
        for _ in range(4):                       # prefill + a few decode steps, then sleep mid-request
            eng.step()
        llm.sleep(level)
        assert all(c is None for c in eng.runner.kv_caches)
        if level == 2:
            assert all(t.numel() == 0 for _, t in eng.model.named_params())
        assert not eng.step()                    # a sleeping engine schedules nothing
        llm.wake_up()
        got = []
        while eng.has_unfinished():
            got += [e.token for e in eng.step() if e.token >= 0 and e.request_id == f"mid{level}"]
        # tokens produced before the sleep were already delivered; the rest continue the same stream
        assert want[-len(got):] == got and 0 < len(got) <= 10
        assert llm.generate([p], sp)[0].outputs[0].token_ids == want
