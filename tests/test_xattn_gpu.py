"""x-attention on a B200: the tcgen05 shared stage with its log-sum-exp output plus the tail-merge kernel,
against the fp32 reference; and the rec engine on the device against exhaustive beam expansion."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(lens, W, n_tail, cap, nq=8, nkv=2, d=128, page=16, seed=0):
    from xllm_b200.ops import xattn
    g = torch.Generator(device="cuda").manual_seed(seed)
    dev = "cuda"
    R = len(lens)
    per = [(n + page - 1) // page for n in lens]
    nb = sum(per) + 1
    kc = torch.randn(nb, nkv, page, d, device=dev, generator=g).to(torch.bfloat16)
    vc = torch.randn(nb, nkv, page, d, device=dev, generator=g).to(torch.bfloat16)
    bt = torch.zeros(R, max(per), dtype=torch.int32, device=dev)
    perm = (torch.randperm(nb - 1, device=dev, generator=g) + 1).to(torch.int32)
    o = 0
    for r in range(R):
        bt[r, : per[r]] = perm[o : o + per[r]]
        o += per[r]
    rows = R * W
    q = (torch.randn(rows, nq, d, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    ku = torch.randn(rows, nkv, cap, d, device=dev, generator=g).to(torch.bfloat16)
    vu = torch.randn(rows, nkv, cap, d, device=dev, generator=g).to(torch.bfloat16)
    anc = torch.stack([torch.randint(0, rows, (rows,), device=dev, generator=g) for _ in range(cap)]).to(torch.int32)
    cu = (torch.arange(R + 1, device=dev) * W).to(torch.int32)
    kv_lens = torch.tensor(lens, dtype=torch.int32, device=dev)
    scale = 1 / math.sqrt(d)
    got = xattn.xattention(q, kc, vc, bt, cu, kv_lens, W, ku, vu, anc, n_tail, scale)
    want = xattn.xattention_reference(q.float(), kc.float(), vc.float(), bt, cu, kv_lens, ku.float(), vu.float(), anc,
                                      n_tail, scale)
    torch.cuda.synchronize()
    return got.float(), want


@pytest.mark.parametrize("lens,W,n_tail", [([300, 57, 1024], 64, 2), ([129], 200, 1), ([16, 2000], 128, 3),
                                           ([40, 41], 5, 0)])
def test_xattention_matches_reference(lens, W, n_tail):
    got, want = _case(lens, W, n_tail, cap=max(n_tail, 1))
    assert torch.isfinite(got).all()
    err = (got - want).abs().max().item()
    assert err < 2e-2, err


def test_rec_engine_on_device_matches_exhaustive_beam():
    from xllm_b200 import LLM
    from xllm_b200.engine.rec import ItemTrie, RecEngine, item_logprob_reference, recommend_reference
    from xllm_b200.ops import launches as launch_count
    llm = LLM("tiny-hd128", devices="cuda:0", dtype="bfloat16", block_size=16, num_blocks=256, max_seqs_per_batch=8,
              max_tokens_per_batch=512, enable_graph=False, enable_prefix_cache=False)
    rec = RecEngine(llm.engine)
    g = torch.Generator().manual_seed(3)
    V = llm.engine.args.vocab_size
    prompts = [torch.randint(0, V, (n,), generator=g).tolist() for n in (70, 23)]
    n0 = launch_count()
    got = rec.generate(prompts, beam_width=6, num_steps=3)
    assert launch_count() > n0
    for p, items in zip(prompts, got):
        want = recommend_reference(llm.engine, p, 6, 3)
        # a random-init model in bf16 ranks many items within rounding of each other, so the check is on scores:
        # every returned item's score is the one a dense forward gives it, and the best score is the oracle's
        assert len(items) == 6 and len({tuple(i.token_ids) for i in items}) == 6
        for it in items:
            assert abs(it.logprob - item_logprob_reference(llm.engine, p, it.token_ids)) < 0.1, it
        assert abs(items[0].logprob - want[0].logprob) < 0.1
        assert all(items[i].logprob >= items[i + 1].logprob for i in range(5))
    items = [tuple(torch.randint(0, V, (3,), generator=g).tolist()) for _ in range(30)]
    got = rec.generate(prompts[:1], beam_width=8, num_steps=3, trie=ItemTrie(items, V))[0]
    assert len(got) == 8 and all(tuple(i.token_ids) in set(items) for i in got)
    assert llm.engine.scheduler.block_manager(0).num_used_blocks == 0
