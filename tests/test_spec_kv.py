"""Rejection-sampling verification and the KV push kernel."""
import pytest
import torch

from xllm_b200.engine import kv_transfer as kvt
from xllm_b200.ops import spec


def test_reshard_plan():
    # 8 KV heads, prefill TP=2 -> decode TP=4: source rank 1 owns heads 4..7 = decode ranks 2, 3
    assert kvt.plan_head_slices(2, 1, 4, 8) == [(2, 0, 0, 2), (3, 2, 0, 2)]
    assert kvt.plan_head_slices(4, 3, 2, 8) == [(1, 0, 2, 2)]
    assert kvt.plan_head_slices(1, 0, 1, 8) == [(0, 0, 0, 8)]


def test_verify_reference_greedy():
    p = torch.zeros(1, 4, 10)
    for i, t in enumerate([3, 5, 7, 9]):
        p[0, i, t] = 1.0
    toks, n = spec.verify_reference(torch.tensor([[3, 5, 1]]), p, greedy=torch.tensor([True]))
    assert toks.tolist() == [[3, 5, 7, -1]] and n.tolist() == [3]
    toks, n = spec.verify_reference(torch.tensor([[3, 5, 7]]), p, greedy=torch.tensor([True]))
    assert toks.tolist() == [[3, 5, 7, 9]] and n.tolist() == [4]


@pytest.mark.gpu
def test_verify_kernel_greedy_and_stochastic():
    torch.manual_seed(0)
    B, K, V = 6, 4, 1000
    probs = torch.softmax(torch.randn(B, K + 1, V, device="cuda") * 2, -1)
    am = probs.argmax(-1)
    draft = am[:, :K].clone()
    draft[1, 2] = (draft[1, 2] + 1) % V   # first mismatch at position 2
    draft[3, 0] = (draft[3, 0] + 1) % V
    toks, n = spec.verify(draft, probs, greedy=torch.ones(B, dtype=torch.bool, device="cuda"))
    want, wn = spec.verify_reference(draft.cpu(), probs.cpu(), greedy=torch.ones(B, dtype=torch.bool))
    assert torch.equal(toks.cpu(), want) and torch.equal(n.cpu(), wn)
    # stochastic: q == p accepts everything; a draft token with p = 0 is always rejected and never re-drawn
    q = probs[:, :K].contiguous()
    d = torch.multinomial(q.reshape(-1, V), 1).view(B, K)
    toks, n = spec.verify(d, probs, q, seed=3)
    assert bool((n == K + 1).all()) and torch.equal(toks[:, :K], d)
    p2 = probs.clone()
    p2[:, 0, 7] = 0
    p2[:, 0] /= p2[:, 0].sum(-1, keepdim=True)
    d2 = torch.full((B, K), 7, device="cuda")
    firsts = []
    for it in range(50):
        toks, n = spec.verify(d2, p2, None, seed=11, offset=4 * it)
        assert bool((n == 1).all()) and bool((toks[:, 0] != 7).all()) and bool((toks[:, 1:] == -1).all())
        firsts.append(toks[:, 0])
    # the recovered sample follows p (support check: only tokens with p > 0)
    f = torch.stack(firsts)
    assert bool((p2[:, 0].gather(1, f.T.contiguous()) > 0).all())


@pytest.mark.gpu
def test_kv_push_and_wait_same_device():
    torch.manual_seed(1)
    L, nb, nkv, page, d = 3, 10, 4, 16, 128
    src = [(torch.randn(nb, nkv, page, d, device="cuda", dtype=torch.bfloat16),
            torch.randn(nb, nkv, page, d, device="cuda", dtype=torch.bfloat16)) for _ in range(L)]
    dst = [(torch.zeros(nb, nkv, page, d, device="cuda", dtype=torch.bfloat16),
            torch.zeros(nb, nkv, page, d, device="cuda", dtype=torch.bfloat16)) for _ in range(L)]
    flags = torch.zeros(L, dtype=torch.int32, device="cuda")
    status = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    pusher = kvt.KVPusher(src, page, "cuda")
    target = kvt.PushTarget([(k.data_ptr(), v.data_ptr()) for k, v in dst], pusher.block_bytes, flags.data_ptr())
    pairs = torch.tensor([[1, 5], [2, 7], [9, 3]], dtype=torch.int32, device="cuda")
    pusher.push_all(pairs, target, epoch=1)
    kvt.wait_layer(flags, L - 1, 1, status)
    torch.cuda.synchronize()
    assert status.item() == 0 and flags.tolist() == [1, 1, 1]
    for l in range(L):
        for w in (0, 1):
            for s, t in pairs.tolist():
                assert torch.equal(dst[l][w][t], src[l][w][s])
            assert torch.count_nonzero(dst[l][w][0]) == 0
    # a flag that nothing sets: the bounded wait gives up and reports it (no hang)
    kvt.wait_layer(flags, 0, 5, status, budget_cycles=2_000_000)
    torch.cuda.synchronize()
    assert status.item() == 1
    # head re-slicing: only heads 2..3 of the source go to heads 0..1 of a 2-head destination cache
    dst2 = torch.zeros(nb, 2, page, d, device="cuda", dtype=torch.bfloat16)
    t2 = kvt.PushTarget([(dst2.data_ptr(), dst2.data_ptr())] * L, 2 * pusher.head_bytes, flags.data_ptr(), head0=0)
    pusher.push_layer(0, pairs, t2, epoch=2, src_head0=2, n_heads=2)
    torch.cuda.synchronize()
    assert torch.equal(dst2[5], src[0][1][1][2:4])
