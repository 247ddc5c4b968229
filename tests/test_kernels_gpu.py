"""Numerics of every sm_100a kernel against the plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

from xllm_b200 import ops
from xllm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol, rtol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g} (tol {atol})"


@pytest.mark.parametrize("tokens,hidden", [(1, 4096), (7, 4096), (300, 5120), (33, 1024), (5, 7168)])
def test_rmsnorm(tokens, hidden):
    torch.manual_seed(0)
    x = torch.randn(tokens, hidden, device=DEV, dtype=torch.bfloat16)
    w = (torch.randn(hidden, device=DEV) * 0.1 + 1).to(torch.bfloat16)
    y = ops.rmsnorm(x, w, 1e-6)
    yr, _ = ref.rmsnorm(x, w, 1e-6)
    _close(y, yr, 2e-2)
    res = torch.randn_like(x)
    res2 = res.clone()
    y = ops.rmsnorm(x, w, 1e-6, residual=res)
    yr, rr = ref.rmsnorm(x, w, 1e-6, residual=res2)
    _close(res, rr, 1e-2)
    _close(y, yr, 3e-2)


@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_tanh"])
def test_act_and_mul(act):
    torch.manual_seed(1)
    x = torch.randn(37, 2 * 1536, device=DEV, dtype=torch.bfloat16)
    _close(ops.act_and_mul(x, act), ref.act_and_mul(x, act), 2e-2)


@pytest.mark.parametrize("d,rot,interleaved,qk_norm", [(128, 128, False, True), (128, 64, False, False),
                                                      (64, 64, True, False), (64, 64, False, True)])
def test_rope_kv_write(d, rot, interleaved, qk_norm):
    torch.manual_seed(2)
    T, nq, nkv, page, nblocks = 45, 8, 2, 16, 12
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device=DEV, dtype=torch.bfloat16)
    pos = torch.randint(0, 500, (T,), device=DEV)
    cs = ref.build_cos_sin_cache(rot, 512, 1e6, None, DEV)
    qw = (torch.randn(d, device=DEV) * 0.1 + 1).to(torch.bfloat16) if qk_norm else None
    kw = (torch.randn(d, device=DEV) * 0.1 + 1).to(torch.bfloat16) if qk_norm else None
    slots = torch.randperm(nblocks * page, device=DEV)[:T].to(torch.int32)
    slots[3] = -1
    kc = torch.zeros(nblocks, nkv, page, d, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q = ops.rope_kv_write(qkv, nq, nkv, d, pos, cs, rot, slots, kc, vc, qw, kw, 1e-6, interleaved)
    qr, kr, vr = ref.rope_kv(qkv, nq, nkv, d, pos, cs, rot, qw, kw, 1e-6, interleaved)
    kcr, vcr = torch.zeros_like(kc), torch.zeros_like(vc)
    ref.write_kv_cache(kr, vr, kcr, vcr, slots)
    _close(q, qr, 3e-2)
    _close(kc, kcr, 3e-2)
    assert torch.equal(vc, vcr)


def _paged_setup(B, nq, nkv, d, page, lens, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    max_blocks = max((L + page - 1) // page for L in lens) + 1
    nblocks = B * max_blocks + 2
    kc = torch.randn(nblocks, nkv, page, d, device=DEV, dtype=torch.bfloat16, generator=g)
    vc = torch.randn(nblocks, nkv, page, d, device=DEV, dtype=torch.bfloat16, generator=g)
    perm = torch.randperm(nblocks - 1, device=DEV, generator=g)[: B * max_blocks] + 1
    bt = perm.view(B, max_blocks).to(torch.int32)
    return kc, vc, bt


@pytest.mark.parametrize("nq,nkv,d,page", [(32, 8, 128, 16), (8, 8, 128, 16), (16, 2, 64, 32), (40, 2, 128, 64),
                                           (4, 1, 256, 16)])
@pytest.mark.parametrize("splits", [1, 4])
def test_paged_decode_attention(nq, nkv, d, page, splits):
    lens = [1, 17, 200, 555, 64, 1023]
    B = len(lens)
    kc, vc, bt = _paged_setup(B, nq, nkv, d, page, lens)
    q = torch.randn(B, nq, d, device=DEV, dtype=torch.bfloat16)
    sl = torch.tensor(lens, device=DEV, dtype=torch.int32)
    scale = 1 / math.sqrt(d)
    y = ops.paged_decode_attention(q, kc, vc, bt, sl, scale, splits=splits)
    yr = ref.paged_decode_attention(q, kc, vc, bt, sl, scale)
    _close(y, yr, 2e-2)


@pytest.mark.parametrize("d,page,splits,window", [(128, 16, 1, 48), (128, 16, 4, 200), (64, 32, 2, 33), (128, 64, 3, 1)])
def test_paged_decode_attention_sliding_window(d, page, splits, window):
    """Only the last `window` positions count; pages entirely before the window are never read
    (their table entries point at a block full of NaN)."""
    lens = [1, 17, 200, 555, 64, 1023]
    nq, nkv = 8, 2
    B = len(lens)
    kc, vc, bt = _paged_setup(B, nq, nkv, d, page, lens, seed=9)
    q = torch.randn(B, nq, d, device=DEV, dtype=torch.bfloat16)
    sl = torch.tensor(lens, device=DEV, dtype=torch.int32)
    scale = 1 / math.sqrt(d)
    yr = ref.paged_decode_attention(q, kc, vc, bt, sl, scale, window)
    kc[0] = float("nan")
    vc[0] = float("nan")
    for b, n in enumerate(lens):
        dead = max(0, n - window) // page           # pages that end at or before the window start
        bt[b, :dead] = 0
    y = ops.paged_decode_attention(q, kc, vc, bt, sl, scale, splits=splits, window=window)
    assert torch.isfinite(y.float()).all()
    _close(y, yr, 2e-2)


def test_paged_decode_padding_rows_are_zero():
    kc, vc, bt = _paged_setup(3, 8, 2, 128, 16, [40, 40, 40])
    q = torch.randn(3, 8, 128, device=DEV, dtype=torch.bfloat16)
    sl = torch.tensor([40, 0, 7], device=DEV, dtype=torch.int32)
    y = ops.paged_decode_attention(q, kc, vc, bt, sl, 0.1, splits=2)
    assert torch.count_nonzero(y[1]) == 0
    assert torch.isfinite(y.float()).all()


@pytest.mark.parametrize("nq,nkv,d,page", [(8, 2, 128, 16), (4, 4, 64, 32), (16, 2, 128, 128)])
def test_paged_prefill_attention(nq, nkv, d, page):
    q_lens = [5, 64, 130, 1, 257]
    kv_lens = [5, 64, 300, 90, 257]  # third and fourth sequences have cached context
    B = len(q_lens)
    kc, vc, bt = _paged_setup(B, nq, nkv, d, page, kv_lens, seed=4)
    T = sum(q_lens)
    q = torch.randn(T, nq, d, device=DEV, dtype=torch.bfloat16)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device=DEV, dtype=torch.int32)
    kl = torch.tensor(kv_lens, device=DEV, dtype=torch.int32)
    scale = 1 / math.sqrt(d)
    y = ops.paged_prefill_attention(q, kc, vc, bt, cu, kl, max(q_lens), scale)
    yr = ref.paged_attention(q, kc, vc, bt, cu, kl, scale)
    _close(y, yr, 2e-2)
    yw = ops.paged_prefill_attention(q, kc, vc, bt, cu, kl, max(q_lens), scale, window=48)
    ywr = ref.paged_attention(q, kc, vc, bt, cu, kl, scale, window=48)
    _close(yw, ywr, 2e-2)


def test_sample_greedy_and_logprob():
    torch.manual_seed(5)
    logits = torch.randn(9, 151936, device=DEV, dtype=torch.bfloat16)
    ids, _ = ops.sample(logits)
    assert torch.equal(ids, logits.float().argmax(-1))
    ids, lp = ops.sample(logits, want_logprob=True)
    lpr = torch.log_softmax(logits.float(), -1).gather(1, ids[:, None])[:, 0]
    _close(lp, lpr, 1e-3, 1e-3)


def test_sample_topk_topp_support_and_distribution():
    torch.manual_seed(6)
    V, B = 4096, 4
    logits = torch.randn(B, V, device=DEV) * 3
    temp = torch.tensor([0.7, 1.0, 1.3, 0.0], device=DEV)
    top_k = torch.tensor([5, 0, 50, 3], device=DEV, dtype=torch.int32)
    top_p = torch.tensor([1.0, 0.6, 0.9, 1.0], device=DEV)
    probs = ref.filtered_distribution(logits, temp, top_k, top_p)
    counts = torch.zeros(B, V, device=DEV)
    N = 400
    for i in range(N):
        ids, lp = ops.sample(logits, temp, top_k, top_p, seed=11, offset=4 * i, want_logprob=True)
        counts[torch.arange(B), ids] += 1
        assert bool((probs[torch.arange(B), ids] > 0).all()), "sampled a filtered token"
    _close(lp[:3], torch.log(probs[torch.arange(3), ids[:3]]), 1e-3, 1e-3)
    emp = counts / N
    # total variation distance small for the random rows; greedy row is deterministic
    tv = 0.5 * (emp - probs).abs().sum(-1)
    assert bool((tv[:3] < 0.2).all()), tv
    assert emp[3].max().item() == 1.0 and int(emp[3].argmax()) == int(logits[3].argmax())


def test_penalties():
    torch.manual_seed(7)
    logits = torch.randn(3, 1000, device=DEV)
    ids = torch.tensor([[1, 5, 9, -1], [2, 2, -1, -1], [7, 8, 9, 10]], device=DEV, dtype=torch.int32)
    ids[1, 1] = 3
    cnt = torch.tensor([[1, 2, 3, 0], [4, 1, 0, 0], [1, 1, 1, 1]], device=DEV, dtype=torch.int32)
    f = torch.tensor([0.5, 0.0, 0.1], device=DEV)
    p = torch.tensor([0.2, 0.0, 0.0], device=DEV)
    r = torch.tensor([1.0, 1.3, 1.1], device=DEV)
    want = ref.apply_penalties(logits.clone().cpu(), ids.cpu(), cnt.cpu(), f.cpu(), p.cpu(), r.cpu())
    got = ops.apply_penalties(logits.clone(), ids, cnt, f, p, r)
    _close(got.cpu(), want, 1e-5, 1e-5)


def test_embedding_gather_blockcopy_advance():
    torch.manual_seed(8)
    table = torch.randn(1000, 256, device=DEV, dtype=torch.bfloat16)
    ids = torch.randint(0, 1000, (77,), device=DEV)
    assert torch.equal(ops.embedding(ids, table), table[ids])
    part = ops.embedding(ids, table[500:], vocab_start=500)
    want = torch.where((ids >= 500)[:, None], table[ids], torch.zeros_like(table[ids]))
    assert torch.equal(part, want)
    idx = torch.randint(0, 1000, (33,), device=DEV)
    assert torch.equal(ops.gather_rows(table, idx), table[idx])
    cache = torch.randn(2, 10, 4, 16, 64, device=DEV, dtype=torch.bfloat16)  # [layers, blocks, ...]
    want = cache.clone()
    want[:, 7] = want[:, 2]
    want[:, 9] = want[:, 3]
    ptrs = torch.tensor([cache[0].data_ptr(), cache[1].data_ptr()], device=DEV, dtype=torch.int64)
    pairs = torch.tensor([[2, 7], [3, 9]], device=DEV, dtype=torch.int32)
    ops.block_copy(ptrs, 2, pairs, cache[0, 0].numel() * 2)
    assert torch.equal(cache, want)
    toks = torch.tensor([-1, 5, -3], device=DEV)
    ops.resolve_placeholders(toks, torch.tensor([11, 12, 13], device=DEV))
    assert toks.tolist() == [11, 5, 13]


@pytest.mark.parametrize("nq,nkv,page", [(8, 2, 16), (4, 4, 32), (16, 2, 64), (8, 8, 128)])
@pytest.mark.parametrize("impl", ["tcgen05", "legacy"])
def test_paged_prefill_attention_tcgen05_and_legacy(nq, nkv, page, impl, monkeypatch):
    """head_dim 128: the tcgen05/TMEM kernel and the mma.sync kernel against the fp32 reference on
    ragged batches with cached context (chunked prefill), tiles that end inside a page, one-token
    queries and a long sequence with several kv tiles per query tile."""
    monkeypatch.setenv("XLLM_PREFILL_ATTN", impl)
    q_lens = [5, 64, 130, 1, 257, 128, 700]
    kv_lens = [5, 64, 300, 90, 257, 128 + 256, 700 + 3]
    B = len(q_lens)
    kc, vc, bt = _paged_setup(B, nq, nkv, 128, page, kv_lens, seed=9)
    T = sum(q_lens)
    big = torch.randn(T, nq * 128 + 64, device=DEV, dtype=torch.bfloat16)
    q = big[:, : nq * 128].view(T, nq, 128)                      # strided rows, like a slice of the fused QKV output
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device=DEV, dtype=torch.int32)
    kl = torch.tensor(kv_lens, device=DEV, dtype=torch.int32)
    scale = 1 / math.sqrt(128)
    out = torch.zeros(T, nq, 128, device=DEV, dtype=torch.bfloat16)
    for _ in range(2):
        y = ops.paged_prefill_attention(q, kc, vc, bt, cu, kl, max(q_lens), scale, out=out)
    yr = ref.paged_attention(q, kc, vc, bt, cu, kl, scale)
    _close(y, yr, 2e-2)
    from xllm_b200.ops import _lib
    assert _lib.load().xllm_fmha_error_status() == 0
    # a decode-first mixed batch: the prefill kernel only sees the tail of cu_q / kv_lens / block_table
    y2 = ops.paged_prefill_attention(q, kc, vc, bt[2:], cu[2:], kl[2:], max(q_lens), scale, out=torch.zeros_like(out))
    r0 = int(cu[2])
    _close(y2[r0:], yr[r0:], 2e-2)
    assert torch.count_nonzero(y2[:r0]) == 0


@pytest.mark.parametrize("B,nv,dk,dv", [(3, 4, 32, 32), (17, 8, 128, 128), (2, 2, 64, 96), (4, 2, 256, 64), (3, 2, 256, 128),
                                         (2, 3, 48, 40)])
def test_gdn_decode_step_matches_reference(B, nv, dk, dv):
    """Gated-delta-rule state update against the same arithmetic in fp32 tensor ops; the states of
    the slots that are not addressed must stay untouched."""
    from xllm_b200.ops import gdn
    g0 = torch.Generator(device="cuda").manual_seed(B)
    n_slots = B + 3
    state = torch.randn(n_slots, nv, dk, dv, device="cuda", generator=g0) * 0.3
    slots = torch.randperm(n_slots, device="cuda")[:B]
    q = torch.randn(B, nv, dk, device="cuda", generator=g0) * 0.2
    k = torch.nn.functional.normalize(torch.randn(B, nv, dk, device="cuda", generator=g0), dim=-1)
    v = torch.randn(B, nv, dv, device="cuda", generator=g0)
    g = -torch.rand(B, nv, device="cuda", generator=g0)
    beta = torch.rand(B, nv, device="cuda", generator=g0)
    want_S, want_o = gdn.decode_step_reference(state[slots], q, k, v, g, beta)
    before = state.clone()
    out = gdn.decode_step(state, slots, q, k, v, g, beta)
    torch.cuda.synchronize()
    assert torch.allclose(out, want_o, atol=2e-4, rtol=2e-4)
    assert torch.allclose(state[slots], want_S, atol=2e-4, rtol=2e-4)
    rest = torch.ones(n_slots, dtype=torch.bool, device="cuda")
    rest[slots] = False
    assert torch.equal(state[rest], before[rest])


@pytest.mark.parametrize("n,nv,dk,dv,fresh", [(1, 4, 128, 128, True), (37, 8, 128, 128, False), (300, 4, 64, 96, True),
                                               (64, 2, 256, 128, False), (129, 3, 32, 40, False)])
def test_gdn_prefill_matches_the_token_by_token_recurrence(n, nv, dk, dv, fresh):
    """A prompt chunk through the fused-recurrent kernel equals n single-token updates; only the
    addressed slot changes; a fresh sequence ignores what the slot held."""
    from xllm_b200.ops import gdn
    g0 = torch.Generator(device="cuda").manual_seed(n)
    state = torch.randn(5, nv, dk, dv, device="cuda", generator=g0) * 0.3
    slot = 3
    q = torch.randn(n, nv, dk, device="cuda", generator=g0) * 0.2
    k = torch.nn.functional.normalize(torch.randn(n, nv, dk, device="cuda", generator=g0), dim=-1)
    v = torch.randn(n, nv, dv, device="cuda", generator=g0)
    g = -torch.rand(n, nv, device="cuda", generator=g0) * 0.5
    beta = torch.rand(n, nv, device="cuda", generator=g0)
    S0 = torch.zeros_like(state[slot]) if fresh else state[slot].clone()
    want_S, want_o = gdn.prefill_reference(S0, q, k, v, g, beta)
    before = state.clone()
    out = gdn.prefill(state, slot, fresh, q, k, v, g, beta)
    torch.cuda.synchronize()
    assert torch.allclose(out, want_o, atol=1e-3, rtol=1e-3)
    assert torch.allclose(state[slot], want_S, atol=1e-3, rtol=1e-3)
    rest = [i for i in range(5) if i != slot]
    assert torch.equal(state[rest], before[rest])


def test_kernels_do_not_write_outside_their_outputs():
    """Canary rows before and after every output buffer: odd token counts (not multiples of any tile
    size) through norm, activation, gather, GEMM and the state kernel leave the guard rows untouched."""
    from xllm_b200 import ops
    from xllm_b200.ops import gdn
    dev = "cuda"
    g0 = torch.Generator(device=dev).manual_seed(0)

    def guarded(rows, cols, dtype=torch.bfloat16, pad=3):
        buf = torch.full((rows + 2 * pad, cols), 777.0, dtype=dtype, device=dev)
        return buf, buf[pad:pad + rows]

    def intact(buf, rows, pad=3):
        return bool((buf[:pad] == 777.0).all()) and bool((buf[pad + rows:] == 777.0).all())

    for T in (1, 5, 131):
        H = 512
        x = torch.randn(T, H, device=dev, dtype=torch.bfloat16, generator=g0)
        w = torch.ones(H, device=dev, dtype=torch.bfloat16)
        buf, out = guarded(T, H)
        ops.rmsnorm(x, w, 1e-6, out=out)
        assert intact(buf, T) and torch.isfinite(out.float()).all()
        buf, out = guarded(T, H // 2)
        ops.act_and_mul(x, "silu", out=out)
        assert intact(buf, T)
        idx = torch.randint(0, T, (T,), device=dev, generator=g0)
        buf, out = guarded(T, H)
        ops.gather_rows(x, idx, out=out)
        assert intact(buf, T) and torch.equal(out, x[idx])
        wt = torch.randn(384, H, device=dev, dtype=torch.bfloat16, generator=g0) * 0.05
        buf, out = guarded(T, 384)
        ops.linear(x, wt, out=out)
        torch.cuda.synchronize()
        assert intact(buf, T)
        assert torch.allclose(out.float(), x.float() @ wt.float().T, atol=0.08, rtol=0.05)
    B, nv, dk, dv = 5, 3, 32, 48
    state = torch.zeros(B + 2, nv, dk, dv, device=dev)
    state[0] = 777.0
    state[-1] = 777.0
    slots = torch.arange(1, B + 1, device=dev)
    f = lambda *s: torch.randn(*s, device=dev, generator=g0)
    buf, out = guarded(B * nv, dv, torch.float32)
    gdn.decode_step(state, slots, f(B, nv, dk), f(B, nv, dk), f(B, nv, dv), -torch.rand(B, nv, device=dev, generator=g0),
                    torch.rand(B, nv, device=dev, generator=g0), out=out.view(B, nv, dv))
    torch.cuda.synchronize()
    assert intact(buf, B * nv) and bool((state[0] == 777.0).all()) and bool((state[-1] == 777.0).all())


@pytest.mark.parametrize("tokens,hidden", [(3, 256), (129, 2048), (40, 4096), (9, 7168), (2, 16384)])
def test_rmsnorm_row_groups(tokens, hidden):
    """Every thread-group width of the row kernels (32 / 64 / 128 / 256 threads per row), token counts
    that do not fill the last CTA, strided input, and rows the kernel must not touch."""
    torch.manual_seed(3)
    big = torch.randn(tokens + 2, hidden + 64, device=DEV, dtype=torch.bfloat16)
    x = big[1:-1, :hidden]                                   # row stride != hidden
    w = (torch.randn(hidden, device=DEV) * 0.1 + 1).to(torch.bfloat16)
    out = torch.full((tokens + 2, hidden), 7.0, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(tokens, hidden, device=DEV, dtype=torch.bfloat16)
    res0 = res.clone()
    ops.rmsnorm(x, w, 1e-6, residual=res, out=out[1:-1])
    yr, rr = ref.rmsnorm(x, w, 1e-6, residual=res0)
    _close(res, rr, 1e-2)
    _close(out[1:-1], yr, 3e-2)
    assert bool((out[0] == 7).all()) and bool((out[-1] == 7).all())   # canary rows


@pytest.mark.parametrize("tokens,hidden", [(5, 512), (70, 4096), (3, 7168)])
def test_rmsnorm_group_fp8(tokens, hidden):
    """RMSNorm whose output is e4m3 with one scale per (row, 128 columns)."""
    from xllm_b200.ops import fp8 as fp8_ops
    torch.manual_seed(4)
    x = torch.randn(tokens, hidden, device=DEV, dtype=torch.bfloat16) * 3
    w = (torch.randn(hidden, device=DEV) * 0.1 + 1).to(torch.bfloat16)
    res = torch.randn_like(x)
    res0 = res.clone()
    q, sc = fp8_ops.rmsnorm_group_quant(x, w, 1e-6, residual=res)
    yr, rr = ref.rmsnorm(x, w, 1e-6, residual=res0)
    _close(res, rr, 1e-2)
    assert q.dtype == torch.float8_e4m3fn and sc.shape == (tokens, hidden // 128)
    deq = q.float().view(tokens, hidden // 128, 128) * sc[:, :, None]
    want = yr.float().view(tokens, hidden // 128, 128)
    # e4m3 has 3 mantissa bits: half an ulp is 1/16 of the value, plus the bf16 rounding of the norm
    assert bool(((deq - want).abs() <= 0.07 * want.abs() + sc[:, :, None] * 0.6 + 2e-2).all())
    amax = want.abs().amax(-1)
    assert torch.allclose(sc, amax / 448.0, rtol=2e-2, atol=1e-6)


def test_top_logprobs_and_per_row_streams():
    torch.manual_seed(5)
    B, V, n = 9, 5003, 5
    logits = torch.randn(B, V, device=DEV, dtype=torch.float32) * 2
    logits[0, 17] = logits[0, 4000] = 9.0                    # a tie: the lower index comes first
    ids, lp = ops.top_logprobs(logits, n)
    want_lp, want_ids = torch.log_softmax(logits, -1).topk(n, -1)
    assert torch.allclose(lp, want_lp, atol=1e-4)
    assert ids[0, 0].item() == 17 and ids[0, 1].item() == 4000
    assert torch.equal(ids[1:].long(), want_ids[1:])
    idb, lpb = ops.top_logprobs(logits.to(torch.bfloat16), n)
    assert torch.allclose(lpb, torch.log_softmax(logits.to(torch.bfloat16).float(), -1).topk(n, -1)[0], atol=1e-3)
    # a row's draw depends on its own (seed, offset) only: not on its row index nor on its neighbours
    temp = torch.full((B,), 0.9, device=DEV)
    topk = torch.full((B,), 50, device=DEV, dtype=torch.int32)
    topp = torch.full((B,), 0.95, device=DEV)
    seeds = torch.arange(100, 100 + B, device=DEV, dtype=torch.int64)
    offs = torch.arange(B, device=DEV, dtype=torch.int32)
    a, la = ops.sample(logits, temp, topk, topp, seeds=seeds, offsets=offs, want_logprob=True)
    perm = torch.randperm(B, device=DEV)
    b, _ = ops.sample(logits[perm].contiguous(), temp, topk, topp, seeds=seeds[perm].contiguous(),
                      offsets=offs[perm].contiguous())
    assert torch.equal(a[perm], b)
    c, _ = ops.sample(logits, temp, topk, topp, seeds=seeds, offsets=offs + 1)
    assert not torch.equal(a, c)
    # samples come from the filtered distribution
    probs = ref.filtered_distribution(logits.cpu(), temp.cpu(), topk.cpu(), topp.cpu())
    assert bool((probs[torch.arange(B), a.cpu()] > 0).all())
    assert torch.allclose(la.cpu(), torch.log(probs[torch.arange(B), a.cpu()]), atol=2e-3)
