"""Selection kernels (log-softmax, radix top-k, beam step) against fp32 PyTorch references."""
import pytest
import torch

from xllm_b200.ops import select

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,V", [(3, 1000), (9, 151936), (2, 32000)])
def test_log_softmax(dtype, rows, V):
    torch.manual_seed(0)
    x = (torch.randn(rows, V, device=DEV) * 3).to(dtype)
    y = select.log_softmax(x)
    yr = torch.log_softmax(x.float(), -1)
    assert torch.allclose(y, yr, atol=2e-4, rtol=1e-4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,V,k", [(4, 151936, 1), (4, 151936, 20), (3, 32000, 128), (2, 8192, 1024), (2, 40000, 2048), (5, 777, 777),
                                      (2, 65536, 300)])
def test_radix_topk_matches_stable_sort(dtype, rows, V, k):
    torch.manual_seed(1)
    x = torch.randn(rows, V, device=DEV).to(dtype)      # bf16 rows are full of ties: they must go to the lowest index
    for normalize in (False, True):
        v, i = select.topk(x, k, normalize)
        vr, ir = select.topk_reference(x, k, normalize)
        assert torch.equal(i, ir), (dtype, V, k)
        assert torch.allclose(v, vr, atol=2e-4, rtol=1e-4)


def test_radix_topk_with_masked_entries_and_strided_rows():
    torch.manual_seed(2)
    big = torch.randn(6, 40000, device=DEV, dtype=torch.bfloat16)
    x = big[:, :30000]                                   # row stride 40000
    x[:, 100:29000] = float("-inf")
    v, i = select.topk(x, 50)
    vr, ir = select.topk_reference(x, 50)
    assert torch.equal(i, ir) and torch.equal(v, vr)
    x[0, :] = float("-inf")                              # a row without any finite entry still yields k ids
    v, i = select.topk(x, 8)
    assert i[0].tolist() == list(range(8))


@pytest.mark.parametrize("B,W,k,n_out", [(1, 4, 8, 8), (7, 16, 16, 16), (3, 128, 8, 128), (2, 32, 32, 1024)])
def test_beam_step(B, W, k, n_out):
    torch.manual_seed(3)
    lp = torch.log_softmax(torch.randn(B, W, 4096, device=DEV), -1)
    clp, cid = lp.topk(k, dim=-1)
    cum = torch.randn(B, W, device=DEV) * 2
    cum[:, -1] = float("-inf")                           # a dead beam proposes nothing
    tok, par, sc = select.beam_step(clp, cid.to(torch.int32), cum, n_out)
    tr, pr, sr = select.beam_step_reference(clp, cid.to(torch.int32), cum, n_out)
    live = torch.isfinite(sr)
    assert torch.equal(tok[live], tr[live]) and torch.equal(par[live], pr[live])
    assert torch.allclose(sc[live], sr[live], atol=1e-5)
    assert (par[live] != W - 1).all()


def test_beam_topk_end_to_end_equals_flat_topk():
    torch.manual_seed(4)
    W, V = 6, 50000
    logits = (torch.randn(W, V, device=DEV) * 2).to(torch.bfloat16)
    cum = torch.randn(W, device=DEV)
    tok, par, sc = select.beam_topk(logits, cum, 12)
    flat = (torch.log_softmax(logits.float(), -1) + cum[:, None]).flatten()
    top = torch.sort(flat, descending=True, stable=True)
    assert torch.equal(par.long(), top.indices[:12] // V) and torch.equal(tok.long(), top.indices[:12] % V)
    assert torch.allclose(sc, top.values[:12], atol=2e-4)
