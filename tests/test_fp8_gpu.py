"""fp8 quantisation kernels and the tcgen05 e4m3 scaled GEMM against PyTorch references."""
import pytest
import torch

from xllm_b200.ops import fp8

pytestmark = pytest.mark.gpu


def test_quant_kernels_match_reference():
    torch.manual_seed(0)
    x = torch.randn(37, 1024, device="cuda", dtype=torch.bfloat16) * 3
    q, s = fp8.quant_per_token(x)
    qr, sr = fp8.quant_per_token_ref(x)
    assert torch.allclose(s, sr, rtol=1e-6) and torch.allclose(q.float(), qr.float(), atol=0, rtol=0.07)
    st = torch.tensor([0.05], device="cuda")
    q2, _ = fp8.quant_per_token(x, st)
    assert torch.allclose(q2.float(), fp8.quant_per_token_ref(x, st)[0].float(), rtol=0.07, atol=1e-3)
    qg, sg = fp8.quant_group128(x)
    qgr, sgr = fp8.quant_group128_ref(x)
    assert torch.allclose(sg, sgr, rtol=1e-6) and torch.allclose(qg.float(), qgr.float(), rtol=0.07, atol=0)
    w = torch.randn(300, 512, device="cuda") * 0.1
    wq, ws = fp8.quant_block128_ref(w)
    assert torch.equal(fp8.dequant_block128(wq, ws), fp8.dequant_block128_ref(wq, ws))
    assert (fp8.dequant_block128(wq, ws).float() - w).abs().max() < 0.03


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (7, 512, 1024), (300, 4096, 4096), (2048, 6144, 4096), (130, 264, 144)])
@pytest.mark.parametrize("per_row,per_col", [(False, False), (True, True)])
def test_scaled_mm(M, N, K, per_row, per_col):
    torch.manual_seed(M + N)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    if per_row:
        aq, a_s = fp8.quant_per_token(a)
    else:
        a_s = (a.float().abs().max() / 448).reshape(1)
        aq, _ = fp8.quant_per_token(a, a_s)
    if per_col:
        wq, w_s = fp8.quant_per_token(w)
    else:
        w_s = (w.float().abs().max() / 448).reshape(1)
        wq, _ = fp8.quant_per_token(w, w_s)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    y = fp8.scaled_mm(aq, wq, a_s, w_s, bias)
    ref = (aq.float() * a_s.reshape(-1, 1)) @ (wq.float() * w_s.reshape(-1, 1)).T + bias.float()
    err = (y.float() - ref).abs()
    assert bool((err <= 3e-2 + 1e-2 * ref.abs()).all()), err.max().item()
