"""tcgen05 GEMM against an fp32 PyTorch reference (and cuBLAS bf16 for scale)."""
import pytest
import torch

from xllm_b200.ops import gemm_tcgen05 as g

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (1, 4096, 4096), (7, 1024, 512),
                                   (256, 6144, 4096), (300, 4096, 12288), (1000, 24576, 4096),
                                   (129, 264, 136), (4096, 4096, 4096), (64, 151936, 1024)])
@pytest.mark.parametrize("tile_n,pair", [(0, -1), (256, 0), (64, 0), (256, 1), (128, 1), (64, 1)])
def test_gemm_matches_fp32(M, N, K, tile_n, pair):
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05)
    y = g.gemm_nt(x, w, tile_n=tile_n, pair=pair)
    assert g.error_status() == 0
    ref = x.float() @ w.float().T
    err = (y.float() - ref).abs()
    tol = 2e-2 + 1e-2 * ref.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item()} at M={M} N={N} K={K}"


def test_gemm_bias_and_strided_rows():
    torch.manual_seed(0)
    big = torch.randn(200, 1024 + 64, device="cuda", dtype=torch.bfloat16)
    x = big[:, :1024]  # row stride 1088
    w = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16) * 0.05
    b = torch.randn(512, device="cuda", dtype=torch.bfloat16)
    y = g.gemm_nt(x, w, bias=b)
    ref = x.float() @ w.float().T + b.float()
    assert torch.allclose(y.float(), ref, atol=3e-2, rtol=2e-2)
    assert g.error_status() == 0


@pytest.mark.parametrize("M,N,K", [(8, 4096, 12288), (256, 6144, 4096), (300, 512, 192), (2048, 24576, 4096)])
@pytest.mark.parametrize("tile_n,pair", [(0, -1), (64, 0), (256, 0), (64, 1), (128, 1), (256, 1)])
def test_gemm_packed_weight(M, N, K, tile_n, pair):
    torch.manual_seed(1)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    pw = g.pack_weight(w)
    assert torch.equal(g.unpack_weight(pw), w)
    y = g.gemm_nt(x, pw, tile_n=tile_n, pair=pair)
    ref = x.float() @ w.float().T
    err = (y.float() - ref).abs()
    assert bool((err <= 2e-2 + 1e-2 * ref.abs()).all()), err.max().item()
    assert g.error_status() == 0


@pytest.mark.parametrize("M,N,K", [(8, 4096, 12288), (256, 4096, 4096), (256, 4096, 12288), (300, 6144, 4096),
                                   (129, 264, 1352), (512, 4096, 12288)])
@pytest.mark.parametrize("tile_n,pair,split_k", [(0, -1, 0), (64, 0, 2), (128, 0, 4), (256, 0, 3), (256, 1, 4),
                                                 (128, 1, 8), (64, 1, 16)])
@pytest.mark.parametrize("packed", [False, True])
def test_gemm_split_k(M, N, K, tile_n, pair, split_k, packed):
    """K cut into slices whose fp32 partials meet in the device scratch; run twice so that the
    arrival counters are seen to be left at zero by the first launch."""
    if packed and (N % 64 or K % 64):
        pytest.skip("packed weights need multiples of 64")
    torch.manual_seed(M + N + K + split_k)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ww = g.pack_weight(w) if packed else w
    ref = x.float() @ w.float().T + b.float()
    tol = 3e-2 + 1e-2 * ref.abs()
    for _ in range(2):
        y = g.gemm_nt(x, ww, bias=b, tile_n=tile_n, pair=pair, split_k=split_k)
        assert g.error_status() == 0
        err = (y.float() - ref).abs()
        assert bool((err <= tol).all()), f"max err {err.max().item()}"


@pytest.mark.parametrize("M,N,K", [(8, 1024, 4096), (256, 4096, 4096), (300, 512, 200), (129, 264, 1352)])
@pytest.mark.parametrize("tile_n,pair,split_k", [(64, 0, 1), (128, 0, 1), (128, 0, 3), (64, 1, 1), (128, 1, 2)])
def test_gemm_one_k_block_per_stage(M, N, K, tile_n, pair, split_k):
    """The narrow tiles default to two K blocks per ring stage; the one-block kernels stay covered."""
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    ref = x.float() @ w.float().T
    tol = 3e-2 + 1e-2 * ref.abs()
    g.set_k_per_stage(1)
    try:
        y = g.gemm_nt(x, w, tile_n=tile_n, pair=pair, split_k=split_k)
    finally:
        g.set_k_per_stage(2)
    assert g.error_status() == 0
    assert bool(((y.float() - ref).abs() <= tol).all())


@pytest.mark.parametrize("M,N,K", [(8, 1024, 4096), (256, 4096, 4096), (300, 512, 200), (129, 264, 1352), (64, 512, 64),
                                   (200, 384, 128)])
@pytest.mark.parametrize("tile_n,pair,split_k", [(64, 0, 1), (128, 0, 1), (128, 0, 3), (64, 1, 1), (128, 1, 2)])
@pytest.mark.parametrize("dual", [True, False])
def test_gemm_dual_issue_and_single_issue(M, N, K, tile_n, pair, split_k, dual):
    """Narrow tiles: two MMA-issuing warps with one accumulator each (summed in the epilogue), and
    the single-issuer form of the same kernels; K = 64 / 128 gives units of one ring stage, where
    the second accumulator is never written and must not be read."""
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ref = x.float() @ w.float().T + b.float()
    tol = 3e-2 + 1e-2 * ref.abs()
    g.set_dual_issue(dual)
    try:
        for _ in range(2):
            y = g.gemm_nt(x, w, bias=b, tile_n=tile_n, pair=pair, split_k=split_k)
            assert g.error_status() == 0
            assert bool(((y.float() - ref).abs() <= tol).all())
    finally:
        g.set_dual_issue(False)


@pytest.mark.parametrize("M,N,K", [(8, 24576, 512), (256, 24576, 1024), (300, 600, 320), (512, 4096, 4096), (129, 200, 136)])
@pytest.mark.parametrize("pair,split_k", [(0, 1), (1, 1), (0, 2), (1, 2)])
def test_gemm_192_wide_tiles(M, N, K, pair, split_k):
    """192-column tiles (three 64-column epilogue chunks, 384 of 512 TMEM columns) including ragged N."""
    if pair and M <= 128:
        pytest.skip("pair tiles need more than 128 rows")
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ref = x.float() @ w.float().T + b.float()
    y = g.gemm_nt(x, w, bias=b, tile_n=192, pair=pair, split_k=split_k)
    assert g.error_status() == 0
    assert bool(((y.float() - ref).abs() <= 3e-2 + 1e-2 * ref.abs()).all())
