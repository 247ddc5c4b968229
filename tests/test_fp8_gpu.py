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


@pytest.mark.parametrize("M,N,K", [(1, 128, 128), (37, 576, 512), (300, 4096, 7168), (128, 1536, 2048), (130, 264, 1024)])
def test_block_scaled_fp8_gemm(M, N, K):
    """1 x 128 activation scales x 128 x 128 weight scales applied per K block inside the kernel."""
    from xllm_b200.ops import fp8 as f8
    from xllm_b200.ops import gemm_tcgen05
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16) * (1 + 3 * torch.rand(M, 1, device="cuda")).to(torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    w[:, :128] *= 7.0                                   # K blocks with very different scales
    a_q, a_s = f8.quant_group128(x)
    w_q, w_s = f8.quant_block128_ref(w)
    out = torch.full((M + 2, N), 5.0, device="cuda", dtype=torch.bfloat16)
    got = f8.block_scaled_mm(a_q, a_s, w_q, w_s.contiguous(), out=out[1:-1])
    want = f8.block_scaled_mm_ref(a_q, a_s, w_q, w_s)
    err = (got.float() - want.float()).abs()
    assert bool((err <= 2e-2 * want.float().abs() + 2e-2 * want.float().abs().mean() + 1e-3).all()), err.max().item()
    assert bool((out[0] == 5).all()) and bool((out[-1] == 5).all())
    assert gemm_tcgen05.error_status() == 0
    # and against the unquantised product: the error is the quantisation error of e4m3, a few percent
    full = x.float() @ w.float().T
    rel = (got.float() - full).norm() / full.norm()
    assert rel < 0.06, rel.item()


def test_block_scaled_fp8_grouped_gemm():
    from xllm_b200.ops import fp8 as f8
    torch.manual_seed(9)
    E, N, K = 4, 256, 512
    te = torch.tensor([2, 0, -1, 3, 3], device="cuda", dtype=torch.int32)
    rows = te.numel() * 128
    x = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(E, N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    a_q, a_s = f8.quant_group128(x)
    wq, ws = zip(*(f8.quant_block128_ref(w[e]) for e in range(E)))
    w_q, w_s = torch.stack(wq).contiguous(), torch.stack(ws).contiguous()
    out = torch.full((rows, N), 3.0, device="cuda", dtype=torch.bfloat16)
    f8.block_scaled_mm_grouped(a_q, a_s, w_q, w_s, te, out)
    for t, e in enumerate(te.tolist()):
        sl = slice(t * 128, (t + 1) * 128)
        if e < 0:
            assert bool((out[sl] == 3).all())
            continue
        want = f8.block_scaled_mm_ref(a_q[sl], a_s[sl], w_q[e], w_s[e])
        err = (out[sl].float() - want.float()).abs()
        assert bool((err <= 2e-2 * want.float().abs() + 2e-2 * want.float().abs().mean() + 1e-3).all()), (t, err.max().item())


def test_fp8_execution_engine_tracks_dequantised_engine():
    """A DeepSeek-shaped model with random e4m3 weights: executing the linears and the experts on the
    block-scaled fp8 GEMMs gives logits close to the same weights dequantised to bf16."""
    import dataclasses

    from xllm_b200.api.embedding import hidden_states
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
    from xllm_b200.models import ModelArgs, create_model
    from xllm_b200.ops import fp8 as f8
    args = ModelArgs(model_type="deepseek_v3", vocab_size=8000, hidden_size=1024, num_hidden_layers=3,
                     num_attention_heads=16, num_key_value_heads=16, head_dim=192, intermediate_size=2048, num_experts=8,
                     num_experts_per_tok=2, moe_intermediate_size=512, n_shared_experts=1, first_k_dense_replace=1,
                     scoring_func="sigmoid", n_group=2, topk_group=1, routed_scaling_factor=2.5, router_bias=True,
                     q_lora_rank=512, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                     qk_norm=False, rope_theta=10000.0, max_position_embeddings=4096, quant_method="fp8",
                     quant_block=[128, 128])
    m8 = create_model(dataclasses.replace(args, fp8_execution=True, mla_latent_cache=True), torch.bfloat16, "cuda:0")
    m8.init_random(seed=3)
    assert any(t.dtype == torch.float8_e4m3fn for _, t in m8.named_params())
    mw = create_model(dataclasses.replace(args, mla_latent_cache=True), torch.bfloat16, "cuda:0")
    p8 = dict(m8.named_params())
    for n, t in mw.named_params():          # the same weights, dequantised
        src = p8[n]
        if src.dtype == torch.float8_e4m3fn:
            sn = n + "_scale" if "experts." in n and not n.endswith("weight") else n + "_scale_inv"
            sc = p8[sn]
            if src.dim() == 3:
                d = torch.stack([f8.dequant_block128_ref(src[e], sc[e]) for e in range(src.shape[0])])
                if getattr(t, "_xllm_interleaved", False):       # ... and the experts' gate|up rows too
                    from xllm_b200.ops.gemm_tcgen05 import interleave_gate_up
                    d = interleave_gate_up(*d.chunk(2, dim=1))
                t.copy_(d)
            else:
                d = f8.dequant_block128_ref(src, sc)
                if getattr(t, "_xllm_interleaved", False):       # the bf16 model keeps dense gate|up rows interleaved
                    from xllm_b200.ops.gemm_tcgen05 import interleave_gate_up
                    d = interleave_gate_up(*d.chunk(2))
                t.copy_(d)
        else:
            t.copy_(src)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 8000, (200,), generator=g).tolist()

    def logits(model, a):
        eng = LLMEngine(EngineConfig(model="t", device="cuda:0", dtype="bfloat16", block_size=16, num_blocks=64,
                                     max_seqs_per_batch=4, max_tokens_per_batch=256, max_model_len=256, enable_graph=False),
                        model=model, model_args=a)
        return model.logits(hidden_states(eng, ids)).float()

    l8 = logits(m8, dataclasses.replace(args, fp8_execution=True, mla_latent_cache=True))
    lw = logits(mw, dataclasses.replace(args, mla_latent_cache=True))
    rel = float((l8 - lw).abs().mean() / lw.std())
    same = float((l8.argmax(-1) == lw.argmax(-1)).float().mean())
    assert rel < 0.1 and same > 0.7, (rel, same)     # e4m3 activations: a few percent of noise
