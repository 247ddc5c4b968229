"""Gated-activation GEMM epilogue and the interleaved activation kernel against fp32 references, and a
dense MLP layer with interleaved weights against the same layer in the plain layout."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,I,K,act", [(1024, 1024, 512, "silu"), (700, 768, 1024, "silu"), (2304, 1536, 4096, "silu"),
                                       (640, 256, 256, "gelu"), (513, 128, 64, "gelu_tanh")])
def test_gemm_act_mul_matches_reference(T, I, K, act):
    from xllm_b200.ops import gemm_tcgen05 as g
    gen = torch.Generator(device="cuda").manual_seed(T)
    x = (torch.randn(T, K, device="cuda", generator=gen) * 0.5).to(torch.bfloat16)
    wg = (torch.randn(I, K, device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(I, K, device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
    w = g.interleave_gate_up(wg, wu).contiguous()
    d0, d1 = g.deinterleave_gate_up(w)
    assert torch.equal(d0, wg) and torch.equal(d1, wu)
    canary = torch.full((T + 8, I + 8), 7.0, device="cuda", dtype=torch.bfloat16)
    out = canary[:T, :I]
    g.gemm_act_mul(x, w, act, out=out)
    f = {"silu": torch.nn.functional.silu, "gelu": torch.nn.functional.gelu,
         "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh")}[act]
    want = f(x.float() @ wg.float().T) * (x.float() @ wu.float().T)
    err = (out.float() - want).abs().max().item()
    assert err < 0.05 + 0.01 * want.abs().max().item(), err
    assert (canary[T:] == 7.0).all() and (canary[:, I:] == 7.0).all()        # nothing written outside the result
    assert g.error_status() == 0
    # the two-launch form over the same interleaved weight
    y = torch.nn.functional.linear(x, w)
    two = g.act_and_mul_interleaved(y, act)
    ref2 = f(y.float().view(T, I // 64, 2, 64)[:, :, 0]) * y.float().view(T, I // 64, 2, 64)[:, :, 1]
    ref2 = ref2.reshape(T, I)
    assert (two.float() - ref2).abs().max() < 0.02 * max(1.0, ref2.abs().max().item())       # bf16 rounding of the output


def test_dense_mlp_interleaved_equals_plain_layout(monkeypatch):
    from xllm_b200.models.layers import DenseMLP
    H, I = 512, 1536
    gen = torch.Generator().manual_seed(0)
    wg, wu, wd = torch.randn(I, H, generator=gen) * 0.05, torch.randn(I, H, generator=gen) * 0.05, torch.randn(H, I, generator=gen) * 0.05
    outs = {}
    for flag in ("1", "0"):
        monkeypatch.setenv("XLLM_FUSED_ACT", flag)
        mlp = DenseMLP(H, I, "silu", torch.bfloat16, "cuda")
        assert mlp.gate_up.interleaved == (flag == "1")
        loaders = dict(mlp.named_loaders())
        loaders["gate_proj.weight"](wg)
        loaders["up_proj.weight"](wu)
        loaders["down_proj.weight"](wd)
        for T in (16, 600, 2500):                      # decode size: two launches; prompt sizes: fused epilogue
            x = (torch.randn(T, H, generator=torch.Generator().manual_seed(T)) * 0.5).to(torch.bfloat16).cuda()
            outs[(flag, T)] = mlp(x).float()
    for T in (16, 600, 2500):
        a, b = outs[("1", T)], outs[("0", T)]
        assert (a - b).abs().max() < 0.02 * max(1.0, b.abs().max().item()), T


@pytest.mark.parametrize("T,E,top_k,H,I", [(300, 8, 2, 512, 256), (1500, 16, 4, 1024, 192), (64, 4, 2, 256, 64)])
def test_fused_moe_interleaved_experts_equal_plain_layout(T, E, top_k, H, I):
    """The grouped GEMM with the gated activation in its epilogue (interleaved expert weights, 256- and
    128-wide tiles) against the three-launch form on the same numbers, and both against the fp32 reference."""
    from xllm_b200.ops import gemm_tcgen05 as g
    from xllm_b200.ops import moe as M
    gen = torch.Generator(device="cuda").manual_seed(T + E)
    x = (torch.randn(T, H, device="cuda", generator=gen) * 0.5).to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda", generator=gen)
    wgu = (torch.randn(E, 2 * I, H, device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E, I, H, device="cuda", generator=gen) * 0.05).to(torch.bfloat16).transpose(1, 2).contiguous()
    wil = g.interleave_gate_up(*wgu.chunk(2, dim=1)).contiguous()
    back = torch.cat(g.deinterleave_gate_up(wil), dim=1)
    assert torch.equal(back, wgu)
    plain = M.fused_moe(x, logits, wgu, wd, top_k)
    fused = M.fused_moe(x, logits, wil, wd, top_k, interleaved=True)
    assert g.error_status() == 0
    assert torch.equal(plain, fused), (plain.float() - fused.float()).abs().max()
    want = M.fused_moe_reference(x.float().cpu(), logits.float().cpu(), wgu.float().cpu(), wd.float().cpu(), top_k)
    assert (fused.float().cpu() - want).abs().max() < 0.05 + 0.02 * want.abs().max()


def test_moe_block_interleaves_on_the_device_and_loads_checkpoint_names(monkeypatch):
    from xllm_b200.models import ModelArgs
    from xllm_b200.models.qwen_moe import SparseMoeBlock as MoEBlock
    args = ModelArgs(model_type="qwen3_moe", vocab_size=1000, hidden_size=256, num_hidden_layers=1, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=64, intermediate_size=512, moe_intermediate_size=128, num_experts=8,
                     num_experts_per_tok=2)
    gen = torch.Generator().manual_seed(0)
    ckpt = {}
    for e in range(8):
        ckpt[f"experts.{e}.gate_proj.weight"] = torch.randn(128, 256, generator=gen) * 0.05
        ckpt[f"experts.{e}.up_proj.weight"] = torch.randn(128, 256, generator=gen) * 0.05
        ckpt[f"experts.{e}.down_proj.weight"] = torch.randn(256, 128, generator=gen) * 0.05
    ckpt["gate.weight"] = torch.randn(8, 256, generator=gen)
    x = (torch.randn(200, 256, generator=gen) * 0.5).to(torch.bfloat16).cuda()
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("XLLM_FUSED_ACT", flag)
        blk = MoEBlock(args, torch.bfloat16, "cuda:0")
        assert blk.interleaved == (flag == "1")
        blk.load_weights(list(ckpt.items()), strict=True)
        outs.append(blk(x))
    assert torch.equal(outs[0], outs[1])
