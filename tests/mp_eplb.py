"""torchrun worker (2+ GPUs): expert re-placement on the GPUs.  A MoE layer with data-parallel tokens
and experts spread over the ranks gets a skewed routing (a few hot experts, all on rank 0); after
`rebalance()` the layer computes the same function, the hot experts are spread over the ranks, and
their weights were pulled from the ranks that held them."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from xllm_b200.models import ModelArgs  # noqa: E402
from xllm_b200.models.qwen_moe import SparseMoeBlock  # noqa: E402
from xllm_b200.parallel.state import init_parallel  # noqa: E402


def main():
    W = int(os.environ["WORLD_SIZE"])
    ps = init_parallel(dp_size=W, ep_size=W)
    ps.max_tokens_per_batch = 512
    dev, r = ps.device, ps.rank
    E, K, H, I = 8 * W, 2, 512, 256
    args = ModelArgs(model_type="qwen3_moe", hidden_size=H, num_experts=E, num_experts_per_tok=K, moe_intermediate_size=I,
                     norm_topk_prob=True, vocab_size=1000, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=4,
                     head_dim=128, intermediate_size=1024)
    blk = SparseMoeBlock(args, torch.bfloat16, dev, ps)
    g = torch.Generator(device=dev).manual_seed(5)          # the same logical model on every rank
    gate = torch.randn(E, H, device=dev, generator=g) * 0.05
    gate[:4] *= 6.0                                          # experts 0..3 (all on rank 0) attract most tokens
    wgu = (torch.randn(E, 2 * I, H, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    El = E // W
    blk.gate.weight.copy_(gate.to(torch.bfloat16))
    blk.w_gate_up.copy_(wgu[r * El:(r + 1) * El])
    blk.w_down.copy_(wd[r * El:(r + 1) * El])
    store = blk.enable_eplb()
    assert blk.w_gate_up.data_ptr() == store.buf.data_ptr()
    gx = torch.Generator(device=dev).manual_seed(100 + r)   # every rank has its own tokens
    xs = [torch.randn(T, H, device=dev, generator=gx).to(torch.bfloat16) for T in (64, 300, 17)]
    before = [blk.forward(x).clone() for x in xs]
    load0 = store.load.clone()
    dist.all_reduce(load0)
    per_rank0 = load0.view(W, El).sum(1)
    assert float(per_rank0[0]) > 1.5 * float(per_rank0.mean()), per_rank0.tolist()
    changed = store.rebalance(min_gain=0.05)
    assert changed and store.placement != list(range(E))
    hot_ranks = {store.placement.index(e) // El for e in range(4)}
    assert len(hot_ranks) > 1, store.placement                    # the hot experts no longer share a rank
    moved = torch.tensor([store.moved_bytes], device=dev, dtype=torch.float64)
    dist.all_reduce(moved)
    assert float(moved.item()) > 0
    after = [blk.forward(x) for x in xs]
    for a, b in zip(before, after):
        assert torch.allclose(a.float(), b.float(), atol=2e-2, rtol=2e-2), float((a.float() - b.float()).abs().max())
    load1 = store.load.clone()
    dist.all_reduce(load1)
    per_rank1 = load1.view(W, El).sum(1)
    imb0 = float(per_rank0.max() / per_rank0.mean())
    imb1 = float(per_rank1.max() / per_rank1.mean())
    assert imb1 < imb0 - 0.05, (imb0, imb1)
    # a second round on balanced loads changes nothing; the layer keeps working through another switch
    assert not store.rebalance(min_gain=0.5)
    assert getattr(ps, "ep_comm").error_status() == 0
    return (f"EPLB_OK world={W} experts={E}: max/mean rank load {imb0:.2f} -> {imb1:.2f}, "
            f"{float(moved.item()) / 2 ** 20:.1f} MiB of expert weights pulled over NVLink")


if __name__ == "__main__":
    from mp_common import guarded
    guarded(main)
