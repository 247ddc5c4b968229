"""Worker for test_tp_gpu.py: expert-parallel MoE through the all-to-all kernels against a
single-rank fp32 reference of the same layer."""
import os
import sys

import torch
import torch.distributed as dist

from xllm_b200.ops import moe as moe_ops
from xllm_b200.parallel.ep import EpComm
from xllm_b200.parallel.state import init_parallel


def main():
    ps = init_parallel()
    W, r, dev = ps.world_size, ps.rank, ps.device
    E, K, H, I = 16 * W // 2 if W > 2 else 16, 4, 512, 256
    comm = EpComm(dist.group.WORLD, r, W, dev, E, H, K, max_local_tokens=512)
    El = E // W
    torch.manual_seed(7)  # the same expert weights everywhere; each rank keeps its slice
    wgu = (torch.randn(E, 2 * I, H, device=dev) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device=dev) * 0.05).to(torch.bfloat16)
    my_gu, my_d = wgu[r * El:(r + 1) * El].contiguous(), wd[r * El:(r + 1) * El].contiguous()
    for it, T in enumerate((1, 37, 256, 500)):
        torch.manual_seed(100 * r + it)
        x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
        logits = torch.randn(T, E, device=dev, dtype=torch.float32)
        shared = torch.randn(T, H, device=dev, dtype=torch.bfloat16) if it % 2 else None
        for scoring, kw in (("softmax", {}), ("sigmoid", dict(n_group=4, topk_group=2, scale=2.5))):
            want = moe_ops.fused_moe_reference(x, logits, wgu, wd, K, scoring, None, kw.get("n_group", 1),
                                               kw.get("topk_group", 1), True, kw.get("scale", 1.0), 0, shared)
            got = comm.moe(x, logits, my_gu, my_d, scoring, None, kw.get("n_group", 1), kw.get("topk_group", 1), True,
                           kw.get("scale", 1.0), shared)
            err = (got.float() - want.float()).abs()
            assert bool((err <= 0.06 + 0.03 * want.float().abs()).all()), (T, scoring, err.max().item())
        assert comm.error_status() == 0
    # device-timed: a2a MoE vs the replicate-everything + all-reduce scheme on the same tokens
    T = 512
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    logits = torch.randn(T, E, device=dev, dtype=torch.float32)

    def a2a():
        comm.moe(x, logits, my_gu, my_d)

    xs = [torch.empty_like(x) for _ in range(W)]
    ls = [torch.empty_like(logits) for _ in range(W)]

    def replicate():
        dist.all_gather(xs, x)
        dist.all_gather(ls, logits)
        y = moe_ops.fused_moe(torch.cat(xs), torch.cat(ls), my_gu, my_d, K, expert_begin=r * El, n_experts=E)
        dist.all_reduce(y)

    def timeit(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(10):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ta, tr = timeit(a2a), timeit(replicate)
    assert comm.error_status() == 0
    return f"EP_A2A_OK world={W} E={E} T/rank={T}: a2a {ta * 1e3:.1f} us, replicate+all-reduce {tr * 1e3:.1f} us"


if __name__ == "__main__":
    from mp_common import guarded
    guarded(main)
