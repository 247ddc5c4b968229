"""Worker for test_tp_gpu.py: row-parallel GEMM fused with reduce-scatter (+ residual + RMSNorm +
all-gather) against torch matmul + torch.distributed all-reduce, and a device-timed comparison."""
import os
import sys

import torch
import torch.distributed as dist

from xllm_b200 import ops
from xllm_b200.ops import gemm_tcgen05
from xllm_b200.ops import reference as ref
from xllm_b200.parallel import symm
from xllm_b200.parallel.state import init_parallel


def main():
    ps = init_parallel()
    W, r, dev = ps.world_size, ps.rank, ps.device
    H = 4096
    comm = symm.attach(ps, 8192, H)
    assert comm is not None
    for T, K in ((1, 512), (7, 512), (300, 1536), (1000, 1024), (4096, 1536)):
        torch.manual_seed(100 + T)  # same residual / norm weight on every rank
        res_full = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
        nw = (torch.randn(H, device=dev) * 0.1 + 1).to(torch.bfloat16)
        torch.manual_seed(1000 * r + T)  # this rank's operands
        x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(H, K, device=dev, dtype=torch.bfloat16) * 0.05
        part = (x.float() @ w.float().T).to(torch.bfloat16).float()  # partials cross the link as bf16
        total = part.clone()
        dist.all_reduce(total)
        for tile_n in (128, 256):
            got = comm.gemm_rs_norm(x, w, None, None, 0.0, tile_n=tile_n).clone()
            err = (got.float() - total).abs()
            assert bool((err <= 0.08 + 0.02 * total.abs()).all()), (T, tile_n, err.max().item())
        b, e, S = comm.shard(T)
        shard = torch.zeros(S, H, device=dev, dtype=torch.bfloat16)
        shard[: e - b] = res_full[b:e]
        for it in range(2):
            want_res = (total + res_full.float()).to(torch.bfloat16)
            want, _ = ref.rmsnorm(want_res, nw, 1e-6)
            got = comm.gemm_rs_norm(x, w, shard, nw, 1e-6).clone()
            assert torch.allclose(shard[: e - b].float(), want_res[b:e].float(), atol=0.1, rtol=0.03), T
            assert torch.allclose(got.float(), want.float(), atol=0.1, rtol=0.04), (T, (got.float() - want.float()).abs().max())
            res_full = want_res
            # the barrier-based kernel shares epochs and buffers with the push-based pair
            comm.partial_buffer(T).copy_(part.to(torch.bfloat16))
            plain = comm.allreduce(T).clone()
            assert torch.allclose(plain.float(), total, atol=0.08, rtol=0.02), T
        assert comm.error_status() == 0 and gemm_tcgen05.error_status() == 0
    # ---- device-timed comparison: fused pair of kernels vs cuBLAS + NCCL all-reduce + norm kernel
    T, K = 4096, 12288 // W
    x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
    w = torch.randn(H, K, device=dev, dtype=torch.bfloat16) * 0.05
    nw = torch.ones(H, device=dev, dtype=torch.bfloat16)
    b, e, S = comm.shard(T)
    shard = torch.zeros(S, H, device=dev, dtype=torch.bfloat16)
    res = torch.zeros(T, H, device=dev, dtype=torch.bfloat16)

    def fused():
        comm.gemm_rs_norm(x, w, shard, nw, 1e-6)

    y_local = torch.empty(T, H, device=dev, dtype=torch.bfloat16)

    def gemm_only():
        ops.linear(x, w, out=y_local)

    def barrier_fused():
        ops.linear(x, w, out=comm.partial_buffer(T))
        comm.allreduce_norm(T, shard, nw, 1e-6)

    def baseline():
        y = torch.nn.functional.linear(x, w)
        dist.all_reduce(y)
        ops.rmsnorm(y, nw, 1e-6, residual=res)

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

    tf, tb = timeit(fused), timeit(baseline)
    tg, tbar = timeit(gemm_only), timeit(barrier_fused)
    assert comm.error_status() == 0
    flops = 2.0 * T * H * K
    link_bytes = (W - 1) / W * T * H * 2 * 2  # scatter of partials out + gather of normalised rows in
    return (f"GEMM_RS_OK world={W} T={T} K={K}: fused {tf * 1e3:.1f} us, cublas+nccl+norm {tb * 1e3:.1f} us "
              f"local gemm alone {tg * 1e3:.1f} us, gemm + barrier all-reduce+norm kernel {tbar * 1e3:.1f} us "
              f"(gemm alone at 1.6 PF: {flops / 1.6e15 * 1e6:.1f} us, link at 770 GB/s: {link_bytes / 770e9 * 1e6:.1f} us)")


if __name__ == "__main__":
    from mp_common import guarded
    guarded(main)
