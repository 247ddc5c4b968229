#!/usr/bin/env python
"""Small, self-ending workloads for `ncu` captures of single kernels (inputs larger than L2, a few
hundred MB on the device, a handful of launches).

    python benchmarks/profile_case.py --kernel gemm       # tcgen05 GEMM, 8192 x 8192 x 4096
    python benchmarks/profile_case.py --kernel gemm_small # M = 256 weight-streaming shape
    python benchmarks/profile_case.py --kernel decode     # paged GQA decode attention, B=64 ctx=4096
    python benchmarks/profile_case.py --kernel prefill    # paged prefill attention, 4 x 2048
    python benchmarks/profile_case.py --kernel norm       # fused add + RMSNorm, 16384 x 4096
    python benchmarks/profile_case.py --kernel moe        # grouped GEMM of the MoE layer
"""
import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from xllm_b200 import ops  # noqa: E402
from xllm_b200.ops import gemm_tcgen05, moe  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="gemm")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    dev = "cuda"
    torch.manual_seed(0)
    if a.kernel in ("gemm", "gemm_small"):
        M, N, K = (8192, 8192, 4096) if a.kernel == "gemm" else (256, 24576, 4096)
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        fn = lambda: gemm_tcgen05.gemm_nt(x, w, out=out)
    elif a.kernel == "decode":
        B, ctx, nq, nkv, d, page = 64, 4096, 32, 8, 128, 16
        nb = B * (ctx // page) + 1
        kc = torch.randn(nb, nkv, page, d, device=dev, dtype=torch.bfloat16)
        vc = torch.randn(nb, nkv, page, d, device=dev, dtype=torch.bfloat16)
        bt = (torch.randperm(nb - 1, device=dev)[: B * (ctx // page)] + 1).view(B, -1).to(torch.int32)
        q = torch.randn(B, nq, d, device=dev, dtype=torch.bfloat16)
        sl = torch.full((B,), ctx, device=dev, dtype=torch.int32)
        out = torch.empty_like(q)
        fn = lambda: ops.paged_decode_attention(q, kc, vc, bt, sl, 1 / math.sqrt(d), splits=1, out=out)
    elif a.kernel == "prefill":
        B, L, nq, nkv, d, page = 4, 2048, 32, 8, 128, 16
        nb = B * (L // page) + 1
        kc = torch.randn(nb, nkv, page, d, device=dev, dtype=torch.bfloat16)
        vc = torch.randn(nb, nkv, page, d, device=dev, dtype=torch.bfloat16)
        bt = (torch.arange(B * (L // page), device=dev) + 1).view(B, -1).to(torch.int32)
        q = torch.randn(B * L, nq, d, device=dev, dtype=torch.bfloat16)
        cu = (torch.arange(B + 1, device=dev) * L).to(torch.int32)
        kl = torch.full((B,), L, device=dev, dtype=torch.int32)
        out = torch.empty_like(q)
        fn = lambda: ops.paged_prefill_attention(q, kc, vc, bt, cu, kl, L, 1 / math.sqrt(d), out=out)
    elif a.kernel == "norm":
        T, H = 16384, 4096
        x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
        res = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
        w = torch.ones(H, device=dev, dtype=torch.bfloat16)
        out = torch.empty_like(x)
        fn = lambda: ops.rmsnorm(x, w, 1e-6, residual=res, out=out)
    elif a.kernel == "moe":
        T, E, K, H, I = 4096, 128, 8, 2048, 768
        x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
        logits = torch.randn(T, E, device=dev)
        w1 = torch.randn(E, 2 * I, H, device=dev, dtype=torch.bfloat16) * 0.05
        w2 = torch.randn(E, H, I, device=dev, dtype=torch.bfloat16) * 0.05
        ws = moe.MoeWorkspace(T, K, E, E, H, I, dev)
        fn = lambda: moe.fused_moe(x, logits, w1, w2, K, ws=ws)
    else:
        raise SystemExit(f"unknown kernel {a.kernel}")
    for _ in range(a.iters):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    print(f"{a.kernel}: {e0.elapsed_time(e1):.3f} ms (warm L2; see benchmarks/kernel_bench.py for flushed timings)")


if __name__ == "__main__":
    main()
