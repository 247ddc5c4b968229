"""Decode-size GEMM sweep: every tile / pair / split-K configuration of the tcgen05 GEMM against
cuBLAS on the Qwen3-8B projection shapes, timed without host overhead.

Each configuration is captured in a CUDA graph of 32 launches that rotate over enough weight
matrices to exceed L2 (so every launch streams its weights from HBM), and the replay is timed with
CUDA events.

    python benchmarks/gemm_decode_sweep.py 8 64 256 512        # token counts to sweep
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from xllm_b200.ops import gemm_tcgen05 as g  # noqa: E402


def graph_time(fns, rounds=5):
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for f in fns:
            f()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=s):
            for f in fns:
                f()
    gr.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(rounds):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        gr.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / len(fns))
    return sorted(ts)[len(ts) // 2] * 1e3


def main():
    g.prepare()
    Ms = [int(a) for a in sys.argv[1:]] or [8, 64, 256, 512]
    for M in Ms:
        for (N, K, name) in ((6144, 4096, "qkv"), (4096, 4096, "o"), (24576, 4096, "gate_up"), (4096, 12288, "down")):
            R = max(2, min(16, (300 << 20) // (N * K * 2) + 1))
            xs = [torch.randn(M, K, device="cuda", dtype=torch.bfloat16) for _ in range(R)]
            ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) for _ in range(R)]
            o = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            reps = max(1, 32 // R)
            res = []
            for pair in (0, 1):
                if pair and M <= 128:
                    continue
                for tn in (64, 128, 192, 256):
                    for ks in (1, 2, 3, 4, 6, 8):
                        if M * N * 4 > (64 << 20) and ks > 1:
                            continue
                        t = graph_time([(lambda i=i: g.gemm_nt(xs[i], ws[i], out=o, tile_n=tn, pair=pair, split_k=ks))
                                        for i in range(R)] * reps, 3)
                        res.append((t, pair, tn, ks))
            auto = graph_time([(lambda i=i: g.gemm_nt(xs[i], ws[i], out=o)) for i in range(R)] * reps)
            cublas = graph_time([(lambda i=i: torch.nn.functional.linear(xs[i], ws[i])) for i in range(R)] * reps)
            res.sort()
            print(f"M={M} {name:8s} cublas {cublas:6.1f} auto {auto:6.1f} best: " +
                  " ".join(f"p{p}t{tn}k{ks}:{t:.1f}" for t, p, tn, ks in res[:6]), flush=True)
            assert g.error_status() == 0
            del xs, ws


if __name__ == "__main__":
    main()
