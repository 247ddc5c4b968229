#!/usr/bin/env python
"""Per-kernel timings against the roofline (CUDA events, warm-up, L2 flushed between iterations).

    python benchmarks/kernel_bench.py [--what gemm,decode,prefill,small] [--json out.json]

Prints, for every kernel and shape of the Qwen3-8B serving step, the achieved TFLOP/s or GB/s, the
fraction of the measured peak (MEASURED_PEAKS.json when present) and the cuBLAS / PyTorch number for
the same shape where one exists.
"""
import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from xllm_b200 import ops  # noqa: E402
from xllm_b200.ops import gemm_tcgen05  # noqa: E402


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def bench(fn, iters=10, warmup=3):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        _flush.zero_()  # evict L2 (126 MB) between timed runs
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2] * 1e-3 if ts else 0.0


def bench_pair(fa, fb, iters=10, warmup=3):
    """Two alternatives timed alternately (a, b, a, b, ...), L2 flushed before each: clock drift under the
    power cap hits both alike.  Returns the two medians in seconds."""
    bench(fa, iters=0, warmup=warmup)
    bench(fb, iters=0, warmup=warmup)
    ta, tb = [], []
    for _ in range(iters):
        for f, ts in ((fa, ta), (fb, tb)):
            _flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
    ta.sort()
    tb.sort()
    return ta[len(ta) // 2] * 1e-3, tb[len(tb) // 2] * 1e-3


def bench_rotating(fns, rounds=5, warmup=1):
    """Back-to-back launches of closures that work on different buffers (together larger than L2),
    one event pair around the whole train: per-launch time without host launch gaps."""
    for _ in range(warmup):
        for f in fns:
            f()
    ts = []
    for _ in range(rounds):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for f in fns:
            f()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / len(fns))
    ts.sort()
    return ts[len(ts) // 2] * 1e-3


def gemm_rows(results, hbm, tf, tag):
    shapes = []
    for M in (8192, 2048, 256, 64, 8):
        shapes += [(M, 6144, 4096, "qkv"), (M, 4096, 4096, "o"), (M, 24576, 4096, "gate_up"), (M, 4096, 12288, "down")]
    shapes.append((256, 151936, 4096, "lm_head"))
    for M, N, K, name in shapes:
        wbytes = N * K * 2
        R = max(2, min(16, (300 << 20) // wbytes + 1)) if M <= 2048 and N < 100000 else 1
        xs = [torch.randn(M, K, device="cuda", dtype=torch.bfloat16) for _ in range(R)]
        ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(R)]
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        if R == 1:
            t_mine = bench(lambda: gemm_tcgen05.gemm_nt(xs[0], ws[0], out=out))
            t_lib = bench(lambda: torch.nn.functional.linear(xs[0], ws[0]))
        else:
            reps = max(1, 32 // R)
            t_mine = bench_rotating([(lambda i=i: gemm_tcgen05.gemm_nt(xs[i], ws[i], out=out)) for i in range(R)] * reps)
            t_lib = bench_rotating([(lambda i=i: torch.nn.functional.linear(xs[i], ws[i], )) for i in range(R)] * reps)
        flops = 2.0 * M * N * K
        bytes_ = 2.0 * (M * K + N * K + M * N)
        ideal = max(flops / (tf * 1e12), bytes_ / (hbm * 1e9))
        r = dict(kernel="gemm_bf16_tcgen05", shape=f"{name} M={M} N={N} K={K}", ms=t_mine * 1e3,
                 tflops=flops / t_mine / 1e12, gbs=bytes_ / t_mine / 1e9, frac_of_roofline=ideal / t_mine,
                 cublas_ms=t_lib * 1e3, vs_cublas=t_lib / t_mine, peaks=tag)
        results.append(r)
        print(f"gemm {r['shape']:<34} {r['ms']:8.3f} ms {r['tflops']:8.1f} TF/s  {r['gbs']:7.0f} GB/s  "
              f"roofline {r['frac_of_roofline']:.2f} ({tag})  cuBLAS {r['cublas_ms']:.3f} ms  x{r['vs_cublas']:.2f}")
        assert gemm_tcgen05.error_status() == 0
        del xs, ws


def decode_rows(results, hbm, tf, tag):
    nq, nkv, d, page = 32, 8, 128, 16
    for B, ctx in ((256, 1280), (256, 1536), (64, 4096), (16, 8192), (1, 32768)):
        nb = B * ((ctx + page - 1) // page) + 1
        kc = torch.randn(nb, nkv, page, d, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn(nb, nkv, page, d, device="cuda", dtype=torch.bfloat16)
        bt = (torch.randperm(nb - 1, device="cuda")[: B * ((ctx + page - 1) // page)] + 1).view(B, -1).to(torch.int32)
        q = torch.randn(B, nq, d, device="cuda", dtype=torch.bfloat16)
        sl = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
        out = torch.empty_like(q)
        splits = ops.decode_splits(B, nkv, nq // nkv)
        ws = ops.decode_workspace(B, nq, d, splits, "cuda")
        t = bench(lambda: ops.paged_decode_attention(q, kc, vc, bt, sl, 1 / math.sqrt(d), splits=splits, workspace=ws, out=out))
        bytes_ = 2.0 * B * ctx * nkv * d * 2
        r = dict(kernel="paged_decode_kernel", shape=f"B={B} ctx={ctx} nq={nq} nkv={nkv} splits={splits}", ms=t * 1e3,
                 gbs=bytes_ / t / 1e9, frac_of_roofline=bytes_ / t / 1e9 / hbm, peaks=tag)
        results.append(r)
        print(f"decode-attn {r['shape']:<44} {r['ms']:8.3f} ms {r['gbs']:7.0f} GB/s  {r['frac_of_roofline']:.2f} of {tag} HBM")


def prefill_rows(results, hbm, tf, tag):
    nq, nkv, d, page = 32, 8, 128, 16
    for B, L in ((8, 1024), (16, 1024), (2, 4096), (1, 8192)):
        nb = B * (L // page) + 1
        kc = torch.randn(nb, nkv, page, d, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn(nb, nkv, page, d, device="cuda", dtype=torch.bfloat16)
        bt = (torch.arange(B * (L // page), device="cuda") + 1).view(B, -1).to(torch.int32)
        q = torch.randn(B * L, nq, d, device="cuda", dtype=torch.bfloat16)
        cu = (torch.arange(B + 1, device="cuda") * L).to(torch.int32)
        kl = torch.full((B,), L, device="cuda", dtype=torch.int32)
        out = torch.empty_like(q)
        t = bench(lambda: ops.paged_prefill_attention(q, kc, vc, bt, cu, kl, L, 1 / math.sqrt(d), out=out))
        flops = 4.0 * B * nq * d * L * L / 2
        r = dict(kernel="paged_prefill_kernel", shape=f"B={B} L={L}", ms=t * 1e3, tflops=flops / t / 1e12,
                 frac_of_roofline=flops / t / 1e12 / tf, peaks=tag)
        results.append(r)
        print(f"prefill-attn {r['shape']:<20} {r['ms']:8.3f} ms {r['tflops']:8.1f} TF/s  {r['frac_of_roofline']:.2f} of {tag} bf16 peak")


def small_rows(results, hbm, tf, tag):
    H = 4096
    for T in (256, 8192):
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        res = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(x)
        t = bench(lambda: ops.rmsnorm(x, w, 1e-6, residual=res, out=out))
        b = T * H * 2 * 4.0
        results.append(dict(kernel="add_rmsnorm", shape=f"T={T} H={H}", ms=t * 1e3, gbs=b / t / 1e9,
                            frac_of_roofline=b / t / 1e9 / hbm, peaks=tag))
        print(f"add_rmsnorm T={T:<6} {t*1e3:8.3f} ms {b/t/1e9:7.0f} GB/s")
        gu = torch.randn(T, 2 * 12288, device="cuda", dtype=torch.bfloat16)
        o2 = torch.empty(T, 12288, device="cuda", dtype=torch.bfloat16)
        t = bench(lambda: ops.silu_and_mul(gu, out=o2))
        b = T * 12288 * 2 * 3.0
        results.append(dict(kernel="silu_and_mul", shape=f"T={T} I=12288", ms=t * 1e3, gbs=b / t / 1e9,
                            frac_of_roofline=b / t / 1e9 / hbm, peaks=tag))
        print(f"silu_and_mul T={T:<6} {t*1e3:8.3f} ms {b/t/1e9:7.0f} GB/s")
    logits = torch.randn(256, 151936, device="cuda", dtype=torch.bfloat16)
    t = bench(lambda: ops.sample(logits))
    b = logits.numel() * 2.0
    results.append(dict(kernel="sample_greedy", shape="B=256 V=151936", ms=t * 1e3, gbs=b / t / 1e9,
                        frac_of_roofline=b / t / 1e9 / hbm, peaks=tag))
    print(f"sample greedy B=256 {t*1e3:8.3f} ms {b/t/1e9:7.0f} GB/s")


def gdn_rows(results, hbm, tf, tag):
    """Gated-delta-rule decode step (Qwen3-Next geometry: 32 value heads, 128 x 128 state per head).
    The state is read and written once: 2 x B x 32 x 64 KB per call, far larger than L2."""
    from xllm_b200.ops import gdn
    nv, dk, dv = 32, 128, 128
    for B in (64, 256):
        state = torch.randn(B, nv, dk, dv, device="cuda") * 0.1
        slots = torch.arange(B, device="cuda")
        q = torch.randn(B, nv, dk, device="cuda") * 0.1
        k = torch.nn.functional.normalize(torch.randn(B, nv, dk, device="cuda"), dim=-1)
        v = torch.randn(B, nv, dv, device="cuda")
        g = -torch.rand(B, nv, device="cuda")
        beta = torch.rand(B, nv, device="cuda")
        out = torch.empty(B, nv, dv, device="cuda")
        t = bench(lambda: gdn.decode_step(state, slots, q, k, v, g, beta, out=out))
        b = 2.0 * state.numel() * 4
        results.append(dict(kernel="gdn_decode_step", shape=f"B={B} nv={nv} dk={dk} dv={dv}", ms=t * 1e3, gbs=b / t / 1e9,
                            frac_of_roofline=b / t / 1e9 / hbm, peaks=tag))
        print(f"gdn_decode_step B={B:<4} {t*1e3:8.3f} ms {b/t/1e9:7.0f} GB/s  {b/t/1e9/hbm:5.2f} of {tag} copy bandwidth")


def mla_rows(results, hbm, tf, tag):
    """Absorbed MLA decode over the latent cache: every cached token is 1152 bytes, read once per
    group of 16 heads; 128 heads (TP 1) re-read it from L2."""
    from xllm_b200.ops import mla
    page = 16
    for N, nh, ctx in ((256, 16, 2048), (64, 16, 8192), (256, 128, 2048), (16, 128, 8192)):
        nb = N * (ctx // page) + 1
        cache = torch.randn(nb, 1, page, 576, device="cuda", dtype=torch.bfloat16)
        bt = (torch.randperm(nb - 1, device="cuda")[: N * (ctx // page)] + 1).view(N, -1).to(torch.int32)
        q = torch.randn(N, nh, 576, device="cuda", dtype=torch.bfloat16) * 0.3
        sl = torch.full((N,), ctx, device="cuda", dtype=torch.int32)
        out = torch.empty(N, nh, 512, device="cuda", dtype=torch.bfloat16)
        t = bench(lambda: mla.decode(q, cache, bt, 0.07, seq_lens=sl, out=out))
        b = N * ctx * 1152.0
        fl = 2.0 * N * nh * ctx * (576 + 512)
        results.append(dict(kernel="mla_decode_kernel", shape=f"rows={N} heads={nh} ctx={ctx}", ms=t * 1e3, gbs=b / t / 1e9,
                            tflops=fl / t / 1e12, frac_of_roofline=max(b / (hbm * 1e9), fl / (tf * 1e12)) / t, peaks=tag))
        print(f"mla_decode rows={N:<4} heads={nh:<4} ctx={ctx:<5} {t*1e3:8.3f} ms {b/t/1e9:7.0f} GB/s {fl/t/1e12:7.1f} TF/s")


def fp8_rows(results, hbm, tf, tag):
    """Block-scaled fp8 GEMM (1 x 128 activation scales, 128 x 128 weight scales) on DeepSeek-V3 shapes,
    with the bf16 tcgen05 GEMM, the per-tensor fp8 GEMM and cuBLAS bf16 on the same shapes."""
    from xllm_b200.ops import fp8
    for M, N, K, name in ((4096, 7168, 7168, "square"), (4096, 4096, 7168, "gate_up/8"), (4096, 7168, 2048, "down expert"),
                          (256, 7168, 7168, "decode"), (256, 24576, 1536, "q_b")):
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
        a_q, a_s = fp8.quant_group128(x)
        w_q, w_s = fp8.quant_block128_ref(w)
        a_t, s_t = fp8.quant_per_token(x)
        ws1 = torch.ones(1, device="cuda")
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t_blk = bench(lambda: fp8.block_scaled_mm(a_q, a_s, w_q, w_s, out=out))
        t_pt = bench(lambda: fp8.scaled_mm(a_t, w_q, s_t, ws1, out=out))
        t_bf = bench(lambda: gemm_tcgen05.gemm_nt(x, w, out=out))
        t_lib = bench(lambda: torch.nn.functional.linear(x, w))
        fl = 2.0 * M * N * K
        results.append(dict(kernel="gemm_fp8_block_kernel", shape=f"{name} M={M} N={N} K={K}", ms=t_blk * 1e3,
                            tflops=fl / t_blk / 1e12, per_tensor_fp8_ms=t_pt * 1e3, bf16_ms=t_bf * 1e3, cublas_bf16_ms=t_lib * 1e3,
                            peaks=tag))
        print(f"fp8 block {name:<12} M={M:<5} N={N:<6} K={K:<5} {t_blk*1e3:7.3f} ms {fl/t_blk/1e12:7.1f} TF/s | per-tensor fp8 "
              f"{t_pt*1e3:7.3f} ms | bf16 tcgen05 {t_bf*1e3:7.3f} ms | cuBLAS bf16 {t_lib*1e3:7.3f} ms")


def moe_rows(results, hbm, tf, tag):
    """The whole MoE layer (route, permute, grouped GEMM gate|up, SiLU-mul, grouped GEMM down, finalize) on
    Qwen3-30B-A3B and DeepSeek-V3-like expert shapes: the three-launch expert form against the grouped GEMM
    with the gated activation in its epilogue (interleaved expert weights)."""
    from xllm_b200.ops import moe
    for T, E, K, H, I, name in ((8192, 128, 8, 2048, 768, "qwen3-30b-a3b prefill"), (256, 128, 8, 2048, 768, "qwen3-30b-a3b decode"),
                                (8192, 32, 8, 7168, 2048, "deepseek-v3 experts of one EP-8 rank")):
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        logits = torch.randn(T, E, device="cuda")
        w1 = torch.randn(E, 2 * I, H, device="cuda", dtype=torch.bfloat16) * 0.05
        w2 = torch.randn(E, H, I, device="cuda", dtype=torch.bfloat16) * 0.05
        ws = moe.MoeWorkspace(T, K, E, E, H, I, "cuda")
        out = torch.empty_like(x)
        t_plain, t_fused = bench_pair(lambda: moe.fused_moe(x, logits, w1, w2, K, ws=ws, out=out),
                                      lambda: moe.fused_moe(x, logits, w1, w2, K, ws=ws, out=out, interleaved=True))
        fl = 2.0 * T * K * 3 * I * H
        results.append(dict(kernel="fused_moe", shape=f"{name} T={T} E={E} top{K} H={H} I={I}", ms=t_fused * 1e3,
                            tflops=fl / t_fused / 1e12, three_launch_ms=t_plain * 1e3, peaks=tag))
        print(f"moe {name:<38} T={T:<5} {t_fused*1e3:7.3f} ms {fl/t_fused/1e12:7.1f} TF/s ({fl/t_fused/1e12/tf*100:5.1f}% of {tag} cuBLAS bf16)"
              f" | GEMM, activation kernel, GEMM: {t_plain*1e3:7.3f} ms")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="gemm,decode,prefill,small")
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    hbm, tf, tag = peaks()
    results = []
    for w in a.what.split(","):
        {"gemm": gemm_rows, "decode": decode_rows, "prefill": prefill_rows, "small": small_rows, "gdn": gdn_rows, "mla": mla_rows,
         "fp8": fp8_rows, "moe": moe_rows}[w](results, hbm, tf, tag)
    if a.json:
        with open(a.json, "w") as f:
            json.dump(results, f, indent=1)


if __name__ == "__main__":
    main()
