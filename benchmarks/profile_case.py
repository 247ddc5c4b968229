#!/usr/bin/env python
"""Small, self-ending workloads for `ncu` captures of single kernels (inputs larger than L2, a few
hundred MB on the device, a handful of launches).

    python benchmarks/profile_case.py --kernel gemm       # tcgen05 GEMM, 8192 x 8192 x 4096
    python benchmarks/profile_case.py --kernel gemm_small # M = 256 weight-streaming shape
    python benchmarks/profile_case.py --kernel decode     # paged GQA decode attention, B=64 ctx=4096
    python benchmarks/profile_case.py --kernel prefill    # paged prefill attention, 4 x 2048
    python benchmarks/profile_case.py --kernel norm       # fused add + RMSNorm, 16384 x 4096
    python benchmarks/profile_case.py --kernel moe        # grouped GEMM of the MoE layer
    python benchmarks/profile_case.py --kernel mla        # absorbed MLA decode, 64 rows x 16 heads, ctx 4096
    python benchmarks/profile_case.py --kernel fp8_block  # block-scaled fp8 GEMM, 4096 x 7168 x 7168
    python benchmarks/profile_case.py --kernel rope       # qk-norm + RoPE + paged KV write, 8192 tokens
    python benchmarks/profile_case.py --kernel act        # SiLU-mul, 8192 x 24576
    python benchmarks/profile_case.py --kernel sample     # sampler, 256 rows x 151936
    python benchmarks/profile_case.py --kernel quant      # 1 x 128 group quantisation, 8192 x 7168
    python benchmarks/profile_case.py --kernel gdn        # gated-delta-rule decode step
    python benchmarks/profile_case.py --kernel route      # MoE routing, 8192 tokens x 256 experts
    python benchmarks/profile_case.py --kernel topk       # radix top-k, 1024 rows x 151936, k = 64
    python benchmarks/profile_case.py --kernel logsoftmax # log-softmax, 1024 rows x 151936
    python benchmarks/profile_case.py --kernel gemm_act   # gate_up GEMM with the SiLU-mul epilogue, 2304 x 24576 x 4096
    python benchmarks/profile_case.py --kernel xattn      # beam attention: 16 requests x 128 beams over 2048-token prompts
    python benchmarks/profile_case.py --kernel gdn_prefill # gated-delta-rule prompt chunk, 4096 tokens x 32 heads
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
    elif a.kernel == "mla":
        from xllm_b200.ops import mla
        N, nh, ctx, page = 64, 16, 4096, 16
        nb = N * (ctx // page) + 1
        cache = torch.randn(nb, 1, page, 576, device=dev, dtype=torch.bfloat16)
        bt = (torch.randperm(nb - 1, device=dev)[: N * (ctx // page)] + 1).view(N, -1).to(torch.int32)
        q = torch.randn(N, nh, 576, device=dev, dtype=torch.bfloat16) * 0.3
        sl = torch.full((N,), ctx, device=dev, dtype=torch.int32)
        out = torch.empty(N, nh, 512, device=dev, dtype=torch.bfloat16)
        fn = lambda: mla.decode(q, cache, bt, 0.07, seq_lens=sl, splits=4, out=out)
    elif a.kernel == "fp8_block":
        from xllm_b200.ops import fp8
        M, N, K = 4096, 7168, 7168
        a_q, a_s = fp8.quant_group128(torch.randn(M, K, device=dev, dtype=torch.bfloat16))
        w_q, w_s = fp8.quant_block128_ref(torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        fn = lambda: fp8.block_scaled_mm(a_q, a_s, w_q, w_s, out=out)
    elif a.kernel == "rope":
        from xllm_b200.ops import reference as ref
        T, nq, nkv, d, page = 8192, 32, 8, 128, 16
        qkv = torch.randn(T, (nq + 2 * nkv) * d, device=dev, dtype=torch.bfloat16)
        pos = torch.arange(T, device=dev) % 4096
        cs = ref.build_cos_sin_cache(d, 4096, 1e6, None, dev)
        w = torch.ones(d, device=dev, dtype=torch.bfloat16)
        kc = torch.zeros(T // page + 1, nkv, page, d, device=dev, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        slots = torch.arange(T, device=dev, dtype=torch.int32)
        fn = lambda: ops.rope_kv_write(qkv, nq, nkv, d, pos, cs, d, slots, kc, vc, w, w, 1e-6)
    elif a.kernel == "act":
        x = torch.randn(8192, 2 * 12288, device=dev, dtype=torch.bfloat16)
        out = torch.empty(8192, 12288, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.act_and_mul(x, "silu", out=out)
    elif a.kernel == "sample":
        B, V = 256, 151936
        logits = torch.randn(B, V, device=dev, dtype=torch.bfloat16)
        t = torch.full((B,), 0.8, device=dev)
        k = torch.full((B,), 50, device=dev, dtype=torch.int32)
        pp = torch.full((B,), 0.9, device=dev)
        seeds = torch.arange(B, device=dev, dtype=torch.int64)
        offs = torch.zeros(B, device=dev, dtype=torch.int32)
        fn = lambda: ops.sample(logits, t, k, pp, seeds=seeds, offsets=offs, want_logprob=True)
    elif a.kernel == "quant":
        from xllm_b200.ops import fp8
        x = torch.randn(8192, 7168, device=dev, dtype=torch.bfloat16)
        fn = lambda: fp8.quant_group128(x)
    elif a.kernel == "gdn":
        from xllm_b200.ops import gdn
        B, nv, dk, dv = 256, 32, 128, 128
        state = torch.zeros(B, nv, dk, dv, device=dev, dtype=torch.float32)
        slots = torch.arange(B, device=dev, dtype=torch.int64)
        q, k = torch.randn(B, nv, dk, device=dev), torch.randn(B, nv, dk, device=dev) * 0.1
        v = torch.randn(B, nv, dv, device=dev)
        g, beta = -torch.rand(B, nv, device=dev), torch.rand(B, nv, device=dev)
        fn = lambda: gdn.decode_step(state, slots, q, k, v, g, beta)
    elif a.kernel == "route":
        from xllm_b200.ops import _lib
        T, E, K = 8192, 256, 8
        logits = torch.randn(T, E, device=dev)
        bias = torch.zeros(E, device=dev)
        ws = moe.MoeWorkspace(T, K, E, E, 128, 128, dev)
        lib = _lib.load()
        fn = lambda: lib.xllm_moe_route(logits.data_ptr(), 1, bias.data_ptr(), ws.topk_ids.data_ptr(), ws.topk_w.data_ptr(),
                                        ws.counts.data_ptr(), ws.slot.data_ptr(), T, E, K, 8, 4, 1, 1, 2.5, 0, E,
                                        torch.cuda.current_stream().cuda_stream)
    elif a.kernel in ("topk", "logsoftmax"):
        from xllm_b200.ops import select
        logits = torch.randn(1024, 151936, device=dev, dtype=torch.bfloat16)
        fn = (lambda: select.topk(logits, 64)) if a.kernel == "topk" else (lambda: select.log_softmax(logits))
    elif a.kernel == "gemm_act":
        M, I, K = 2304, 12288, 4096
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(2 * I, K, device=dev, dtype=torch.bfloat16) * 0.02
        out = torch.empty(M, I, device=dev, dtype=torch.bfloat16)
        fn = lambda: gemm_tcgen05.gemm_act_mul(x, w, "silu", out=out)
        if os.environ.get("GEMM_ACT_COMPARE"):   # the two-launch form: GEMM into [M, 2I], then the activation kernel
            mid = torch.empty(M, 2 * I, device=dev, dtype=torch.bfloat16)

            def fn():
                gemm_tcgen05.gemm_nt(x, w, out=mid)
                gemm_tcgen05.act_and_mul_interleaved(mid, "silu", out=out)
    elif a.kernel == "xattn":
        from xllm_b200.ops import xattn
        R, W, ctx, nq, nkv, d, page, cap = 16, 128, 2048, 32, 8, 128, 16, 2
        nb = R * (ctx // page) + 1
        kc = torch.randn(nb, nkv, page, d, device=dev, dtype=torch.bfloat16)
        vc = torch.randn(nb, nkv, page, d, device=dev, dtype=torch.bfloat16)
        bt = (torch.randperm(nb - 1, device=dev)[: R * (ctx // page)] + 1).view(R, -1).to(torch.int32)
        q = torch.randn(R * W, nq, d, device=dev, dtype=torch.bfloat16) * 0.3
        ku = torch.randn(R * W, nkv, cap, d, device=dev, dtype=torch.bfloat16)
        vu = torch.randn_like(ku)
        anc = torch.randint(0, R * W, (cap, R * W), device=dev, dtype=torch.int32)
        cu = (torch.arange(R + 1, device=dev) * W).to(torch.int32)
        kl = torch.full((R,), ctx, device=dev, dtype=torch.int32)
        out = torch.empty_like(q)
        fn = lambda: xattn.xattention(q, kc, vc, bt, cu, kl, W, ku, vu, anc, 2, 1 / math.sqrt(d), out=out)
        if os.environ.get("XATTN_COMPARE"):   # the same rows through the paged decode kernel: every beam re-reads the prompt
            bt_rows = bt.repeat_interleave(W, 0).contiguous()
            sl = torch.full((R * W,), ctx, device=dev, dtype=torch.int32)
            fn = lambda: ops.paged_decode_attention(q, kc, vc, bt_rows, sl, 1 / math.sqrt(d), out=out)
    elif a.kernel == "gdn_prefill":
        from xllm_b200.ops import gdn
        n, nv, dk, dv = 4096, 32, 128, 128
        state = torch.zeros(4, nv, dk, dv, device=dev, dtype=torch.float32)
        q, k = torch.randn(n, nv, dk, device=dev), torch.randn(n, nv, dk, device=dev) * 0.1
        v = torch.randn(n, nv, dv, device=dev)
        g, beta = -torch.rand(n, nv, device=dev), torch.rand(n, nv, device=dev)
        fn = lambda: gdn.prefill(state, 1, True, q, k, v, g, beta)
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
