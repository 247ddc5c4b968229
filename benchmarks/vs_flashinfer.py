#!/usr/bin/env python
"""This build's kernels against their FlashInfer counterparts (the library the reference's CUDA path calls:
xllm/core/layers/cuda/flashinfer_attention.cpp, flashinfer sampling / norm / activation ops), same inputs,
same device, CUDA events, L2 flushed between iterations.

    python benchmarks/vs_flashinfer.py                 # every case
    python benchmarks/vs_flashinfer.py --only decode   # decode | prefill | sampling | norm | act

FlashInfer compiles a module the first time a configuration is used (nvcc, tens of seconds); set
FLASHINFER_WORKSPACE_BASE to keep the compiled modules between runs.  A case whose FlashInfer side cannot be
built or run prints `unavailable` with the reason and the run goes on.  Prints one table row per case and
a final JSON line.
"""
import argparse
import json
import math
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from xllm_b200 import ops  # noqa: E402

_flush = None


def timed(fn, iters=10, warmup=3):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        _flush.zero_()                                   # larger than L2: the next launch starts cold
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def paged_case(B, ctx, nq=32, nkv=8, d=128, page=16, q_len=1, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    per = (ctx + page - 1) // page
    nb = B * per + 1
    kc = torch.randn(nb, nkv, page, d, device="cuda", dtype=torch.bfloat16, generator=g)
    vc = torch.randn(nb, nkv, page, d, device="cuda", dtype=torch.bfloat16, generator=g)
    bt = (torch.randperm(nb - 1, device="cuda", generator=g)[: B * per] + 1).view(B, per).to(torch.int32)
    q = torch.randn(B * q_len, nq, d, device="cuda", dtype=torch.bfloat16, generator=g)
    kv_lens = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
    indptr = (torch.arange(B + 1, device="cuda") * per).to(torch.int32)
    indices = bt.reshape(-1).contiguous()
    last = torch.full((B,), (ctx - 1) % page + 1, device="cuda", dtype=torch.int32)
    return dict(q=q, kc=kc, vc=vc, bt=bt, kv_lens=kv_lens, indptr=indptr, indices=indices, last=last, nq=nq, nkv=nkv, d=d,
                page=page, B=B, ctx=ctx, q_len=q_len)


def check(a, b, what, tol=3e-2):
    err = (a.float() - b.float()).abs().max().item()
    if not err < tol:
        raise RuntimeError(f"{what}: results differ by {err}")
    return err


def case_decode(rows):
    import flashinfer
    ws = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for B, ctx in ((64, 4096), (256, 1280), (16, 16384)):
        c = paged_case(B, ctx)
        scale = 1 / math.sqrt(c["d"])
        out = torch.empty_like(c["q"])
        splits = ops.decode_splits(B, c["nkv"], c["nq"] // c["nkv"], ctx)
        wsp = ops.decode_workspace(B, c["nq"], c["d"], splits, "cuda")
        mine = lambda: ops.paged_decode_attention(c["q"], c["kc"], c["vc"], c["bt"], c["kv_lens"], scale, splits=splits,
                                                  workspace=wsp, out=out)
        t_mine = timed(mine)
        kv_bytes = 2 * B * ctx * c["nkv"] * c["d"] * 2
        name = f"decode attention B={B} ctx={ctx} 32/8x128"
        try:
            w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "HND", use_tensor_cores=True)
            w.plan(c["indptr"], c["indices"], c["last"], c["nq"], c["nkv"], c["d"], c["page"], q_data_type=torch.bfloat16,
                   kv_data_type=torch.bfloat16)
            ref = lambda: w.run(c["q"], (c["kc"], c["vc"]))
            check(mine(), ref(), name)
            t_ref = timed(ref)
            rows.append((name, t_mine, t_ref, f"{kv_bytes / t_mine / 1e9:.2f} vs {kv_bytes / t_ref / 1e9:.2f} TB/s of KV"))
        except Exception as e:                             # noqa: BLE001
            rows.append((name, t_mine, None, f"unavailable: {type(e).__name__}: {str(e)[:120]}"))


def case_prefill(rows):
    import flashinfer
    ws = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")
    for B, L in ((8, 1024), (2, 4096), (1, 16384)):
        c = paged_case(B, L, q_len=L)
        scale = 1 / math.sqrt(c["d"])
        cu = (torch.arange(B + 1, device="cuda") * L).to(torch.int32)
        out = torch.empty_like(c["q"])
        mine = lambda: ops.paged_prefill_attention(c["q"], c["kc"], c["vc"], c["bt"], cu, c["kv_lens"], L, scale, out=out)
        t_mine = timed(mine, iters=6)
        flops = 4 * B * c["nq"] * c["d"] * L * L / 2
        name = f"prefill attention {B} x {L} causal 32/8x128"
        try:
            w = flashinfer.BatchPrefillWithPagedKVCacheWrapper(ws, "HND")
            w.plan(cu, c["indptr"], c["indices"], c["last"], c["nq"], c["nkv"], c["d"], c["page"], causal=True,
                   q_data_type=torch.bfloat16, kv_data_type=torch.bfloat16)
            ref = lambda: w.run(c["q"], (c["kc"], c["vc"]))
            check(mine(), ref(), name)
            t_ref = timed(ref, iters=6)
            rows.append((name, t_mine, t_ref, f"{flops / t_mine / 1e9:.0f} vs {flops / t_ref / 1e9:.0f} TFLOP/s"))
        except Exception as e:                             # noqa: BLE001
            rows.append((name, t_mine, None, f"unavailable: {type(e).__name__}: {str(e)[:120]}"))


def case_sampling(rows):
    import flashinfer
    B, V = 256, 151936
    logits = torch.randn(B, V, device="cuda", dtype=torch.bfloat16)
    t = torch.full((B,), 0.8, device="cuda")
    k = torch.full((B,), 50, device="cuda", dtype=torch.int32)
    p = torch.full((B,), 0.9, device="cuda")
    seeds = torch.arange(B, device="cuda", dtype=torch.int64)
    offs = torch.zeros(B, device="cuda", dtype=torch.int32)
    mine = lambda: ops.sample(logits, t, k, p, seeds=seeds, offsets=offs)
    t_mine = timed(mine)
    name = f"sampling temperature + top-k 50 + top-p 0.9, {B} x {V}"
    try:
        scaled = lambda: (logits.float() / t[:, None])
        ref = lambda: flashinfer.sampling.top_k_top_p_sampling_from_logits(scaled(), k, p)
        ref()
        t_ref = timed(ref)
        rows.append((name, t_mine, t_ref, "FlashInfer side includes the temperature scaling pass it needs"))
    except Exception as e:                                 # noqa: BLE001
        rows.append((name, t_mine, None, f"unavailable: {type(e).__name__}: {str(e)[:120]}"))
    greedy = lambda: ops.sample(logits)
    t_g = timed(greedy)
    t_tg = timed(lambda: logits.argmax(-1))
    rows.append((f"greedy, {B} x {V}", t_g, t_tg, "library side: torch argmax"))


def case_norm(rows):
    import flashinfer
    for T, H in ((8192, 4096), (256, 4096)):
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        res = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        out = torch.empty_like(x)
        mine = lambda: ops.rmsnorm(x, w, 1e-6, residual=res, out=out)
        t_mine = timed(mine)
        name = f"add + RMSNorm {T} x {H}"
        try:
            x2, r2 = x.clone(), res.clone()
            ref = lambda: flashinfer.norm.fused_add_rmsnorm(x2, r2, w, 1e-6)
            ref()
            t_ref = timed(ref)
            rows.append((name, t_mine, t_ref, f"{4 * T * H * 2 / t_mine / 1e9:.2f} vs {4 * T * H * 2 / t_ref / 1e9:.2f} TB/s"))
        except Exception as e:                             # noqa: BLE001
            rows.append((name, t_mine, None, f"unavailable: {type(e).__name__}: {str(e)[:120]}"))


def case_act(rows):
    import flashinfer
    for T, I in ((8192, 12288), (256, 12288)):
        x = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(T, I, device="cuda", dtype=torch.bfloat16)
        mine = lambda: ops.act_and_mul(x, "silu", out=out)
        t_mine = timed(mine)
        name = f"SiLU-mul {T} x {2 * I}"
        try:
            ref = lambda: flashinfer.activation.silu_and_mul(x, out)
            check(mine(), ref(), name)
            t_ref = timed(ref)
            rows.append((name, t_mine, t_ref, f"{3 * T * I * 2 / t_mine / 1e9:.2f} vs {3 * T * I * 2 / t_ref / 1e9:.2f} TB/s"))
        except Exception as e:                             # noqa: BLE001
            rows.append((name, t_mine, None, f"unavailable: {type(e).__name__}: {str(e)[:120]}"))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    a = ap.parse_args()
    cases = {"decode": case_decode, "prefill": case_prefill, "sampling": case_sampling, "norm": case_norm, "act": case_act}
    rows = []
    try:
        import flashinfer
        version = flashinfer.__version__
    except Exception as e:                                 # noqa: BLE001
        print(json.dumps({"unavailable": f"flashinfer cannot be imported: {e}"}))
        return 0
    for name, fn in cases.items():
        if a.only and a.only != name:
            continue
        try:
            fn(rows)
        except Exception as e:                             # noqa: BLE001
            rows.append((name, None, None, f"failed: {type(e).__name__}: {str(e)[:160]}"))
    print(f"| case | this build (ms) | FlashInfer {version} (ms) | ratio (library / ours) | note |")
    print("|---|---|---|---|---|")
    for name, tm, tr, note in rows:
        f = lambda v: "-" if v is None else f"{v:.3f}"
        ratio = "-" if (tm is None or tr is None) else f"{tr / tm:.2f}"
        print(f"| {name} | {f(tm)} | {f(tr)} | {ratio} | {note} |")
    print(json.dumps({"flashinfer": version, "rows": [{"case": n, "ours_ms": tm, "flashinfer_ms": tr, "note": note}
                                                      for n, tm, tr, note in rows]}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
