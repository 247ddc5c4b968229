"""Where does an engine step spend its device time?

Runs the serving workload of `bench.py` (Qwen3-8B shape by default) to a steady state, then records
a window of engine steps with the PyTorch profiler (CUPTI activity records; graph-replayed kernels
are included) and prints device time per kernel name, plus the wall time of the window.  The
numbers are for finding the next kernel to work on; a throughput figure is never taken from a run
under a profiler.

    python benchmarks/step_breakdown.py --skip 300 --steps 20
"""
from __future__ import annotations

import argparse
import collections
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--requests", type=int, default=512)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=512)
    ap.add_argument("--concurrency", type=int, default=256)
    ap.add_argument("--max-tokens-per-batch", type=int, default=8192)
    ap.add_argument("--skip", type=int, default=300, help="engine steps before the recorded window")
    ap.add_argument("--steps", type=int, default=20, help="engine steps in the recorded window")
    ap.add_argument("--top", type=int, default=30)
    args = ap.parse_args()

    import torch
    from torch.profiler import ProfilerActivity, profile

    from xllm_b200 import LLM

    ps = None
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:        # under torchrun: a tensor-parallel engine, rank 0 reports
        from xllm_b200.parallel.state import init_parallel
        ps = init_parallel()
    dev = ps.device if ps else torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    quiet = ps is not None and ps.rank != 0
    llm = LLM(args.model, devices=str(dev), dtype="bfloat16", block_size=16, parallel_state=ps,
              max_seqs_per_batch=args.concurrency, max_tokens_per_batch=args.max_tokens_per_batch,
              max_model_len=args.input_len + args.output_len + 16, enable_prefix_cache=False,
              enable_chunked_prefill=True, enable_schedule_overlap=True, enable_graph=True,
              policy="prefill_first", random_weights=True)
    eng = llm.engine
    eng.runner.warmup([b for b in eng.runner.buckets if b == args.concurrency] or None)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, eng.args.vocab_size, (args.requests, args.input_len), generator=g)
    cursor = in_flight = 0

    def submit_more():
        nonlocal cursor, in_flight
        while cursor < args.requests and in_flight < args.concurrency:
            eng.add_request(f"r-{cursor}", ids[cursor].tolist(), temperature=0.0, max_tokens=args.output_len,
                            ignore_eos=True, offline=True)
            cursor += 1
            in_flight += 1

    def step():
        nonlocal in_flight
        for ev in eng.step():
            if ev.request_finished:
                in_flight -= 1
        submit_more()

    submit_more()
    for _ in range(args.skip):
        step()
    torch.cuda.synchronize()
    # the same number of steps without the profiler: the true step time of this phase
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    if not quiet:
        print(f"unprofiled: {args.steps} steps, {e0.elapsed_time(e1) / args.steps:.2f} ms/step on the device clock, "
              f"{(time.perf_counter() - t0) * 1e3 / args.steps:.2f} ms/step wall")
    kinds = collections.Counter()
    t0 = time.perf_counter()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(args.steps):
            b = getattr(eng, "last_batch_info", None)
            step()
            info = getattr(eng, "last_batch_info", None)
            if info:
                kinds[info] += 1
        torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    per = collections.defaultdict(lambda: [0.0, 0])
    total = 0.0
    for ev in prof.events():
        dt = getattr(ev, "device_time", 0) or getattr(ev, "cuda_time", 0)
        if dt and ev.device_type is not None and "cuda" in str(ev.device_type).lower():
            per[ev.name][0] += dt
            per[ev.name][1] += 1
            total += dt
    if quiet:
        torch.cuda.synchronize()
        os._exit(0)
    print(f"window: {args.steps} steps, wall {wall * 1e3 / args.steps:.2f} ms/step, "
          f"device busy {total / 1e3 / args.steps:.2f} ms/step")
    if kinds:
        print("batches:", dict(kinds))
    for name, (us, n) in sorted(per.items(), key=lambda kv: -kv[1][0])[: args.top]:
        print(f"{us / 1e3 / args.steps:8.3f} ms/step {100 * us / total:5.1f}%  n/step {n / args.steps:7.1f}  "
              f"avg {us / n:8.1f} us  {name[:110]}")


if __name__ == "__main__":
    main()
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        sys.stdout.flush()
        os._exit(0)
