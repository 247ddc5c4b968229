#!/usr/bin/env python
"""Headline serving benchmark: output tokens/s of a Qwen3-8B-shaped bf16 decoder under the closed-loop
load named in BASELINE.json (1024 synthetic requests, input 1024, output 512 with ignore_eos, 256
concurrent, paged KV with block 16, CUDA graphs for decode) at TP = --gpus.

    python bench.py --gpus 1                      # whole workload (default)
    python bench.py --gpus 1 --steps 200 --warmup 5

A "step" is one engine iteration (one scheduled batch -> one forward pass -> one sampled token per
scheduled sequence).  Without --steps the whole 1024-request workload is timed and `steps` reports
how many engine steps it took; with --steps K exactly the first K engine steps of the workload
are timed.  Timing is CUDA events around the step loop, bracketed by barrier + synchronize, max over
ranks.  The `e2e` block repeats the workload through the public API (`LLM.generate`) and times it
with the host clock; every step of both runs copies its inputs from pinned host memory and reads
the sampled tokens back.

`--impl reference` is the arm for the unmodified upstream engine; it cannot be installed offline
 so that arm prints its `unavailable` line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REF_UNAVAILABLE = ("reference cannot be installed offline: its setup.py rejects pip's metadata/build "
                   "commands and every third_party submodule (brpc, cutlass, Mooncake, ...) is empty; "
                   "the build also needs vcpkg, Rust crates and FlashInfer AOT modules from the network")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0, period_ms=200):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index
        self.period = period_ms
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", str(self.period),
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                power.append(float(r[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # clocks under load: ignore idle samples (power well below the busy level)
        if power:
            thr = 0.5 * max(power)
            busy = [s for s, p in zip(sm, power) if p >= thr] or sm
        else:
            busy = sm
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_requests(n, input_len, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    # token ids live in pinned host memory: the engine's per-step H2D copy starts from them
    ids = torch.randint(0, vocab, (n, input_len), generator=g, dtype=torch.int64)
    if torch.cuda.is_available():
        ids = ids.pin_memory()
    return ids


def run(args):
    import torch
    import torch.distributed as dist

    from xllm_b200 import LLM, SamplingParams, ops
    from xllm_b200.parallel.state import init_parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    ps = init_parallel() if world > 1 else None
    rank = ps.rank if ps else 0
    dev = ps.device if ps else torch.device("cuda", 0)
    torch.cuda.set_device(dev)

    max_len = args.input_len + args.output_len + 16
    llm = LLM(args.model, devices=str(dev), dtype="bfloat16", block_size=args.block_size,
              max_seqs_per_batch=args.concurrency, max_tokens_per_batch=args.max_tokens_per_batch,
              max_model_len=max_len, enable_prefix_cache=False, enable_chunked_prefill=True,
              enable_schedule_overlap=not args.no_overlap, enable_graph=not args.no_graph,
              policy="prefill_first", random_weights=True, parallel_state=ps,
              max_memory_utilization=args.max_memory_utilization, num_blocks=args.num_blocks)
    eng = llm.engine
    vocab = eng.args.vocab_size

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def submit(prefix, ids_pinned, out_len):
        for i in range(ids_pinned.shape[0]):
            eng.add_request(f"{prefix}-{i}", ids_pinned[i].tolist(), temperature=0.0, max_tokens=out_len,
                            ignore_eos=True, offline=True)

    # ---------------------------------------------------------------- warm-up (untimed)
    eng.runner.warmup([b for b in eng.runner.buckets if b in (args.concurrency,)] or None)
    warm = make_requests(min(8, args.concurrency), min(args.input_len, 256), vocab, 1)
    submit("warm", warm, max(2, args.warmup))
    wsteps = 0
    while eng.has_unfinished():
        eng.step()
        wsteps += 1
    eng.drain()
    while wsteps < args.warmup:  # at least W warm-up steps
        submit(f"warm{wsteps}", warm[:1], 2)
        while eng.has_unfinished():
            eng.step()
            wsteps += 1
    barrier()

    # ---------------------------------------------------------------- timed run (device clock)
    reqs = make_requests(args.requests, args.input_len, vocab, 0)
    total_target = args.steps if args.steps > 0 else 1 << 60
    out_tokens = 0
    cursor = 0
    in_flight = 0

    def submit_more():
        nonlocal cursor, in_flight
        while cursor < args.requests and in_flight < args.concurrency:
            eng.add_request(f"r-{cursor}", reqs[cursor].tolist(), temperature=0.0, max_tokens=args.output_len,
                            ignore_eos=True, offline=True)
            cursor += 1
            in_flight += 1

    sampler = ClockSampler(dev.index or 0)
    launches0, replays0 = ops.launches(), eng.runner.graph_replays
    h2d0, d2h0 = eng.runner.h2d_bytes, eng.runner.d2h_bytes
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    steps = 0
    submit_more()
    while steps < total_target and (eng.has_unfinished() or cursor < args.requests):
        for ev in eng.step():
            if ev.token >= 0:
                out_tokens += 1
            if ev.request_finished:
                in_flight -= 1
        steps += 1
        submit_more()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    # tokens of the step still in flight (overlap mode) belong to the timed region as well
    for ev in eng.drain():
        if ev.token >= 0:
            out_tokens += 1
    replays = eng.runner.graph_replays - replays0
    per_replay = max(eng.runner.graph_launches_per_replay.values()) if eng.runner.graph_launches_per_replay else 0
    gpu_launches = (ops.launches() - launches0) + replays * per_replay
    h2d_step = (eng.runner.h2d_bytes - h2d0) / max(steps, 1)
    d2h_step = (eng.runner.d2h_bytes - d2h0) / max(steps, 1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = out_tokens / (ms / 1e3)

    # abort whatever the K-step window left unfinished, then the end-to-end run
    if eng.has_unfinished():
        for i in range(cursor):
            eng.abort(f"r-{i}")
        while eng.has_unfinished():
            eng.step()
    e2e = None
    if not args.no_e2e:
        n_e2e = args.requests if args.steps <= 0 else min(args.requests, args.concurrency)
        reqs2 = make_requests(n_e2e, args.input_len, vocab, 2)
        prompts = [reqs2[i] for i in range(n_e2e)]  # pinned host tensors handed to the public API
        sp = SamplingParams(max_tokens=args.output_len if args.steps <= 0 else max(4, min(args.output_len, args.steps // 2)),
                            temperature=0.0, ignore_eos=True)
        h2d0, d2h0, s0 = eng.runner.h2d_bytes, eng.runner.d2h_bytes, eng.steps
        barrier()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp, max_concurrency=args.concurrency)
        barrier()
        dt = time.perf_counter() - t0
        gen = sum(o.usage.num_generated_tokens for o in outs)
        if world > 1:
            t = torch.tensor([dt], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        nst = max(eng.steps - s0, 1)
        e2e = {"value": gen / dt, "unit": "output tok/s", "requests": n_e2e,
               "output_len": sp.max_tokens, "seconds": dt, "steps": nst,
               "h2d_bytes_per_step": (eng.runner.h2d_bytes - h2d0) / nst,
               "d2h_bytes_per_step": (eng.runner.d2h_bytes - d2h0) / nst}

    if rank == 0:
        line = {
            "metric": "output tok/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": steps,
            "warmup": wsteps, "ms_per_step": ms / max(steps, 1), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "xllm_b200",
            "config": {"model": f"{args.model} (random-init, Qwen3-8B shape)" if args.model == "qwen3-8b" else args.model,
                       "requests": args.requests, "input_len": args.input_len, "output_len": args.output_len,
                       "concurrency": args.concurrency, "global_batch": args.concurrency,
                       "seq_len": args.input_len + args.output_len, "block_size": args.block_size,
                       "parallelism": f"tp{world}", "cuda_graphs": not args.no_graph,
                       "schedule_overlap": not args.no_overlap,
                       "window": "whole workload" if args.steps <= 0 else f"first {steps} engine steps",
                       "l2": "inputs larger than L2: every step streams the 16 GB weights / the KV cache",
                       "output_tokens": out_tokens, "kv_blocks": eng.num_blocks},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(gpu_launches),
            "h2d_bytes_per_step": h2d_step, "d2h_bytes_per_step": d2h_step,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # Every collective of this process finished behind the barrier that closed the last timed
        # region, so nothing is in flight.  Leave without tearing the process group down: destroying
        # NCCL communicators that CUDA graphs still reference has been seen to block at exit.
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="engine steps to time; 0 = the whole workload")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="xllm_b200", choices=["xllm_b200", "ours", "reference"])
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--requests", type=int, default=1024)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=512)
    ap.add_argument("--concurrency", type=int, default=256)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--max-tokens-per-batch", type=int, default=16384)
    ap.add_argument("--max-memory-utilization", type=float, default=0.9)
    ap.add_argument("--num-blocks", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-overlap", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REF_UNAVAILABLE}), flush=True)
        return 0
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world == 1:
        # convenience: re-launch under torchrun when started as a plain script
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29533"),
               os.path.abspath(__file__)] + sys.argv[1:]
        return subprocess.call(cmd)
    run(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
