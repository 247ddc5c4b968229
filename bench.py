#!/usr/bin/env python
"""Serving benchmark: output tokens/s, p50 TTFT and p50 TPOT of the closed-loop workloads of
BASELINE.json on N GPUs of one node.

    python bench.py --gpus 1                        # config 2, whole workload (1024 requests)
    python bench.py --gpus 1 --steps 20 --warmup 5  # config 2, K steps of the steady state
    python bench.py --gpus 8 --config 3 --steps 20  # Qwen3-32B shape, chunked 2048-token prefill
    python bench.py --gpus 8 --config 4 --steps 20  # Qwen3-30B-A3B shape, EP + DP attention

Workload (config 2): Qwen3-8B-shaped bf16 decoder, random-init weights, 1024 requests of uniform
random token ids, input 1024 / output 512 with ignore_eos, at most 256 requests in flight (a closed
loop: a finished request admits the next one), paged KV with block 16, CUDA graphs, TP = --gpus.
The scheduler mixes decode rows and prompt chunks in one step (decode_first: every running sequence
decodes, the rest of the token budget goes to prompt chunks), so a step costs one launch of one graph;
prompt work is batched: it is held back until 2048 prompt tokens are pending, because one 2048-token
chunk every fourth step runs its GEMMs at the compute-bound rate while a 512-token chunk in every step
does not.

A "step" is one engine iteration: one scheduled batch -> one forward pass -> one sampled token per
scheduled sequence.  Without --steps the whole workload is timed from a cold queue.  With --steps K
exactly K steps of the workload's STEADY STATE are timed: a closed loop with requests of one length
settles into a regime where, per step, every one of the 256 sequences decodes and 256/512 = 1/2 of a
request finishes and is replaced, i.e. 512 prompt tokens per step on average (two 1024-token prompts
every fourth step).  The set-up (untimed)
builds that regime directly: 256 sequences whose remaining output lengths are staggered 2, 4, ... 512
(their prompts carry the tokens "generated so far", so KV lengths are those of requests in mid
flight).  Then W warm-up steps and K timed steps run it; finished requests are replaced by fresh
1024-token requests inside the window.  Timing is CUDA events around the step loop, bracketed by
barrier + synchronize, max over ranks.  TTFT / TPOT are host clock: submission -> first token
on the host, and the mean gap between a request's tokens.

The `e2e` block runs the whole workload (all requests, same shape, same concurrency, full output
length, from a cold queue) through the public API (`LLM.generate`) on the host clock; every step of both runs copies its inputs
from pinned host memory and reads the sampled tokens back.

`--impl reference` is the arm for the unmodified upstream engine; it cannot be installed offline,
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

# name -> (model preset, input_len, output_len, concurrency, requests, prompt chunk, parallelism)
CONFIGS = {
    "2": dict(model="qwen3-8b", input_len=1024, output_len=512, concurrency=256, requests=1024, chunk=2048,
              parallelism="tp"),
    "3": dict(model="qwen3-32b", input_len=4096, output_len=256, concurrency=64, requests=256, chunk=2048,
              parallelism="tp"),
    "4": dict(model="qwen3-30b-a3b", input_len=2048, output_len=512, concurrency=512, requests=1024, chunk=2048,
              parallelism="ep"),
}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0, period_ms=100):
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


def make_requests(n, length, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    # token ids live in pinned host memory: the engine's per-step H2D copy starts from them
    ids = torch.randint(0, vocab, (n, length), generator=g, dtype=torch.int64)
    if torch.cuda.is_available():
        ids = ids.pin_memory()
    return ids


def p50(xs):
    xs = [x for x in xs if x is not None]
    return statistics.median(xs) if xs else None


class Tracker:
    """Host-side request timing: submission, first token, last token, token count."""

    def __init__(self):
        self.t_submit, self.t_first, self.t_last, self.n_tok = {}, {}, {}, {}

    def submit(self, rid, now):
        self.t_submit[rid] = now

    def token(self, rid, now):
        if rid not in self.t_first:
            self.t_first[rid] = now
            self.n_tok[rid] = 0
        self.t_last[rid] = now
        self.n_tok[rid] += 1

    def ttft_ms(self, since=0.0):
        return p50([(self.t_first[r] - t) * 1e3 for r, t in self.t_submit.items() if r in self.t_first and t >= since])

    def tpot_ms(self):
        return p50([(self.t_last[r] - self.t_first[r]) * 1e3 / (n - 1) for r, n in self.n_tok.items() if n > 1])


def run(args):
    import torch
    import torch.distributed as dist

    from xllm_b200 import LLM, SamplingParams, ops
    from xllm_b200.parallel.state import init_parallel

    cfg = CONFIGS[args.config]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    ep = cfg["parallelism"] == "ep" and world > 1
    ps = None
    if world > 1:
        ps = init_parallel(dp_size=world, ep_size=world) if ep else init_parallel()
    rank = ps.rank if ps else 0
    dev = ps.device if ps else torch.device("cuda", 0)
    torch.cuda.set_device(dev)

    in_len, out_len = args.input_len or cfg["input_len"], args.output_len or cfg["output_len"]
    conc_total = args.concurrency or cfg["concurrency"]
    n_req_total = args.requests or cfg["requests"]
    chunk = args.chunk or cfg["chunk"]
    # with data-parallel attention every rank serves its own share of the requests
    conc = conc_total // world if ep else conc_total
    n_req = n_req_total // world if ep else n_req_total
    budget = args.max_tokens_per_batch or (conc + chunk)
    min_prefill = chunk if args.prefill_batch < 0 else args.prefill_batch
    max_len = in_len + out_len + 16
    llm = LLM(args.model or cfg["model"], devices=str(dev), dtype="bfloat16", block_size=args.block_size,
              max_seqs_per_batch=conc, max_tokens_per_batch=max(budget, 4096 if args.steps > 0 else budget),
              max_tokens_per_chunk_for_prefill=chunk, max_model_len=max_len, enable_prefix_cache=False,
              enable_chunked_prefill=True, enable_schedule_overlap=not args.no_overlap,
              enable_graph=not args.no_graph, policy="decode_first", random_weights=True, parallel_state=ps,
              max_memory_utilization=args.max_memory_utilization, num_blocks=args.num_blocks,
              dp_size=world if ep else 1, ep_size=world if ep else 1, min_prefill_tokens=min_prefill,
              max_prefill_wait_steps=16)
    eng = llm.engine
    vocab = eng.args.vocab_size
    sched = eng.scheduler

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def unfinished():
        return eng.dp_has_unfinished() if ep else eng.has_unfinished()

    track = Tracker()
    counters = {"tokens": 0, "in_flight": 0, "cursor": 0}

    def add(rid, ids, max_tokens):
        eng.add_request(rid, ids, temperature=0.0, max_tokens=max_tokens, ignore_eos=True, offline=True)
        track.submit(rid, time.perf_counter())
        counters["in_flight"] += 1

    def step():
        evs = eng.step()
        now = time.perf_counter()
        for ev in evs:
            if ev.token >= 0:
                counters["tokens"] += 1
                track.token(ev.request_id, now)
            if ev.request_finished:
                counters["in_flight"] -= 1
        return evs

    reqs = make_requests(n_req, in_len, vocab, 100 + rank)

    def submit_more():
        while counters["cursor"] < n_req and counters["in_flight"] < conc:
            i = counters["cursor"]
            add(f"r-{i}", reqs[i].tolist(), out_len)
            counters["cursor"] += 1

    # ---------------------------------------------------------------- set-up (untimed)
    window = args.steps > 0
    wsteps = 0
    if window:
        # the steady state, built directly: sequence j has out_len - r_j tokens behind it and r_j to go
        sched.reconfigure("prefill_first", max(budget, 4096), conc, 0)
        rem = [max(1, (j + 1) * out_len // conc) for j in range(conc)]
        cohort = make_requests(conc, in_len + out_len, vocab, 7 + rank)
        for j in range(conc):
            add(f"c-{j}", cohort[j, : in_len + out_len - rem[j]].tolist(), rem[j] + 1)
        while sched.num_waiting > 0 or sched.num_prefilling > 0:
            step()
        for ev in eng.drain():
            if ev.request_finished:
                counters["in_flight"] -= 1
        sched.reconfigure("decode_first", budget, conc, chunk)
        # both shapes of the regime are captured before any step is timed
        eng.runner.warmup([conc], prefill_tokens=[t for t in eng.runner.prefill_buckets if t >= min(chunk, budget - conc)][:1])
        counters["tokens"] = 0
    else:
        # graphs and kernels warm, nothing of the workload started
        warm = make_requests(min(8, conc), min(in_len, 256), vocab, 1)
        for i in range(warm.shape[0]):
            add(f"w-{i}", warm[i].tolist(), max(4, args.warmup))
        while unfinished():
            step()
            wsteps += 1
        eng.drain()
        eng.runner.warmup([conc], prefill_tokens=[t for t in eng.runner.prefill_buckets if t >= min(chunk, budget - conc)][:1])
        counters["tokens"] = 0
        counters["in_flight"] = 0
    barrier()
    if window:
        submit_more()
        while wsteps < args.warmup:       # W steps of the regime that is timed (captures its graphs)
            step()
            submit_more()
            wsteps += 1
        barrier()

    # the window starts with nothing in flight: tokens of earlier steps are accounted before it
    now = time.perf_counter()
    for ev in eng.drain():
        if ev.token >= 0:
            counters["tokens"] += 1
            track.token(ev.request_id, now)
        if ev.request_finished:
            counters["in_flight"] -= 1
    if window:
        track.__init__()              # TTFT / TPOT of the window only
    if args.profile:
        profile_steps(eng, step, submit_more, args.profile, rank)

    # ---------------------------------------------------------------- timed run (device clock)
    sampler = ClockSampler(dev.index or 0)
    launches0, glaunch0, replays0 = ops.launches(), eng.runner.graph_launches, eng.runner.graph_replays
    h2d0, d2h0 = eng.runner.h2d_bytes, eng.runner.d2h_bytes
    tok0 = counters["tokens"]
    t_window = time.perf_counter()
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    steps = 0
    total_target = args.steps if window else 1 << 60
    submit_more()
    while steps < total_target and (unfinished() or counters["cursor"] < n_req):
        step()
        steps += 1
        submit_more()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    # tokens of the step still in flight (overlap mode) belong to the timed region as well
    now = time.perf_counter()
    for ev in eng.drain():
        if ev.token >= 0:
            counters["tokens"] += 1
            track.token(ev.request_id, now)
    out_tokens = counters["tokens"] - tok0
    graph_replays = eng.runner.graph_replays - replays0
    gpu_launches = (ops.launches() - launches0) + (eng.runner.graph_launches - glaunch0)
    h2d_step = (eng.runner.h2d_bytes - h2d0) / max(steps, 1)
    d2h_step = (eng.runner.d2h_bytes - d2h0) / max(steps, 1)
    ttft, tpot = track.ttft_ms(since=t_window if window else 0.0), track.tpot_ms()
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        if ep:      # every rank produced its own tokens
            t = torch.tensor([float(out_tokens)], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            out_tokens = int(t.item())
    value = out_tokens / (ms / 1e3)

    # abort whatever the K-step window left unfinished, then the end-to-end run
    if eng.has_unfinished():
        for j in range(conc):
            eng.abort(f"c-{j}")
        for i in range(counters["cursor"]):
            eng.abort(f"r-{i}")
    while unfinished():
        eng.step()
    eng.drain()
    e2e = None
    if not args.no_e2e:
        n_e2e = n_req if args.e2e_requests <= 0 else min(n_req, args.e2e_requests)
        reqs2 = make_requests(n_e2e, in_len, vocab, 200 + rank)
        prompts = [reqs2[i] for i in range(n_e2e)]  # pinned host tensors handed to the public API
        sp = SamplingParams(max_tokens=out_len, temperature=0.0, ignore_eos=True)
        h2d0, d2h0, s0 = eng.runner.h2d_bytes, eng.runner.d2h_bytes, eng.steps
        barrier()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp, max_concurrency=conc)
        barrier()
        dt = time.perf_counter() - t0
        gen = sum(o.usage.num_generated_tokens for o in outs)
        if world > 1:
            t = torch.tensor([dt], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
            if ep:
                t = torch.tensor([float(gen)], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.SUM)
                gen = int(t.item())
        nst = max(eng.steps - s0, 1)
        e2e = {"value": gen / dt, "unit": "output tok/s", "requests": n_e2e * (world if ep else 1),
               "output_len": out_len, "seconds": dt, "steps": nst,
               "ttft_p50_ms": p50([m["ttft_ms"] for m in (o.metrics for o in outs) if m]),
               "tpot_p50_ms": p50([m["tpot_ms"] for m in (o.metrics for o in outs) if m]),
               "h2d_bytes_per_step": (eng.runner.h2d_bytes - h2d0) / nst,
               "d2h_bytes_per_step": (eng.runner.d2h_bytes - d2h0) / nst}

    if rank == 0:
        name = args.model or cfg["model"]
        par = (f"ep{world}+dp{world}" if ep else f"tp{world}")
        line = {
            "metric": "output tok/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": steps,
            "warmup": wsteps if not window else args.warmup, "ms_per_step": ms / max(steps, 1),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "impl": "xllm_b200", "ttft_p50_ms": ttft, "tpot_p50_ms": tpot,
            "config": {"name": f"BASELINE.json config #{args.config}",
                       "model": f"{name} (random-init weights of that architecture)",
                       "requests": n_req_total, "input_len": in_len, "output_len": out_len,
                       "concurrency": conc_total, "global_batch": conc_total, "seq_len": in_len + out_len,
                       "block_size": args.block_size, "parallelism": par, "cuda_graphs": not args.no_graph,
                       "schedule_overlap": not args.no_overlap, "policy": "decode_first",
                       "tokens_per_step_budget": budget, "prefill_chunk": chunk, "min_prefill_tokens": min_prefill,
                       "window": ("whole workload from a cold queue" if not window else
                                  f"{steps} steps of the steady state of the closed loop: every step decodes the "
                                  f"running sequences (up to {conc_total}); finished requests are replaced, their prompts "
                                  f"prefilled in chunks of up to {chunk} tokens once {min_prefill} prompt tokens are pending"),
                       "l2": "inputs larger than L2: every step streams the weights and the KV cache of all running "
                             "sequences (tens of GB)",
                       "output_tokens": out_tokens, "kv_blocks": eng.num_blocks},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(gpu_launches), "graph_replays": int(graph_replays),
            "h2d_bytes_per_step": h2d_step, "d2h_bytes_per_step": d2h_step,
        }
        from xllm_b200.ops import gemm as _gemm
        line["library_gemm_fallbacks"] = int(sum(_gemm.library_fallbacks().values()))
        line["vs_library"] = _vs_library(args.config, world, n_req_total, in_len, out_len, conc_total,
                                         e2e.get("value") if isinstance(e2e, dict) else None)
        print(json.dumps(line), flush=True)
    if world > 1:
        # Every collective of this process finished behind the barrier that closed the last timed
        # region, so nothing is in flight.  Leave without tearing the process group down: destroying
        # NCCL communicators that CUDA graphs still reference has been seen to block at exit.
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def profile_steps(eng, step, submit_more, n, rank):
    """Per-kernel device time of n steps of the regime about to be timed (CUPTI activity records through
    the PyTorch profiler), printed to stderr by rank 0.  Runs before the timed region, never inside it."""
    import collections

    import torch
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(n):
            step()
            submit_more()
        torch.cuda.synchronize()
    eng.drain()
    per = collections.defaultdict(lambda: [0.0, 0])
    total = 0.0
    for ev in prof.events():
        dt = getattr(ev, "device_time", 0) or getattr(ev, "cuda_time", 0)
        if dt and ev.device_type is not None and "cuda" in str(ev.device_type).lower():
            per[ev.name][0] += dt
            per[ev.name][1] += 1
            total += dt
    if rank == 0:
        print(f"profile: {n} steps, device busy {total / 1e3 / n:.2f} ms/step", file=sys.stderr)
        for name, (us, k) in sorted(per.items(), key=lambda kv: -kv[1][0])[:24]:
            print(f"{us / 1e3 / n:8.3f} ms/step {100 * us / total:5.1f}%  n/step {k / n:7.1f}  avg {us / k:8.1f} us  "
                  f"{name[:100]}", file=sys.stderr)


def _vs_library(config, n_gpus, requests, in_len, out_len, conc, e2e_value):
    """End-to-end value over the LIBRARY arm's measured value for the same workload
    (baseline/library_results.json, filled from `bench.py --impl library` runs), or None."""
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "library_results.json")
    if e2e_value is None or not os.path.exists(path):
        return None
    try:
        with open(path) as f:
            rows = json.load(f)["results"]
    except (OSError, ValueError, KeyError):
        return None
    for r in rows:
        if (str(r.get("config")) == str(config) and r.get("n_gpus") == n_gpus and r.get("requests") == requests
                and r.get("input_len") == in_len and r.get("output_len") == out_len and r.get("concurrency") == conc):
            return round(float(e2e_value) / float(r["value"]), 4)
    return None


def run_library(args):
    """The same workload through the all-library engine of the image (vLLM: cuBLAS + NCCL +
    FlashAttention/FlashInfer + CUDA graphs), whole workload, end to end.  Prints one JSON line with
    "impl": "library"; it is never the reference arm.  Under a multi-rank launcher only rank 0 runs
    it (the library spawns its own workers on the GPUs of the node)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT", "TORCHELASTIC_RUN_ID",
              "GROUP_RANK", "ROLE_RANK", "LOCAL_WORLD_SIZE", "ROLE_WORLD_SIZE", "GROUP_WORLD_SIZE"):
        os.environ.pop(k, None)
    cfg = CONFIGS[args.config]
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline"))
    line = {"impl": "library", "metric": "output_tokens_per_s", "unit": "tokens/s", "n_gpus": args.gpus,
            "higher_is_better": True, "dtype": "bf16", "data": "synthetic token ids, random-init weights",
            "config": {"model": args.model or cfg["model"], "input_len": args.input_len or cfg["input_len"],
                       "output_len": args.output_len or cfg["output_len"],
                       "concurrency": args.concurrency or cfg["concurrency"],
                       "requests": args.requests or cfg["requests"], "window": "whole workload, wall clock around generate()"}}
    try:
        import library_vllm
        c = line["config"]
        r = library_vllm.run(c["model"], args.gpus, c["input_len"], c["output_len"], c["concurrency"], c["requests"],
                             args.chunk or cfg["chunk"], warmup_requests=min(64, c["concurrency"]),
                             expert_parallel=cfg["parallelism"] == "ep", attention_backend=args.library_attention)
        line.update(value=round(r["value"], 1), seconds=round(r["seconds"], 2), library=r["library"],
                    attention_backend=r["attention_backend"], init_seconds=round(r["init_seconds"], 1))
    except BaseException as e:  # noqa: BLE001 - the arm reports why it could not run
        line["unavailable"] = f"{type(e).__name__}: {str(e)[:300]}"
    print(json.dumps(line), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="steady-state engine steps to time; 0 = the whole workload")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="xllm_b200", choices=["xllm_b200", "ours", "reference", "library"])
    ap.add_argument("--library-attention", default="", help="library arm: attention backend name handed to vLLM")
    ap.add_argument("--config", default="2", choices=sorted(CONFIGS), help="BASELINE.json config number")
    ap.add_argument("--model", default="")
    ap.add_argument("--requests", type=int, default=0)
    ap.add_argument("--input-len", type=int, default=0)
    ap.add_argument("--output-len", type=int, default=0)
    ap.add_argument("--concurrency", type=int, default=0)
    ap.add_argument("--chunk", type=int, default=0, help="prompt tokens per step (and per chunk)")
    ap.add_argument("--prefill-batch", type=int, default=-1,
                    help="hold prompt work back until this many prompt tokens are pending (-1: --chunk, 0: never hold)")
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--max-tokens-per-batch", type=int, default=0)
    ap.add_argument("--max-memory-utilization", type=float, default=0.9)
    ap.add_argument("--num-blocks", type=int, default=0)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-overlap", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-requests", type=int, default=0, help="requests of the end-to-end run (0: the whole workload)")
    ap.add_argument("--profile", type=int, default=0, help="print a per-kernel breakdown of this many steps first")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REF_UNAVAILABLE}), flush=True)
        return 0
    if args.impl == "library":
        return run_library(args)
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
