#!/usr/bin/env python
"""Generative recommendation end to end: R histories, beam width W, items of S tokens, through `LLM.recommend`
(batched prompt prefill, beam rounds with x-attention over the shared prompt pages, selection kernels).

    python benchmarks/rec_bench.py --model qwen3-8b --requests 16 --history 1024 --beam 128 --steps 3
    python benchmarks/rec_bench.py --catalogue 1000000      # beams restricted to a catalogue of that many items

Prints one JSON line: items per second, requests per second, milliseconds per call (CUDA events around the
calls after warm-up; inputs are copied from the host every call)."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from xllm_b200 import LLM  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--requests", type=int, default=16)
    ap.add_argument("--history", type=int, default=1024)
    ap.add_argument("--beam", type=int, default=128)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--catalogue", type=int, default=0, help="restrict the beams to this many random items (0: no catalogue)")
    ap.add_argument("--codebook", type=int, default=8192, help="distinct tokens per item position of the catalogue")
    a = ap.parse_args()
    llm = LLM(a.model, devices="cuda:0", dtype="bfloat16", block_size=16, max_seqs_per_batch=max(8, a.requests),
              max_tokens_per_batch=max(8192, a.requests * a.history), enable_graph=False, enable_prefix_cache=False,
              random_weights=True, max_memory_utilization=0.5)
    V = llm.engine.args.vocab_size
    g = torch.Generator().manual_seed(0)
    hist = [torch.randint(0, V, (a.history,), generator=g).tolist() for _ in range(a.requests)]
    trie = None
    if a.catalogue:
        from xllm_b200.engine.rec import ItemTrie
        trie = ItemTrie(torch.randint(0, min(a.codebook, V), (a.catalogue, a.steps), generator=g).numpy(), V, device="cuda:0")
    for _ in range(2):
        out = llm.recommend(hist, beam_width=a.beam, num_steps=a.steps, valid_items=trie)
    assert len(out) == a.requests and len(out[0]) == a.beam
    if trie is not None:
        assert all(tuple(it.token_ids) in trie for it in out[0][:8])
    ts = []
    for _ in range(a.iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        llm.recommend(hist, beam_width=a.beam, num_steps=a.steps, valid_items=trie)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ms = sorted(ts)[len(ts) // 2]
    print(json.dumps({"metric": "recommended items per second", "value": round(a.requests * a.beam / ms * 1e3, 1),
                      "requests_per_s": round(a.requests / ms * 1e3, 2), "ms_per_call": round(ms, 2), "model": a.model,
                      "requests": a.requests, "history_tokens": a.history, "beam_width": a.beam, "item_tokens": a.steps, "catalogue_items": 0 if trie is None else trie.n_items,
                      "dtype": "bf16", "data": "synthetic token ids, random-init weights"}))


if __name__ == "__main__":
    main()
