"""Serving benchmark over HTTP: N concurrent streaming clients against the OpenAI-compatible server,
on the same model / lengths / concurrency as the offline benchmark, so that the two numbers can be
compared (the serving stack - request pool, engine loop, native response pool, epoll transport -
should cost a few per cent at most).

    python benchmarks/serve_bench.py --model qwen3-8b --concurrency 256 --requests 512 \
        --input-len 1024 --output-len 512

The server runs in this process (the engine loop is the main thread); the load generator is a child
process (asyncio, raw sockets) so that it does not share the interpreter lock with the server.
Prints one JSON line: output tokens/s over the wall clock of the whole run, TTFT / TPOT p50 as seen by
the clients.  Parity: the reference is measured the same way, through its HTTP endpoint
(xllm/api_service/api_service.cpp, benchmark scripts under xllm's docs).
"""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import random
import subprocess
import sys
import tempfile
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def synthetic_tokenizer_file(vocab_size: int, path: str):
    """A byte-level BPE tokenizer.json with `vocab_size` entries and no merges: every id decodes to a
    few bytes of text, which is all the response path needs."""
    # the GPT-2 byte <-> printable-character table of byte-level BPE vocabularies
    keep = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    b2u, extra = {}, 0
    for b in range(256):
        if b in keep:
            b2u[b] = chr(b)
        else:
            b2u[b] = chr(256 + extra)
            extra += 1
    vocab = {}
    for b in range(256):
        vocab[b2u[b]] = len(vocab)
    i = 0
    while len(vocab) < vocab_size:
        w = "Ġw" + str(i)          # 'Ġw123' = " w123"
        if w not in vocab:
            vocab[w] = len(vocab)
        i += 1
    obj = {"version": "1.0", "added_tokens": [], "normalizer": None,
           "pre_tokenizer": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": True},
           "decoder": {"type": "ByteLevel"}, "model": {"type": "BPE", "vocab": vocab, "merges": []}}
    with open(path, "w") as f:
        json.dump(obj, f)


# ------------------------------------------------------------------------------------------ client
async def _one_request(host, port, body: bytes, stats: dict):
    t0 = time.perf_counter()
    reader, writer = await asyncio.open_connection(host, port)
    writer.write(b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: "
                 + str(len(body)).encode() + b"\r\nConnection: close\r\n\r\n" + body)
    await writer.drain()
    first = None
    last = t0
    n_chunks = 0
    completion_tokens = 0
    buf = b""
    finished = False
    while not finished:
        data = await reader.read(65536)
        if not data:
            break
        now = time.perf_counter()
        buf += data
        while b"\n\n" in buf:
            ev, buf = buf.split(b"\n\n", 1)
            k = ev.find(b"data: ")
            if k < 0:
                continue
            payload = ev[k + 6:]
            if payload.startswith(b"[DONE]"):
                finished = True         # the server keeps the connection alive: do not wait for EOF
                continue
            if b'"usage"' in payload:
                try:
                    completion_tokens = json.loads(payload)["usage"]["completion_tokens"]
                except Exception:
                    pass
                continue
            if first is None:
                first = now
            last = now
            n_chunks += 1
    writer.close()
    stats["ttft"].append((first or last) - t0)
    if completion_tokens > 1 and first is not None:
        stats["tpot"].append((last - first) / (completion_tokens - 1))
    stats["tokens"] += completion_tokens
    stats["done"] += 1


async def _client_main(host, port, concurrency, requests, input_len, output_len, vocab, seed):
    rng = random.Random(seed)
    stats = {"ttft": [], "tpot": [], "tokens": 0, "done": 0}
    sem = asyncio.Semaphore(concurrency)

    async def worker(i):
        ids = [rng.randrange(300, vocab - 1000) for _ in range(input_len)]
        body = json.dumps({"prompt": ids, "max_tokens": output_len, "temperature": 0, "ignore_eos": True, "stream": True,
                           "stream_options": {"include_usage": True}}).encode()
        async with sem:
            await _one_request(host, port, body, stats)

    t0 = time.perf_counter()
    await asyncio.gather(*[worker(i) for i in range(requests)])
    dt = time.perf_counter() - t0
    med = lambda v: sorted(v)[len(v) // 2] if v else 0.0
    print(json.dumps({"seconds": dt, "output_tokens": stats["tokens"], "requests_done": stats["done"],
                      "ttft_p50_ms": med(stats["ttft"]) * 1e3, "tpot_p50_ms": med(stats["tpot"]) * 1e3}), flush=True)


def client_entry(argv):
    host, port, conc, reqs, il, ol, vocab, seed = argv
    asyncio.run(_client_main(host, int(port), int(conc), int(reqs), int(il), int(ol), int(vocab), int(seed)))


# ------------------------------------------------------------------------------------------ server
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--client", nargs=8, default=None, help=argparse.SUPPRESS)
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--device", default="")
    ap.add_argument("--concurrency", type=int, default=256)
    ap.add_argument("--requests", type=int, default=512)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=512)
    ap.add_argument("--chunk", type=int, default=2048)
    ap.add_argument("--request-threads", type=int, default=4)
    ap.add_argument("--response-threads", type=int, default=4)
    ap.add_argument("--warmup-requests", type=int, default=32)
    ap.add_argument("--no-tokenizer", action="store_true", help="serve token ids only (no detokenisation)")
    args = ap.parse_args()
    if args.client:
        return client_entry(args.client)

    import torch
    from xllm_b200 import LLM, _rt
    from xllm_b200.api.server import ApiServer
    from xllm_b200.utils.tokenizer import TokenizerWrapper

    dev = args.device or ("cuda:0" if torch.cuda.is_available() else "cpu")
    cuda = dev.startswith("cuda")
    conc = args.concurrency
    llm = LLM(args.model, devices=dev, dtype="bfloat16" if cuda else "float32", block_size=16,
              max_seqs_per_batch=conc, max_tokens_per_batch=conc + args.chunk,
              max_tokens_per_chunk_for_prefill=args.chunk, max_model_len=args.input_len + args.output_len + 16,
              enable_prefix_cache=False, enable_chunked_prefill=True, enable_schedule_overlap=cuda, enable_graph=cuda,
              policy="decode_first", random_weights=True, min_prefill_tokens=args.chunk if cuda else 0,
              max_prefill_wait_steps=16)
    eng = llm.engine
    tok = None
    if not args.no_tokenizer:
        d = tempfile.mkdtemp(prefix="servebench_")
        path = os.path.join(d, "tokenizer.json")
        synthetic_tokenizer_file(eng.args.vocab_size, path)
        impl = _rt.BpeTokenizer()
        impl.load_hf_file(path)
        tok = TokenizerWrapper(impl, "", {}, "qwen3")
    srv = ApiServer(eng, tok, model_name=args.model, host="127.0.0.1", port=0, max_concurrent_requests=4 * conc,
                    request_threads=args.request_threads, response_threads=args.response_threads)
    result = {}

    def drive():
        me = os.path.abspath(__file__)
        common = ["127.0.0.1", str(srv.port)]
        if args.warmup_requests:
            subprocess.run([sys.executable, me, "--client", *common, str(min(conc, args.warmup_requests)),
                            str(args.warmup_requests), str(args.input_len), "8", str(eng.args.vocab_size), "1"],
                           capture_output=True, text=True)
        r = subprocess.run([sys.executable, me, "--client", *common, str(conc), str(args.requests), str(args.input_len),
                            str(args.output_len), str(eng.args.vocab_size), "2"], capture_output=True, text=True)
        try:
            result.update(json.loads(r.stdout.strip().splitlines()[-1]))
        except Exception:
            result["error"] = (r.stdout + r.stderr)[-800:]
        srv.shutdown()

    t = threading.Thread(target=drive, daemon=True)
    t.start()
    srv.serve_forever(idle_poll_ms=2)
    t.join(timeout=30)
    line = {"metric": "output_tokens_per_s", "unit": "tokens/s", "transport": "http+sse", "model": args.model,
            "concurrency": conc, "requests": args.requests, "input_len": args.input_len, "output_len": args.output_len,
            "request_threads": args.request_threads, "response_threads": args.response_threads if srv.rp else 0,
            "detokenize": tok is not None}
    if "error" in result:
        line["error"] = result["error"]
    else:
        line.update(value=round(result["output_tokens"] / result["seconds"], 1), seconds=round(result["seconds"], 2),
                    requests_done=result["requests_done"], ttft_p50_ms=round(result["ttft_p50_ms"], 1),
                    tpot_p50_ms=round(result["tpot_p50_ms"], 2))
    print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
