"""HTTP service end to end on CPU with the tiny model: completions (plain + SSE), chat with a
tokenizer and chat template, admin routes, health, metrics, disconnect handling."""
import http.client
import json
import threading
import time

import pytest
import torch

from xllm_b200 import _rt
from xllm_b200.api.server import ApiServer
from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
from xllm_b200.utils.tokenizer import TokenizerWrapper


def _tokenizer(tmp_path):
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=400, special_tokens=["<|im_start|>", "<|im_end|>", "<|endoftext|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(["hello world this is a tiny corpus for the server test " * 5, "user assistant system\n"], trainer)
    p = tmp_path / "tokenizer.json"
    tok.save(str(p))
    impl = _rt.BpeTokenizer()
    impl.load_hf_file(str(p))
    return TokenizerWrapper(impl, "", {}, "qwen3")


@pytest.fixture()
def server(tmp_path):
    eng = LLMEngine(EngineConfig(model="tiny", device="cpu", dtype="float32", num_blocks=128, enable_graph=False,
                                 max_seqs_per_batch=8, max_tokens_per_batch=256))
    srv = ApiServer(eng, _tokenizer(tmp_path), model_name="tiny", host="127.0.0.1", port=0,
                    reasoning_parser="qwen3", tool_call_parser="qwen25")
    t = threading.Thread(target=srv.serve_forever, args=(10,), daemon=True)
    t.start()
    yield srv
    srv.shutdown()
    t.join(timeout=5)


def _post(port, path, body, stream=False):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=60)
    c.request("POST", path, json.dumps(body), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read().decode()
    c.close()
    return r.status, data


def test_completions_plain_and_stream(server):
    st, data = _post(server.port, "/v1/completions", {"prompt": [5, 6, 7, 8, 9], "max_tokens": 6, "temperature": 0,
                                                      "ignore_eos": True})
    assert st == 200
    obj = json.loads(data)
    assert obj["object"] == "text_completion" and obj["usage"]["completion_tokens"] == 6
    assert obj["choices"][0]["finish_reason"] == "length"
    text = obj["choices"][0]["text"]
    st, data = _post(server.port, "/v1/completions", {"prompt": [5, 6, 7, 8, 9], "max_tokens": 6, "temperature": 0,
                                                      "ignore_eos": True, "stream": True,
                                                      "stream_options": {"include_usage": True}})
    assert st == 200
    events = [json.loads(l[6:]) for l in data.split("\n") if l.startswith("data: ") and l != "data: [DONE]"]
    assert data.rstrip().endswith("data: [DONE]")
    assert "".join(e["choices"][0]["text"] for e in events if e["choices"]) == text
    assert events[-1]["usage"]["completion_tokens"] == 6


def test_chat_models_health_metrics_admin(server):
    st, data = _post(server.port, "/v1/chat/completions", {"messages": [{"role": "user", "content": "hello world"}],
                                                           "max_tokens": 5, "temperature": 0, "ignore_eos": True})
    assert st == 200
    obj = json.loads(data)
    assert obj["object"] == "chat.completion" and obj["choices"][0]["message"]["role"] == "assistant"
    assert obj["usage"]["prompt_tokens"] > 5
    st, data = _post(server.port, "/v1/messages", {"messages": [{"role": "user", "content": "hello"}], "system": "s",
                                                   "max_tokens": 4, "temperature": 0, "ignore_eos": True})
    assert st == 200 and json.loads(data)["type"] == "message" and json.loads(data)["stop_reason"] == "max_tokens"
    c = http.client.HTTPConnection("127.0.0.1", server.port, timeout=10)
    c.request("GET", "/v1/models")
    assert json.loads(c.getresponse().read())["data"][0]["id"] == "tiny"
    c.request("GET", "/health")
    r = c.getresponse()
    assert r.status == 200 and json.loads(r.read())["status"] == "ok"
    c.request("GET", "/metrics")
    m = c.getresponse().read().decode()
    assert "num_generated_tokens_total" in m and "time_to_first_token_latency_milliseconds_bucket" in m
    c.close()
    assert _post(server.port, "/pause", {"mode": "KEEP"})[0] == 200
    assert _post(server.port, "/v1/completions", {"prompt": [1, 2, 3], "max_tokens": 2})[0] == 503
    assert _post(server.port, "/resume", {})[0] == 200
    assert _post(server.port, "/v1/completions", {"prompt": [1, 2, 3], "max_tokens": 2, "ignore_eos": True})[0] == 200
    assert _post(server.port, "/v1/nope", {})[0] == 404
    st, data = _post(server.port, "/v1/embeddings", {"input": ["hello world", "tiny corpus"]})
    assert st == 200 and len(json.loads(data)["data"]) == 2 and len(json.loads(data)["data"][0]["embedding"]) == 256
    server.healthy, server.unhealthy_reason = False, "worker 1 did not answer"
    c = http.client.HTTPConnection("127.0.0.1", server.port, timeout=10)
    c.request("GET", "/health")
    r = c.getresponse()
    assert r.status == 503 and "worker 1" in r.read().decode()
    c.close()


def test_client_disconnect_aborts_request(server):
    import socket
    s = socket.create_connection(("127.0.0.1", server.port))
    body = json.dumps({"prompt": list(range(3, 40)), "max_tokens": 2000, "ignore_eos": True, "stream": True})
    s.sendall(f"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Length: {len(body)}\r\n\r\n{body}".encode())
    s.recv(200)
    s.close()
    for _ in range(400):
        if not server.engine.has_unfinished() and not server.calls:
            break
        time.sleep(0.02)
    assert not server.calls and not server.engine.has_unfinished()
    assert server.engine.stats()["kv_utilization"] == 0.0


def test_rerank_and_sample_routes(server):
    st, data = _post(server.port, "/v1/rerank", {"query": "hello world", "documents": ["hello world", "tiny corpus", "user"],
                                                 "top_n": 2})
    assert st == 200
    obj = json.loads(data)
    assert len(obj["results"]) == 2 and obj["results"][0]["index"] == 0          # the identical text ranks first
    assert obj["results"][0]["relevance_score"] >= obj["results"][1]["relevance_score"]
    st, data = _post(server.port, "/v1/sample", {"prompt": "this is a tiny corpus for this test", "logprobs": 3,
                                                 "selector": {"type": "literal", "value": "this"}})
    assert st == 200
    obj = json.loads(data)
    assert obj["object"] == "sample_completion" and len(obj["choices"]) == 2     # "this" occurs twice
    for c in obj["choices"]:
        lp = c["logprobs"]["token_logprobs"]
        assert len(lp) == 3 and lp[0] >= lp[1] >= lp[2] and lp[0] <= 0
    st, _ = _post(server.port, "/v1/sample", {"prompt": "x", "selector": {"type": "regex", "value": "x"}})
    assert st == 400


def test_image_generation_route(server):
    import base64
    import struct
    import zlib
    st, data = _post(server.port, "/v1/images/generations", {"prompt": "a red square", "n": 2, "size": "32x24", "steps": 6})
    data = json.loads(data)
    assert st == 200 and len(data["data"]) == 2
    png = base64.b64decode(data["data"][0]["b64_json"])
    assert png[:8] == b"\x89PNG\r\n\x1a\n"
    w, h = struct.unpack(">II", png[16:24])
    assert (w, h) == (32, 24)
    n = struct.unpack(">I", png[33:37])[0]                      # the IDAT chunk follows the 25-byte IHDR chunk
    assert png[37:41] == b"IDAT" and len(zlib.decompress(png[41:41 + n])) == h * (1 + 3 * w)
    st, again = _post(server.port, "/v1/images/generations", {"prompt": "a red square", "size": "32x24", "steps": 6})
    again = json.loads(again)
    assert again["data"][0]["b64_json"] == data["data"][0]["b64_json"]      # the prompt seeds the noise
    st, err = _post(server.port, "/v1/images/generations", {"n": 1})
    assert st == 400


def _raw(port, payload: bytes, read=True, timeout=10):
    import socket
    s = socket.create_connection(("127.0.0.1", port), timeout=timeout)
    s.sendall(payload)
    data = b""
    if read:
        try:
            while True:
                chunk = s.recv(65536)
                if not chunk:
                    break
                data += chunk
        except socket.timeout:
            pass
    s.close()
    return data


def test_malformed_requests_close_their_connection_only(server):
    """A bad Content-Length, an oversized body announcement, a garbled request line and a megabyte
    without an end of headers are each answered (or dropped) and closed; the serving thread lives on."""
    port = server.port
    r = _raw(port, b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Length: abc\r\n\r\n")
    assert r.startswith(b"HTTP/1.1 400") and b"Connection: close" in r
    r = _raw(port, b"POST /v1/completions HTTP/1.1\r\nContent-Length: 99999999999999999999999\r\n\r\n")
    assert r.startswith(b"HTTP/1.1 400")
    r = _raw(port, b"POST /v1/completions HTTP/1.1\r\nContent-Length: 999999999999\r\n\r\n" + b"x" * 100000)
    assert r.startswith(b"HTTP/1.1 413")          # answered and closed although the body kept coming
    r = _raw(port, b"GARBAGE\r\n\r\n")
    assert r.startswith(b"HTTP/1.1 400")
    r = _raw(port, b"A" * (1 << 20) + b"B" * 4096)
    assert r.startswith(b"HTTP/1.1 400") or r == b""
    # still serving
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
    c.request("GET", "/health")
    assert c.getresponse().status == 200
    c.close()


def test_native_response_pool_matches_python_formatting_under_concurrency(tmp_path):
    """The same requests through the C++ response pool and through the Python formatter give the
    same bodies; 24 streaming clients at once keep their chunks in order."""
    tok = _tokenizer(tmp_path)
    outs = {}
    for name, threads in (("native", 3), ("python", 0)):
        eng = LLMEngine(EngineConfig(model="tiny", device="cpu", dtype="float32", num_blocks=256, enable_graph=False,
                                     max_seqs_per_batch=32, max_tokens_per_batch=256))
        srv = ApiServer(eng, tok, model_name="tiny", host="127.0.0.1", port=0, response_threads=threads,
                        request_threads=3 if threads else 0)
        assert (srv.rp is not None) == (threads > 0)
        t = threading.Thread(target=srv.serve_forever, args=(5,), daemon=True)
        t.start()
        res = [None] * 24

        def client(i):
            if i % 2:
                body = {"messages": [{"role": "user", "content": f"hello world {i}"}], "max_tokens": 12, "temperature": 0,
                        "ignore_eos": True, "stream": i % 4 == 1, "stop": ["zzzz"]}
                res[i] = _post(srv.port, "/v1/chat/completions", body)
            else:
                body = {"prompt": [7 + i, 8, 9, 10 + i], "max_tokens": 12, "temperature": 0, "ignore_eos": True,
                        "stream": i % 4 == 0, "stream_options": {"include_usage": True}}
                res[i] = _post(srv.port, "/v1/completions", body)

        ts = [threading.Thread(target=client, args=(i,)) for i in range(24)]
        [x.start() for x in ts]
        [x.join(timeout=120) for x in ts]
        if threads:
            assert srv.rp.drain(5000)
            assert srv.rp.processed >= 24 * 12 and srv.rp.pending == 0
            time.sleep(0.05)                      # one more loop turn collects the finished calls
            assert not srv.calls
        srv.shutdown()
        t.join(timeout=5)
        texts = []
        for i, (st, data) in enumerate(res):
            assert st == 200, data
            if data.startswith("data: "):
                ev = [json.loads(l[6:]) for l in data.split("\n") if l.startswith("data: ") and l != "data: [DONE]"]
                assert data.rstrip().endswith("data: [DONE]")
                if i % 2:
                    texts.append("".join(e["choices"][0]["delta"].get("content", "") for e in ev if e["choices"]))
                    assert ev[0]["choices"][0]["delta"].get("role") == "assistant"
                    assert ev[-1]["choices"][0]["finish_reason"] == "length"
                else:
                    texts.append("".join(e["choices"][0]["text"] for e in ev if e["choices"]))
                    assert ev[-1]["usage"]["completion_tokens"] == 12
            else:
                obj = json.loads(data)
                texts.append(obj["choices"][0]["message"]["content"] if i % 2 else obj["choices"][0]["text"])
                assert obj["usage"]["completion_tokens"] == 12 and obj["choices"][0]["finish_reason"] == "length"
        outs[name] = texts
    assert outs["native"] == outs["python"]


def _spawn_server(tmp_path, **kw):
    eng = LLMEngine(EngineConfig(model="tiny", device="cpu", dtype="float32", num_blocks=128, enable_graph=False,
                                 max_seqs_per_batch=8, max_tokens_per_batch=256, enable_prefix_cache=False))
    srv = ApiServer(eng, _tokenizer(tmp_path), model_name="tiny", host="127.0.0.1", port=0, **kw)
    t = threading.Thread(target=srv.serve_forever, args=(5,), daemon=True)
    t.start()
    return srv, t


def test_fork_master_serves_a_second_model_and_sleeps_it(tmp_path):
    srv, t = _spawn_server(tmp_path)
    try:
        body = {"prompt": [5, 6, 7, 8, 9], "max_tokens": 6, "temperature": 0, "ignore_eos": True}
        st, data = _post(srv.port, "/v1/completions", body)
        base = json.loads(data)["choices"][0]
        st, data = _post(srv.port, "/fork_master", {"model_id": "second", "model": "tiny", "num_blocks": 64})
        assert st == 200 and json.loads(data)["state"] == "READY", data
        assert json.loads(_post(srv.port, "/fork_master", {"model_id": "second"})[1])["ok"]      # idempotent
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=10)
        c.request("GET", "/v1/models")
        assert [m["id"] for m in json.loads(c.getresponse().read())["data"]] == ["tiny", "second"]
        c.close()
        st, data = _post(srv.port, "/v1/completions", dict(body, model="second"))
        got = json.loads(data)
        assert st == 200 and got["model"] == "second" and got["usage"]["completion_tokens"] == 6
        # the fork has no tokenizer (a preset, not a directory): it answers with token ids
        assert got["choices"][0]["finish_reason"] == "length" and len(got["choices"][0]["token_ids"]) == 6
        assert srv.forks["second"].engine is not srv.engine
        assert _post(srv.port, "/sleep", {"model_id": "second", "level": 1})[0] == 200
        assert srv.forks["second"].engine.asleep and not srv.engine.asleep
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=10)
        c.request("GET", "/v2/repository/index")
        assert [m["state"] for m in json.loads(c.getresponse().read())] == ["READY", "SLEEPING"]
        c.close()
        assert _post(srv.port, "/wakeup", {"model_id": "second"})[0] == 200
        st, data = _post(srv.port, "/v1/completions", dict(body, model="second"))
        assert st == 200 and json.loads(data)["choices"][0]["token_ids"] == got["choices"][0]["token_ids"]
        st, data = _post(srv.port, "/v1/completions", body)                                   # the first model is untouched
        assert json.loads(data)["choices"][0]["text"] == base["text"]
    finally:
        srv.shutdown()
        t.join(timeout=5)


def test_link_p2p_pairs_two_servers_as_prefill_and_decode(tmp_path):
    p_srv, pt = _spawn_server(tmp_path)
    d_srv, dt = _spawn_server(tmp_path)
    try:
        bodies = [{"prompt": list(range(3 + i, 40 + 3 * i)), "max_tokens": 9, "temperature": 0, "ignore_eos": True,
                   "stream": bool(i % 2)} for i in range(4)]

        def text(resp):
            st, data = resp
            assert st == 200, data
            if data.startswith("data: "):
                ev = [json.loads(l[6:]) for l in data.split("\n") if l.startswith("data: ") and l != "data: [DONE]"]
                return "".join(e["choices"][0]["text"] for e in ev if e["choices"])
            return json.loads(data)["choices"][0]["text"]

        want = [text(_post(p_srv.port, "/v1/completions", b)) for b in bodies]
        st, data = _post(d_srv.port, "/link_p2p", {"role": "decode", "port": 0})
        assert st == 200
        port = json.loads(data)["port"]
        st, data = _post(p_srv.port, "/link_p2p", {"role": "prefill", "host": "127.0.0.1", "port": port})
        assert st == 200, data
        assert _post(p_srv.port, "/link_p2p", {"role": "prefill", "port": port})[0] == 409
        got = [None] * 4
        ts = [threading.Thread(target=lambda i=i: got.__setitem__(i, text(_post(p_srv.port, "/v1/completions", bodies[i]))))
              for i in range(4)]
        [x.start() for x in ts]
        [x.join(timeout=120) for x in ts]
        assert got == want
        assert p_srv.pd_prefill.handed_over == 4 and d_srv.pd_decode.adopted == 4
        assert _post(p_srv.port, "/unlink_p2p", {})[0] == 200 and p_srv.pd_prefill is None
        for _ in range(200):
            if d_srv.pd_decode is None:
                break
            time.sleep(0.01)
        assert d_srv.pd_decode is None
        assert text(_post(p_srv.port, "/v1/completions", bodies[0])) == want[0]                # a plain instance again
        assert p_srv.engine.scheduler.block_stats(0).num_used == 0 and d_srv.engine.scheduler.block_stats(0).num_used == 0
    finally:
        p_srv.shutdown()
        d_srv.shutdown()
        pt.join(timeout=5)
        dt.join(timeout=5)
