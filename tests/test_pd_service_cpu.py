"""PD disaggregation between two PROCESSES on CPU: the decode instance is a child process behind a
socket, KV travels as messages on the same connection; the token streams must equal those of one
engine, blocks must all come back, and a peer that goes away is noticed on the host."""
import os
import subprocess
import sys

import pytest
import torch

from xllm_b200 import LLM, SamplingParams
from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
from xllm_b200.engine.pd_service import Channel, DecodeService, PrefillService, SocketCopy

HERE = os.path.dirname(os.path.abspath(__file__))
KW = dict(model="tiny", device="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
          max_tokens_per_batch=128, enable_graph=False, enable_prefix_cache=False)


def _spawn_decode(port, num_blocks=64, mode="serve"):
    return subprocess.Popen([sys.executable, os.path.join(HERE, "mp_pd_cpu_decode.py"), str(port), str(num_blocks), mode],
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)


def _prefill_side(srv):
    ch = Channel.accept(srv, timeout=120.0)
    p = LLMEngine(EngineConfig(**KW), hold_finished_blocks=True)
    return p, PrefillService(p, ch, SocketCopy(p.runner))


def test_two_process_pd_matches_single_engine():
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (5, 16, 33, 70, 150)]
    llm = LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
              max_tokens_per_batch=128, enable_graph=False)
    want = [o.outputs[0].token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=10, temperature=0.0,
                                                                                   ignore_eos=True))]
    srv = Channel.listen()
    child = _spawn_decode(srv.getsockname()[1])
    try:
        p, svc = _prefill_side(srv)
        for i, pr in enumerate(prompts):
            assert svc.add_request(f"r{i}", pr, max_tokens=10, temperature=0.0, ignore_eos=True)
        got = {f"r{i}": [] for i in range(len(prompts))}
        fin = set()

        def on(ev):
            if ev.token >= 0:
                got[ev.request_id].append(ev.token)
            if ev.request_finished:
                fin.add(ev.request_id)

        assert svc.run_until_done(on, max_seconds=120.0)
        svc.close()
        out, _ = child.communicate(timeout=60)
    finally:
        if child.poll() is None:
            child.kill()
    assert [got[f"r{i}"] for i in range(len(prompts))] == want, out
    assert fin == set(got) and not svc.failed
    assert svc.handed_over == len(prompts)
    assert svc.t.pushed_bytes > 0
    assert p.scheduler.block_stats(0).num_used == 0
    assert "PD_DECODE_DONE ok=True adopted=5 used=0 reserved=0" in out, out


def test_two_process_pd_backpressure_and_one_token_requests():
    """Eight decode blocks cannot hold four 40-token prompts at once: reservations are refused and
    retried; a request that wants one token never leaves the prefill side."""
    g = torch.Generator().manual_seed(5)
    srv = Channel.listen()
    child = _spawn_decode(srv.getsockname()[1], num_blocks=8)
    try:
        p, svc = _prefill_side(srv)
        for i in range(4):
            svc.add_request(f"q{i}", torch.randint(0, 32000, (40,), generator=g).tolist(), max_tokens=6, temperature=0.0,
                            ignore_eos=True)
        svc.add_request("one", [1, 2, 3, 4], max_tokens=1, temperature=0.0, ignore_eos=True)
        n = {}

        def on(ev):
            if ev.token >= 0:
                n[ev.request_id] = n.get(ev.request_id, 0) + 1

        assert svc.run_until_done(on, max_seconds=120.0)
        svc.close()
        out, _ = child.communicate(timeout=60)
    finally:
        if child.poll() is None:
            child.kill()
    assert n == {"q0": 6, "q1": 6, "q2": 6, "q3": 6, "one": 1}, (n, out)
    assert "adopted=4 used=0 reserved=0" in out, out


def test_prefill_side_notices_a_decode_instance_that_went_away():
    srv = Channel.listen()
    child = _spawn_decode(srv.getsockname()[1], mode="vanish")
    try:
        p, svc = _prefill_side(srv)
        svc.add_request("a", list(range(1, 40)), max_tokens=50, temperature=0.0, ignore_eos=True)
        svc.add_request("b", list(range(3, 90)), max_tokens=50, temperature=0.0, ignore_eos=True)
        seen = []
        assert svc.run_until_done(seen.append, max_seconds=120.0)
        child.wait(timeout=60)
    finally:
        if child.poll() is None:
            child.kill()
    assert svc.failed and all("went away" in r or "refused" in r for r in svc.failed.values()), svc.failed
    assert any(ev.finished and ev.finish_reason.startswith("error") for ev in seen)
    assert p.scheduler.block_stats(0).num_used == 0       # held blocks were released


def test_decode_side_reclaims_when_the_prefill_instance_goes_away():
    """In-process pair over a real socket: reservations and adopted sequences are given back when
    the connection closes between steps."""
    srv = Channel.listen()
    import threading
    box = {}
    th = threading.Thread(target=lambda: box.setdefault("c", Channel.accept(srv, 30.0)))
    th.start()
    ch_d = Channel.connect("127.0.0.1", srv.getsockname()[1])
    th.join()
    ch_p = box["c"]
    d = LLMEngine(EngineConfig(**KW))
    dsvc = DecodeService(d, ch_d, SocketCopy(d.runner))
    ch_p.send({"op": "reserve", "rid": "x", "n_tokens": 40})
    ch_p.send({"op": "reserve", "rid": "y", "n_tokens": 20})
    for _ in range(50):
        dsvc.step(0.01)
        if d.scheduler.num_reserved() == 2:
            break
    assert d.scheduler.num_reserved() == 2 and d.scheduler.block_stats(0).num_used > 0
    replies = ch_p.poll(0.5)
    assert [m["op"] for m in replies] == ["reserved", "reserved"] and all(m["blocks"] for m in replies)
    # hand one over with nothing pushed (socket plane: wait() has nothing to wait for), then vanish
    ch_p.send({"op": "first", "rid": "x", "tokens": list(range(1, 41)) + [7], "num_prompt": 40,
               "sampling": {"max_tokens": 30, "ignore_eos": True}, "epoch": 0})
    for _ in range(50):
        dsvc.step(0.01)
        if dsvc.adopted:
            break
    assert dsvc.adopted == 1
    ch_p.close()
    for _ in range(100):
        dsvc.step(0.01)
        if dsvc.stopped and not d.has_unfinished():
            break
    d.drain()
    assert dsvc.stopped and d.scheduler.num_reserved() == 0
    assert d.scheduler.block_stats(0).num_used == 0 and dsvc.reclaimed_blocks > 0


def test_offline_requests_decode_on_the_prefill_instance():
    """Online / offline co-location: offline requests are not handed over; they decode on the prefill instance
    between the online prompts, give the single-engine tokens, and go on when the decode instance is gone."""
    g = torch.Generator().manual_seed(12)
    online = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (20, 45)]
    offline = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (30, 12, 60)]
    llm = LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
              max_tokens_per_batch=128, enable_graph=False)
    sp = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
    want_on = [o.outputs[0].token_ids for o in llm.generate(online, sp)]
    want_off = [o.outputs[0].token_ids for o in llm.generate(offline, sp)]
    srv = Channel.listen()
    child = _spawn_decode(srv.getsockname()[1])
    try:
        p, svc = _prefill_side(srv)
        for i, pr in enumerate(offline):
            assert svc.add_request(f"off{i}", pr, max_tokens=8, temperature=0.0, ignore_eos=True, offline=True)
        for i, pr in enumerate(online):
            assert svc.add_request(f"on{i}", pr, max_tokens=8, temperature=0.0, ignore_eos=True)
        got, fin = {}, set()

        def on(ev):
            if ev.token >= 0:
                got.setdefault(ev.request_id, []).append(ev.token)
            if ev.request_finished:
                fin.add(ev.request_id)

        assert svc.run_until_done(on, max_seconds=120.0)
        assert [got[f"on{i}"] for i in range(2)] == want_on and [got[f"off{i}"] for i in range(3)] == want_off
        assert svc.handed_over == 2 and svc.kept_local == 3 and not svc.local and not svc.failed
        assert p.scheduler.block_stats(0).num_used == 0
        # the decode instance leaves: an offline request still runs to the end here
        svc.close()
        out, _ = child.communicate(timeout=60)
        assert "adopted=2" in out, out
        assert svc.add_request("late", offline[0], max_tokens=8, temperature=0.0, ignore_eos=True, offline=True)
        got.pop("off0", None)
        assert svc.run_until_done(on, max_seconds=60.0)
        assert got["late"] == want_off[0]
    finally:
        if child.poll() is None:
            child.kill()


def test_idle_decode_instance_pulls_offline_requests_over():
    """The decode instance signals spare capacity; the prefill instance moves offline requests that are
    decoding locally over to it (prompt + tokens so far go through the ordinary handover).  The client sees one
    uninterrupted stream per request, equal to a single engine's, and every block comes back on both sides."""
    g = torch.Generator().manual_seed(21)
    offline = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (30, 12, 44)]
    llm = LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
              max_tokens_per_batch=128, enable_graph=False)
    sp = SamplingParams(max_tokens=24, temperature=0.0, ignore_eos=True)
    want = [o.outputs[0].token_ids for o in llm.generate(offline, sp)]
    srv = Channel.listen()
    child = _spawn_decode(srv.getsockname()[1], mode="pull")
    try:
        p, svc = _prefill_side(srv)
        for i, pr in enumerate(offline):
            assert svc.add_request(f"off{i}", pr, max_tokens=24, temperature=0.0, ignore_eos=True, offline=True)
        got, fin = {}, []

        def on(ev):
            if ev.token >= 0:
                got.setdefault(ev.request_id, []).append(ev.token)
            if ev.request_finished:
                fin.append(ev.request_id)

        assert svc.run_until_done(on, max_seconds=120.0)
        assert [got[f"off{i}"] for i in range(3)] == want
        assert sorted(fin) == ["off0", "off1", "off2"]                  # one finish each: the local abort is not shown
        assert svc.migrated >= 1 and svc.handed_over == svc.migrated and not svc.failed and not svc.migrating
        assert not svc.local and not svc.local_state and not svc.remote
        assert p.scheduler.block_stats(0).num_used == 0
        svc.close()
        out, _ = child.communicate(timeout=60)
        assert f"adopted={svc.migrated}" in out and "used=0 reserved=0" in out, out
    finally:
        if child.poll() is None:
            child.kill()


def test_pull_frame_round_trips_in_both_codecs():
    from xllm_b200 import proto
    m = {"op": "pull", "free_blocks": 37, "max_requests": 1}
    assert proto.decode(proto.encode(m)) == m
