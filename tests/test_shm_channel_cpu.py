"""Shared-memory control channel: ordered delivery to several reader processes across ring wrap-around,
back-pressure when a reader lags, end-of-stream, and deadlines."""
import multiprocessing as mp
import os
import time

import pytest

from xllm_b200.engine.shm_channel import ShmChannel


def _reader(name, idx, n_msgs, delay, q):
    ch = ShmChannel(name, create=False, reader=idx)
    got = []
    try:
        for _ in range(n_msgs):
            got.append(ch.recv(timeout_s=20))
            if delay:
                time.sleep(delay)
        try:
            ch.recv(timeout_s=5)
        except EOFError:
            got.append("EOF")
    finally:
        ch.close()
    q.put((idx, got))


def test_messages_reach_every_reader_in_order_across_wraparound():
    name = f"xllm_test_{os.getpid()}"
    ch = ShmChannel(name, create=True, n_readers=2, capacity=4096)      # small ring: wraps many times
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    n = 300
    procs = [ctx.Process(target=_reader, args=(name, i, n, 0.0005 if i == 1 else 0.0, q)) for i in range(2)]
    for p in procs:
        p.start()
    msgs = [("step", [("add", (f"req-{i}", list(range(i % 40))), {"max_tokens": i})]) for i in range(n)]
    t0 = time.perf_counter()
    for m in msgs:
        ch.send(m, timeout_s=20)                                       # blocks while the slow reader is a ring behind
    dt = time.perf_counter() - t0
    time.sleep(0.3)
    ch.close()
    out = dict(q.get(timeout=30) for _ in range(2))
    for p in procs:
        p.join(timeout=10)
    for i in range(2):
        assert out[i][:-1] == msgs and out[i][-1] == "EOF"
    assert dt < 10


def test_deadlines_and_limits():
    name = f"xllm_test_b_{os.getpid()}"
    ch = ShmChannel(name, create=True, n_readers=1, capacity=256)
    rd = ShmChannel(name, create=False, reader=0)
    with pytest.raises(ValueError):
        ch.send(b"x" * 1000)
    with pytest.raises(TimeoutError):
        rd.recv(timeout_s=0.1)
    ch.send("a")
    assert rd.poll() and rd.recv() == "a" and not rd.poll()
    for i in range(3):
        ch.send(b"y" * 60)
    with pytest.raises(TimeoutError):                                  # the ring is full and nobody reads
        ch.send(b"y" * 60, timeout_s=0.1)
    assert rd.recv() == b"y" * 60
    ch.send(b"z" * 60, timeout_s=1)
    rd.close()
    ch.close()
