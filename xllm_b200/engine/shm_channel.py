"""Control channel between the ranks of one node through POSIX shared memory.

Parity: the shared-memory channel between the reference's master and its spawned workers
(xllm/core/distributed_runtime/shm_channel.cpp with framework/.../shared_memory_manager: the per-step
inputs are written once and read by every local worker instead of going through an RPC each).

One writer (the leading rank), N readers.  Messages are pickled records `[u32 length][payload]` appended to
a byte ring; the header holds the writer's byte count and one byte count per reader.  A reader sees a message
as soon as the writer has advanced its count (the payload is written first); the writer waits only when the
slowest reader is a whole ring behind.  Waiting spins briefly and then sleeps in 50 us steps, so a step's
control message costs microseconds instead of the two collectives and the device synchronisation of an
object broadcast over the process group.  Every wait has a deadline and raises `TimeoutError`.
"""
from __future__ import annotations

import pickle
import struct
import time
from multiprocessing import shared_memory
from typing import Any, Optional

_MAGIC = 0x584C4C4D43484E31          # "XLLMCHN1"
_HDR = 64                            # magic, capacity, n_readers, head, closed
_SLOT = 64                           # one cache line per reader's tail


class ShmChannel:
    def __init__(self, name: str, create: bool, n_readers: int = 1, capacity: int = 1 << 22, reader: int = -1):
        self.name, self.owner, self.reader = name, create, reader
        if create:
            size = _HDR + _SLOT * n_readers + capacity
            try:
                self.shm = shared_memory.SharedMemory(name=name, create=True, size=size)
            except FileExistsError:                       # a stale segment of a dead job with the same name
                old = shared_memory.SharedMemory(name=name)
                old.close()
                old.unlink()
                self.shm = shared_memory.SharedMemory(name=name, create=True, size=size)
            self.buf = self.shm.buf
            self.buf[: _HDR + _SLOT * n_readers] = bytes(_HDR + _SLOT * n_readers)
            struct.pack_into("<QQQQQ", self.buf, 0, 0, capacity, n_readers, 0, 0)
            struct.pack_into("<Q", self.buf, 0, _MAGIC)   # last: readers wait for the magic
            self.cap, self.n = capacity, n_readers
        else:
            deadline = time.time() + 30.0
            while True:
                try:
                    self.shm = shared_memory.SharedMemory(name=name)
                    if struct.unpack_from("<Q", self.shm.buf, 0)[0] == _MAGIC:
                        break
                    self.shm.close()
                except FileNotFoundError:
                    pass
                if time.time() > deadline:
                    raise TimeoutError(f"shared-memory channel {name} never appeared")
                time.sleep(0.01)
            try:                                          # the creator owns the segment's lifetime: an attaching
                from multiprocessing import resource_tracker   # process must not unlink it when it exits
                resource_tracker.unregister(self.shm._name, "shared_memory")
            except Exception:
                pass
            self.buf = self.shm.buf
            _, self.cap, self.n, _, _ = struct.unpack_from("<QQQQQ", self.buf, 0)
            assert 0 <= reader < self.n
        self.data = _HDR + _SLOT * self.n
        self.tail = self._tail(reader) if reader >= 0 else 0

    # ---- header fields
    def _head(self) -> int:
        return struct.unpack_from("<Q", self.buf, 24)[0]

    def _closed(self) -> bool:
        return struct.unpack_from("<Q", self.buf, 32)[0] != 0

    def _tail(self, r: int) -> int:
        return struct.unpack_from("<Q", self.buf, _HDR + _SLOT * r)[0]

    def _min_tail(self) -> int:
        return min(self._tail(r) for r in range(self.n))

    @staticmethod
    def _wait(cond, timeout_s: float, what: str):
        t0 = time.perf_counter()
        spins = 0
        while not cond():
            spins += 1
            if spins > 200:
                if time.perf_counter() - t0 > timeout_s:
                    raise TimeoutError(what)
                time.sleep(50e-6)

    def _copy_in(self, pos: int, raw: bytes):
        off = pos % self.cap
        first = min(len(raw), self.cap - off)
        self.buf[self.data + off: self.data + off + first] = raw[:first]
        if first < len(raw):
            self.buf[self.data: self.data + len(raw) - first] = raw[first:]

    def _copy_out(self, pos: int, n: int) -> bytes:
        off = pos % self.cap
        first = min(n, self.cap - off)
        out = bytes(self.buf[self.data + off: self.data + off + first])
        if first < n:
            out += bytes(self.buf[self.data: self.data + n - first])
        return out

    # ---- writer
    def send(self, obj: Any, timeout_s: float = 60.0):
        assert self.owner, "only the creating rank writes"
        raw = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
        rec = struct.pack("<I", len(raw)) + raw
        if len(rec) > self.cap:
            raise ValueError(f"message of {len(rec)} bytes exceeds the channel's {self.cap}")
        head = self._head()
        self._wait(lambda: head + len(rec) - self._min_tail() <= self.cap, timeout_s,
                   "a reader of the control channel stopped consuming")
        self._copy_in(head, rec)
        struct.pack_into("<Q", self.buf, 24, head + len(rec))

    # ---- reader
    def recv(self, timeout_s: float = 600.0) -> Any:
        assert self.reader >= 0
        self._wait(lambda: self._head() > self.tail or self._closed(), timeout_s, "the control channel's writer went silent")
        if self._head() <= self.tail:
            raise EOFError("control channel closed")
        (n,) = struct.unpack("<I", self._copy_out(self.tail, 4))
        raw = self._copy_out(self.tail + 4, n)
        self.tail += 4 + n
        struct.pack_into("<Q", self.buf, _HDR + _SLOT * self.reader, self.tail)
        return pickle.loads(raw)

    def poll(self) -> bool:
        return self._head() > self.tail

    def close(self):
        try:
            if self.owner:
                struct.pack_into("<Q", self.buf, 32, 1)
            self.buf = None
            self.shm.close()
            if self.owner:
                self.shm.unlink()
        except (FileNotFoundError, BufferError, AttributeError):
            pass


def open_for_group(ps, capacity: int = 1 << 22) -> Optional[ShmChannel]:
    """The control channel of an instance whose ranks all live on this host: the leading rank creates it
    and tells the others its name through ONE object broadcast; later control traffic skips the process
    group.  None when the ranks span hosts (or `XLLM_SHM_CONTROL=0`)."""
    import os
    import socket

    import torch.distributed as dist
    if os.environ.get("XLLM_SHM_CONTROL", "1") == "0" or ps.world_size <= 1:
        return None
    hosts = [None] * ps.world_size
    dist.all_gather_object(hosts, socket.gethostname(), group=ps.world_group)
    if len(set(hosts)) != 1:
        return None
    leader = getattr(ps, "leader", 0)
    me = ps.rank
    name = [f"xllm_ctl_{os.getpid()}_{int(time.time() * 1000) & 0xFFFFFF}" if me == 0 else None]
    dist.broadcast_object_list(name, src=leader, group=ps.world_group)
    if me == 0:
        ch = ShmChannel(name[0], create=True, n_readers=ps.world_size - 1, capacity=capacity)
    else:
        ch = ShmChannel(name[0], create=False, reader=me - 1)
    dist.barrier(group=ps.world_group)                   # everyone is attached before the first message
    return ch
