"""Liveness of the ranks of an instance and discovery of instances.

Parity:
  * `HealthCheckManager` (xllm/core/common/health_check_manager.h): the master polls every worker
    (`RemoteWorker::check_health`) every few seconds and turns `/health` unhealthy when one stops
    answering,
  * `XServiceClient` / `EtcdClient` (runtime/xservice_client.cpp, common/etcd_client.cpp): every
    instance registers itself (name, role PREFILL / DECODE / MIX, address) under a key with a lease
    that its heartbeat keeps alive; peers for PD disaggregation are found by listing the keys.

Both are built on one small key-value interface (`set`, `get`, `keys`), served here by
`torch.distributed` stores (TCPStore for multi-process, HashStore in one process); an etcd-backed
store can be dropped in behind the same three calls.  Failure detection never needs a GPU: a rank
publishes a heartbeat *between* steps, and the others read the store before their next launch, so
a vanished rank is noticed on the host and no collective is entered with a dead peer.
"""
from __future__ import annotations

import json
import time
from dataclasses import asdict, dataclass
from typing import Callable, Dict, List, Optional


class KV:
    """Adapter over a torch.distributed store (or any object with set/get); keeps a key index so
    that prefixes can be listed."""

    def __init__(self, store):
        self.store = store

    def set(self, key: str, value: str):
        self.store.set(key, value)
        idx = self._index()
        if key not in idx:
            idx.append(key)
            self.store.set("__keys__", json.dumps(idx))

    def get(self, key: str) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def _index(self) -> List[str]:
        raw = None
        try:
            if not hasattr(self.store, "check") or self.store.check(["__keys__"]):
                raw = self.store.get("__keys__").decode()
        except Exception:
            raw = None
        return json.loads(raw) if raw else []

    def keys(self, prefix: str) -> List[str]:
        return [k for k in self._index() if k.startswith(prefix)]


class HeartbeatMonitor:
    def __init__(self, kv: KV, rank: int, world: int, timeout_s: float = 3.0, clock: Callable[[], float] = time.time,
                 prefix: str = "hb"):
        self.kv, self.rank, self.world, self.timeout, self.clock, self.prefix = kv, rank, world, timeout_s, clock, prefix
        self.on_failure: List[Callable[[List[int]], None]] = []

    def beat(self, step: int = 0):
        self.kv.set(f"{self.prefix}/{self.rank}", json.dumps({"t": self.clock(), "step": step}))

    def leave(self):
        """Orderly exit: tell the others at once instead of letting the timeout expire."""
        self.kv.set(f"{self.prefix}/{self.rank}", json.dumps({"t": -1.0, "step": -1}))

    def last_seen(self, rank: int) -> Optional[float]:
        raw = self.kv.get(f"{self.prefix}/{rank}")
        return json.loads(raw)["t"] if raw else None

    def dead_ranks(self) -> List[int]:
        now = self.clock()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            t = self.last_seen(r)
            if t is None:
                continue                      # has not started yet
            if t < 0 or now - t > self.timeout:
                dead.append(r)
        return dead

    def check(self) -> bool:
        """True when every peer that ever reported is alive; calls the failure hooks otherwise."""
        dead = self.dead_ranks()
        if dead:
            for cb in self.on_failure:
                cb(dead)
        return not dead


@dataclass
class InstanceInfo:
    name: str
    role: str                  # "PREFILL" | "DECODE" | "MIX"
    address: str
    tp_size: int = 1
    dp_size: int = 1
    kv_block_size: int = 16
    lease_until: float = 0.0


class InstanceRegistry:
    """Lease-based service registry (the etcd usage of the reference, behind `KV`)."""

    def __init__(self, kv: KV, lease_s: float = 10.0, clock: Callable[[], float] = time.time, prefix: str = "xllm/instances"):
        self.kv, self.lease, self.clock, self.prefix = kv, lease_s, clock, prefix

    def register(self, info: InstanceInfo):
        info.lease_until = self.clock() + self.lease
        self.kv.set(f"{self.prefix}/{info.name}", json.dumps(asdict(info)))

    heartbeat = register           # renewing the lease is re-registering

    def deregister(self, name: str):
        self.kv.set(f"{self.prefix}/{name}", "")

    def list(self, role: Optional[str] = None) -> List[InstanceInfo]:
        out = []
        for k in self.kv.keys(self.prefix + "/"):
            raw = self.kv.get(k)
            if not raw:
                continue
            info = InstanceInfo(**json.loads(raw))
            if info.lease_until < self.clock():
                continue                      # lease expired: the instance stopped heartbeating
            if role is None or info.role == role:
                out.append(info)
        return out

    def pick(self, role: str, key: str = "") -> Optional[InstanceInfo]:
        """Stable choice of an instance of `role` (hash of `key` over the live ones)."""
        live = sorted(self.list(role), key=lambda i: i.name)
        if not live:
            return None
        return live[hash(key) % len(live)]


class HealthState:
    """What `/health` reports: healthy until a monitor says otherwise."""

    def __init__(self):
        self.healthy = True
        self.reason = ""

    def fail(self, dead: List[int]):
        self.healthy = False
        self.reason = "ranks not responding: " + ",".join(map(str, dead))
