"""Clients of the cluster services an instance talks to: etcd (discovery, leases) and the routing service
(instance registration, heartbeats with load / latency / cache events, static PD peer lists).

Parity: `EtcdClient` (xllm/core/common/etcd_client.cpp: set / get / get_prefix / rm / add_watch with a
lease kept alive by a background thread) and `XServiceClient` (core/runtime/xservice_client.cpp with
proto/xservice.proto: RegisterInstance, GetInstanceInfo, Heartbeat, GetStaticDecodeList,
GetStaticPrefillList).

Both speak HTTP + JSON from the standard library:
  * etcd through its v3 gRPC gateway (`/v3/kv/put`, `/v3/kv/range`, `/v3/kv/deleterange`,
    `/v3/lease/grant`, `/v3/lease/keepalive`, `/v3/lease/revoke`; keys and values base64-encoded),
  * the routing service through the HTTP + JSON access that its RPC server gives every protobuf
    method (`POST /XllmRpcService/<Method>` with the message as JSON; field names of the .proto).
`EtcdKV` implements the `set / get / keys` interface of `engine/health.py`, so the heartbeat monitor and
the instance registry run on etcd unchanged.  Nothing here touches a GPU.
"""
from __future__ import annotations

import base64
import http.client
import json
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple
from urllib.parse import urlparse


class RpcError(RuntimeError):
    pass


class _Http:
    """One keep-alive connection per calling thread; one retry on a dropped connection."""

    def __init__(self, endpoint: str, timeout_s: float = 3.0):
        u = urlparse(endpoint if "//" in endpoint else "http://" + endpoint)
        self.host, self.port, self.timeout = u.hostname or "127.0.0.1", u.port or 80, timeout_s
        self.local = threading.local()

    def post(self, path: str, body: dict) -> dict:
        data = json.dumps(body).encode()
        last = None
        for attempt in range(2):
            conn = getattr(self.local, "conn", None)
            if conn is None:
                conn = self.local.conn = http.client.HTTPConnection(self.host, self.port, timeout=self.timeout)
            try:
                conn.request("POST", path, data, {"Content-Type": "application/json"})
                r = conn.getresponse()
                raw = r.read()
                if r.status != 200:
                    raise RpcError(f"{path}: HTTP {r.status} {raw[:200]!r}")
                return json.loads(raw) if raw else {}
            except (OSError, http.client.HTTPException) as e:
                last = e
                conn.close()
                self.local.conn = None
        raise RpcError(f"{path}: {last}")


def _b64(s) -> str:
    return base64.b64encode(s.encode() if isinstance(s, str) else s).decode()


def _unb64(s: str) -> str:
    return base64.b64decode(s).decode()


def _prefix_end(prefix: str) -> bytes:
    """The key just after every key with this prefix (etcd's range_end for a prefix query)."""
    b = bytearray(prefix.encode())
    for i in range(len(b) - 1, -1, -1):
        if b[i] < 0xFF:
            b[i] += 1
            return bytes(b[: i + 1])
    return b"\0"


class EtcdKV:
    """etcd v3 over the JSON gateway.  With `lease_s` every key written by this object is attached to one
    lease; `keepalive()` (or the thread started by `start_keepalive`) renews it, and when the process dies
    the keys vanish after `lease_s` — which is how the other instances learn of it."""

    def __init__(self, endpoint: str, lease_s: float = 0.0, timeout_s: float = 3.0):
        self.http = _Http(endpoint, timeout_s)
        self.lease_s = lease_s
        self.lease_id: Optional[str] = None
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        if lease_s > 0:
            self.grant()

    # ---- leases
    def grant(self) -> str:
        out = self.http.post("/v3/lease/grant", {"TTL": int(max(1, round(self.lease_s)))})
        self.lease_id = str(out["ID"])
        return self.lease_id

    def keepalive(self) -> bool:
        """False when etcd no longer knows the lease (it expired: grant a new one and re-register)."""
        if self.lease_id is None:
            return False
        out = self.http.post("/v3/lease/keepalive", {"ID": self.lease_id})
        ttl = int((out.get("result") or out).get("TTL", 0) or 0)
        return ttl > 0

    def revoke(self):
        if self.lease_id is not None:
            try:
                self.http.post("/v3/lease/revoke", {"ID": self.lease_id})
            finally:
                self.lease_id = None

    def start_keepalive(self, on_lost: Optional[Callable[[], None]] = None, period_s: Optional[float] = None):
        period = period_s or max(0.2, self.lease_s / 3.0)

        def loop():
            while not self._stop.wait(period):
                try:
                    if not self.keepalive():
                        self.grant()
                        if on_lost is not None:
                            on_lost()
                except RpcError:
                    pass                       # etcd unreachable: keep trying, the lease may still be alive
        self._thread = threading.Thread(target=loop, name="xllm-etcd-keepalive", daemon=True)
        self._thread.start()

    def close(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        try:
            self.revoke()
        except RpcError:
            pass

    # ---- the KV interface of engine/health.py
    def set(self, key: str, value: str):
        body = {"key": _b64(key), "value": _b64(value)}
        if self.lease_id is not None:
            body["lease"] = self.lease_id
        self.http.post("/v3/kv/put", body)

    def get(self, key: str) -> Optional[str]:
        kvs = self.http.post("/v3/kv/range", {"key": _b64(key)}).get("kvs") or []
        return _unb64(kvs[0].get("value", "")) if kvs else None

    def get_prefix(self, prefix: str) -> Dict[str, str]:
        out = self.http.post("/v3/kv/range", {"key": _b64(prefix), "range_end": _b64(_prefix_end(prefix))})
        return {_unb64(kv["key"]): _unb64(kv.get("value", "")) for kv in out.get("kvs") or []}

    def keys(self, prefix: str) -> List[str]:
        return sorted(self.get_prefix(prefix))

    def delete(self, key: str, prefix: bool = False) -> int:
        body = {"key": _b64(key)}
        if prefix:
            body["range_end"] = _b64(_prefix_end(key))
        return int(self.http.post("/v3/kv/deleterange", body).get("deleted", 0) or 0)


# --------------------------------------------------------------------------------- routing service
INSTANCE_TYPES = {"DEFAULT": 0, "PREFILL": 1, "DECODE": 2, "MIX": 3}


@dataclass
class InstanceMeta:
    """`InstanceMetaInfo` of proto/xservice.proto."""
    name: str                                  # the instance's HTTP address
    rpc_address: str = ""
    type: str = "DEFAULT"
    cluster_ids: List[int] = field(default_factory=list)
    dp_size: int = 1
    addrs: List[str] = field(default_factory=list)
    ports: List[int] = field(default_factory=list)
    incarnation_id: str = ""
    register_ts_ms: int = 0
    kv_split_size: int = 1

    def to_json(self) -> dict:
        return {"name": self.name, "rpc_address": self.rpc_address, "type": INSTANCE_TYPES.get(self.type, 0),
                "cluster_ids": self.cluster_ids, "dp_size": self.dp_size, "addrs": self.addrs, "ports": self.ports,
                "incarnation_id": self.incarnation_id, "register_ts_ms": self.register_ts_ms,
                "kv_split_size": self.kv_split_size}

    @staticmethod
    def from_json(d: dict) -> "InstanceMeta":
        names = {v: k for k, v in INSTANCE_TYPES.items()}
        t = d.get("type", 0)
        return InstanceMeta(name=d.get("name", ""), rpc_address=d.get("rpc_address", ""),
                            type=names.get(t, t if isinstance(t, str) else "DEFAULT"),
                            cluster_ids=[int(x) for x in d.get("cluster_ids", [])], dp_size=int(d.get("dp_size", 1)),
                            addrs=list(d.get("addrs", [])), ports=[int(p) for p in d.get("ports", [])],
                            incarnation_id=d.get("incarnation_id", ""), register_ts_ms=int(d.get("register_ts_ms", 0)),
                            kv_split_size=int(d.get("kv_split_size", 1)))


class ServiceClient:
    """What an instance does towards the routing service: register once (a fresh incarnation id per process
    start), then heartbeat with its load, its recent worst latencies and the prefix-cache blocks it gained
    and lost since the last beat, so that the service can route by cache affinity and load."""

    SERVICE = "/XllmRpcService"

    def __init__(self, endpoint: str, meta: InstanceMeta, probe: Optional[Callable[[], dict]] = None,
                 timeout_s: float = 3.0, clock: Callable[[], float] = time.time):
        self.http = _Http(endpoint, timeout_s)
        self.meta = meta
        self.probe = probe or (lambda: {})
        self.clock = clock
        self.registered = False
        self._stored: List[bytes] = []
        self._removed: List[bytes] = []
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.beats = 0
        self.failures = 0

    def register(self) -> bool:
        self.meta.incarnation_id = self.meta.incarnation_id or uuid.uuid4().hex
        self.meta.register_ts_ms = int(self.clock() * 1000)
        out = self.http.post(f"{self.SERVICE}/RegisterInstance", self.meta.to_json())
        self.registered = int(out.get("status_code", 0) or 0) == 0
        return self.registered

    def instance_info(self, name: str) -> Optional[InstanceMeta]:
        out = self.http.post(f"{self.SERVICE}/GetInstanceInfo", {"name": name})
        return InstanceMeta.from_json(out) if out.get("name") else None

    def static_decode_list(self) -> List[str]:
        return list(self.http.post(f"{self.SERVICE}/GetStaticDecodeList", {"name": self.meta.name}).get("names", []))

    def static_prefill_list(self) -> List[str]:
        return list(self.http.post(f"{self.SERVICE}/GetStaticPrefillList", {"name": self.meta.name}).get("names", []))

    # ---- cache events: block hashes the prefix cache stored / evicted since the last heartbeat
    def note_cache(self, stored=(), removed=()):
        with self._lock:
            self._stored.extend(bytes(h) for h in stored)
            self._removed.extend(bytes(h) for h in removed)

    def heartbeat(self) -> bool:
        with self._lock:
            stored, removed = self._stored, self._removed
            self._stored, self._removed = [], []
        p = self.probe() or {}
        req = {"name": self.meta.name, "incarnation_id": self.meta.incarnation_id,
               "cache_event": {"stored_cache": [_b64(h) for h in stored], "removed_cache": [_b64(h) for h in removed]},
               "load_metrics": {"waiting_requests_num": int(p.get("waiting_requests_num", 0)),
                                "gpu_cache_usage_perc": float(p.get("gpu_cache_usage_perc", 0.0))},
               "latency_metrics": {"recent_max_ttft": int(p.get("recent_max_ttft", 0)),
                                   "recent_max_tbt": int(p.get("recent_max_tbt", 0))}}
        if "worker_free_phy_pages" in p:
            req["xtensor_info"] = {"worker_free_phy_pages": [int(x) for x in p["worker_free_phy_pages"]]}
        try:
            out = self.http.post(f"{self.SERVICE}/Heartbeat", req)
        except RpcError:
            with self._lock:                   # the events are not lost: they ride on the next beat
                self._stored = stored + self._stored
                self._removed = removed + self._removed
            self.failures += 1
            return False
        self.beats += 1
        if out.get("ok") is False:             # the service forgot us (it restarted): register again
            self.registered = False
            try:
                self.register()
            except RpcError:
                self.failures += 1
        return True

    def start(self, period_s: float = 1.0):
        def loop():
            while not self._stop.wait(period_s):
                if not self.registered:
                    try:
                        self.register()
                    except RpcError:
                        self.failures += 1
                        continue
                self.heartbeat()
        self._thread = threading.Thread(target=loop, name="xllm-service-heartbeat", daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)


def engine_probe(engine) -> Callable[[], dict]:
    """Load and latency figures of an `LLMEngine` for the heartbeat."""
    def probe():
        sched = engine.scheduler
        bm = sched.block_manager(0)
        total = max(1, getattr(bm, "num_total_blocks", 0) or getattr(bm, "num_blocks", 1))
        used = getattr(bm, "num_used_blocks", 0)
        stats = getattr(engine, "latency_window", None) or {}
        return {"waiting_requests_num": getattr(sched, "num_waiting", 0),
                "gpu_cache_usage_perc": float(used) / float(total),
                "recent_max_ttft": int(stats.get("max_ttft_ms", 0)), "recent_max_tbt": int(stats.get("max_tbt_ms", 0))}
    return probe
