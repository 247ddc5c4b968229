"""etcd and routing-service clients against in-process fakes that speak the same HTTP + JSON: keys with
leases that expire when the keepalive stops, the heartbeat monitor and instance registry running on etcd,
registration / heartbeat / re-registration towards the routing service."""
import base64
import json
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

import pytest

from xllm_b200.engine.health import InstanceInfo, InstanceRegistry
from xllm_b200.engine.service_client import EtcdKV, InstanceMeta, RpcError, ServiceClient


class _Fake:
    """An etcd v3 JSON gateway and an XllmRpcService in one process."""

    def __init__(self):
        self.kv, self.leases, self.next_lease = {}, {}, 100
        self.instances, self.beats, self.known = {}, [], set()
        self.lock = threading.Lock()
        fake = self

        class H(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):
                pass

            def do_POST(self):
                body = json.loads(self.rfile.read(int(self.headers.get("Content-Length", 0))) or b"{}")
                with fake.lock:
                    out = fake.handle(self.path, body)
                raw = json.dumps(out).encode()
                self.send_response(200 if out is not None else 404)
                self.send_header("Content-Length", str(len(raw)))
                self.end_headers()
                self.wfile.write(raw)

        self.srv = ThreadingHTTPServer(("127.0.0.1", 0), H)
        self.port = self.srv.server_address[1]
        threading.Thread(target=self.srv.serve_forever, daemon=True).start()

    def expire(self):
        now = time.time()
        for lid in [l for l, (ttl, until) in self.leases.items() if until < now]:
            del self.leases[lid]
            self.kv = {k: v for k, v in self.kv.items() if v[1] != lid}

    def handle(self, path, b):
        self.expire()
        d = lambda s: base64.b64decode(s).decode()
        e = lambda s: base64.b64encode(s.encode()).decode()
        if path == "/v3/lease/grant":
            self.next_lease += 1
            self.leases[str(self.next_lease)] = (b["TTL"], time.time() + b["TTL"])
            return {"ID": str(self.next_lease), "TTL": str(b["TTL"])}
        if path == "/v3/lease/keepalive":
            if b["ID"] not in self.leases:
                return {"result": {"ID": b["ID"]}}
            ttl = self.leases[b["ID"]][0]
            self.leases[b["ID"]] = (ttl, time.time() + ttl)
            return {"result": {"ID": b["ID"], "TTL": str(ttl)}}
        if path == "/v3/lease/revoke":
            self.leases.pop(b["ID"], None)
            self.kv = {k: v for k, v in self.kv.items() if v[1] != b["ID"]}
            return {}
        if path == "/v3/kv/put":
            self.kv[d(b["key"])] = (d(b.get("value", "")), b.get("lease"))
            return {}
        if path in ("/v3/kv/range", "/v3/kv/deleterange"):
            lo = d(b["key"])
            hi = d(b["range_end"]) if "range_end" in b else None
            hit = sorted(k for k in self.kv if (k == lo if hi is None else lo <= k < hi))
            if path == "/v3/kv/deleterange":
                for k in hit:
                    del self.kv[k]
                return {"deleted": str(len(hit))}
            return {"kvs": [{"key": e(k), "value": e(self.kv[k][0])} for k in hit], "count": str(len(hit))}
        if path == "/XllmRpcService/RegisterInstance":
            self.instances[b["name"]] = b
            self.known.add(b["name"])
            return {"status_code": 0}
        if path == "/XllmRpcService/GetInstanceInfo":
            return self.instances.get(b["name"], {})
        if path == "/XllmRpcService/Heartbeat":
            self.beats.append(b)
            return {"ok": b["name"] in self.known}
        if path == "/XllmRpcService/GetStaticDecodeList":
            return {"names": sorted(n for n, m in self.instances.items() if m["type"] == 2)}
        if path == "/XllmRpcService/GetStaticPrefillList":
            return {"names": sorted(n for n, m in self.instances.items() if m["type"] == 1)}
        return None


@pytest.fixture()
def fake():
    f = _Fake()
    yield f
    f.srv.shutdown()


def test_etcd_kv_prefixes_and_leases(fake):
    kv = EtcdKV(f"127.0.0.1:{fake.port}")
    kv.set("xllm/a", "1")
    kv.set("xllm/b", "2")
    kv.set("other", "3")
    assert kv.get("xllm/a") == "1" and kv.get("missing") is None
    assert kv.keys("xllm/") == ["xllm/a", "xllm/b"] and kv.get_prefix("xllm/") == {"xllm/a": "1", "xllm/b": "2"}
    assert kv.delete("xllm/", prefix=True) == 2 and kv.keys("xllm/") == [] and kv.get("other") == "3"
    # a leased key lives while the keepalive runs and vanishes after it stops
    leased = EtcdKV(f"127.0.0.1:{fake.port}", lease_s=1.0)
    leased.start_keepalive(period_s=0.2)
    leased.set("inst/p0", "alive")
    time.sleep(1.5)
    assert kv.get("inst/p0") == "alive"
    leased._stop.set()
    leased._thread.join(timeout=2)
    time.sleep(1.4)
    assert kv.get("inst/p0") is None
    assert leased.keepalive() is False           # etcd forgot the lease: the owner must grant and register again
    with pytest.raises(RpcError):
        EtcdKV("127.0.0.1:1", timeout_s=0.2).get("x")


def test_instance_registry_runs_on_etcd(fake):
    kv = EtcdKV(f"127.0.0.1:{fake.port}")
    reg = InstanceRegistry(kv, lease_s=5.0)
    reg.register(InstanceInfo("p0", "PREFILL", "10.0.0.1:9000"))
    reg.register(InstanceInfo("d0", "DECODE", "10.0.0.2:9000", tp_size=4))
    assert [i.name for i in reg.list("DECODE")] == ["d0"] and reg.pick("PREFILL").address == "10.0.0.1:9000"
    reg.deregister("p0")
    assert reg.list("PREFILL") == []


def test_service_client_registers_heartbeats_and_recovers(fake):
    state = {"waiting": 3}
    probe = lambda: {"waiting_requests_num": state["waiting"], "gpu_cache_usage_perc": 0.25, "recent_max_ttft": 120,
                     "recent_max_tbt": 18}
    url = f"http://127.0.0.1:{fake.port}"
    p = ServiceClient(url, InstanceMeta("10.0.0.1:9000", rpc_address="10.0.0.1:9001", type="PREFILL", dp_size=2), probe)
    d = ServiceClient(url, InstanceMeta("10.0.0.2:9000", type="DECODE"))
    assert p.register() and d.register() and p.meta.incarnation_id and p.meta.register_ts_ms > 0
    assert p.static_decode_list() == ["10.0.0.2:9000"] and d.static_prefill_list() == ["10.0.0.1:9000"]
    info = d.instance_info("10.0.0.1:9000")
    assert info.type == "PREFILL" and info.dp_size == 2 and info.rpc_address == "10.0.0.1:9001"
    assert d.instance_info("nobody") is None
    p.note_cache(stored=[b"\x01" * 16, b"\x02" * 16], removed=[b"\x03" * 16])
    assert p.heartbeat()
    beat = fake.beats[-1]
    assert beat["load_metrics"] == {"waiting_requests_num": 3, "gpu_cache_usage_perc": 0.25}
    assert beat["latency_metrics"] == {"recent_max_ttft": 120, "recent_max_tbt": 18}
    assert [base64.b64decode(h) for h in beat["cache_event"]["stored_cache"]] == [b"\x01" * 16, b"\x02" * 16]
    assert p.heartbeat() and fake.beats[-1]["cache_event"] == {"stored_cache": [], "removed_cache": []}
    # the service restarts and forgets the instance: the next beat makes the client register again
    with fake.lock:
        fake.known.clear()
        fake.instances.clear()
    assert p.heartbeat() and p.registered and "10.0.0.1:9000" in fake.instances
    # the service is unreachable: the beat fails, the cache events wait for the next one
    dead = ServiceClient("http://127.0.0.1:1", InstanceMeta("x"), timeout_s=0.2)
    dead.note_cache(stored=[b"\x09" * 16])
    assert not dead.heartbeat() and dead.failures == 1 and dead._stored == [b"\x09" * 16]
    # background loop
    state["waiting"] = 7
    n = len(fake.beats)
    p.start(period_s=0.1)
    time.sleep(0.5)
    p.stop()
    assert len(fake.beats) >= n + 2 and fake.beats[-1]["load_metrics"]["waiting_requests_num"] == 7
