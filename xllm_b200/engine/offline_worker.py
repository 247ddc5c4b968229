"""Worker ranks of an offline multi-GPU `LLM`.

Parity: the offline API of the reference spawns its worker processes itself (xllm/pybind/llm.py with
core/distributed_runtime/spawn_worker_server: one worker server process per device, the master in the
caller's process).  Here `LLM(devices="cuda:0,cuda:1,...")` makes the calling process rank 0 and starts
`python -m xllm_b200.engine.offline_worker` once per further device.  A worker builds the same engine from
the same configuration, joins the job's process group and then follows rank 0's control stream
(`engine/replica.py`) until it says stop or rank 0's process is gone.
"""
from __future__ import annotations

import json
import os
import socket
import subprocess
import sys
import threading
from dataclasses import asdict
from typing import List, Optional


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def parse_devices(devices: Optional[str]) -> List[str]:
    """'cuda:0,cuda:1' -> ['cuda:0', 'cuda:1']; 'cuda' / 'cpu' / None -> one entry."""
    if not devices:
        return ["auto"]
    out = [d.strip() for d in devices.split(",") if d.strip()]
    return ["cuda:0" if d == "cuda" else d for d in out] or ["auto"]


def device_indices(devs: List[str]) -> List[int]:
    return [int(d.split(":")[1]) if ":" in d else i for i, d in enumerate(devs)]


class WorkerGroup:
    """The spawned ranks 1..N-1; owns the children."""

    def __init__(self, cfg, devs: List[str], dp_size: int, ep_size: int, python: str = sys.executable):
        self.world = len(devs)
        self.port = free_port()
        self.procs: List[subprocess.Popen] = []
        self.env0 = {"RANK": "0", "LOCAL_RANK": "0", "WORLD_SIZE": str(self.world), "MASTER_ADDR": "127.0.0.1",
                     "MASTER_PORT": str(self.port)}
        cuda = all(d.startswith("cuda") for d in devs)
        visible = ",".join(str(i) for i in device_indices(devs)) if cuda else None
        parent_visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if cuda and parent_visible:                      # indices are relative to what the caller can see
            pv = parent_visible.split(",")
            visible = ",".join(pv[i] for i in device_indices(devs))
        spec = json.dumps({"cfg": asdict(cfg), "dp_size": dp_size, "ep_size": ep_size, "parent": os.getpid()})
        for r in range(1, self.world):
            env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(self.world), MASTER_ADDR="127.0.0.1",
                       MASTER_PORT=str(self.port), XLLM_OFFLINE_WORKER_SPEC=spec)
            if visible is not None:
                env["CUDA_VISIBLE_DEVICES"] = visible
            self.procs.append(subprocess.Popen([python, "-m", "xllm_b200.engine.offline_worker"], env=env))
        self.visible = visible

    def alive(self) -> bool:
        return all(p.poll() is None for p in self.procs)

    def wait(self, timeout: float = 20.0):
        for p in self.procs:
            try:
                p.wait(timeout=timeout)
            except subprocess.TimeoutExpired:
                p.terminate()
                try:
                    p.wait(timeout=5)
                except subprocess.TimeoutExpired:
                    p.kill()


class _Shim:
    """What `replica.lead_ranks` wraps: an engine and a shutdown hook."""

    def __init__(self, engine):
        self.engine = engine

    def shutdown(self):
        pass


def _watch_parent(pid: int):
    """A worker whose rank 0 died without saying stop would wait in a broadcast forever."""
    import time

    def loop():
        while True:
            try:
                os.kill(pid, 0)
            except OSError:
                os._exit(3)
            time.sleep(1.0)
    threading.Thread(target=loop, daemon=True).start()


def main() -> int:
    spec = json.loads(os.environ["XLLM_OFFLINE_WORKER_SPEC"])
    from ..parallel.state import init_parallel
    from .llm_engine import EngineConfig, LLMEngine
    from .replica import follow_rank0
    _watch_parent(int(spec["parent"]))
    cfg = EngineConfig(**spec["cfg"])
    cfg.device = "auto"
    ps = init_parallel(dp_size=spec["dp_size"], ep_size=spec["ep_size"])
    engine = LLMEngine(cfg, ps=ps)
    return follow_rank0(engine, ps)


if __name__ == "__main__":
    sys.exit(main())
