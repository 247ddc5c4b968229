"""Host-side fault hooks and the device-status watchdog.

Faults are injected on the host only (`XLLM_FAULT`, a comma-separated list):

    worker_exit@step=N[@rank=R]   the rank raises SystemExit at the start of engine step N
    raise@step=N[@rank=R]         the rank raises RuntimeError at engine step N
    slow_rank_ms=K[@rank=R]       every engine step of the rank sleeps K milliseconds first
    rpc_drop=P                    heartbeats / registry writes are dropped with probability P

No hook touches a GPU: a rank leaves between steps with none of its kernels in flight, and the others
learn of it through the store (engine/health.py) before their next launch.  A device-side fault
injector is deliberately not part of this module.

`DeviceWatchdog` turns what the kernels report into health state: every bounded wait that expired
left a non-zero word behind (GEMM, attention, communication kernels); the watchdog polls those words
and marks the instance unhealthy with the reason, so that `/health` answers 503 and an orchestrator
recycles the instance (the reference: HealthCheckManager::set_unhealthy,
xllm/core/common/health_check_manager.h:33-125, /health reporter server/health_reporter.h:27-54).
"""
from __future__ import annotations

import os
import random
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional


@dataclass
class FaultPlan:
    exit_step: Optional[int] = None
    raise_step: Optional[int] = None
    slow_ms: float = 0.0
    drop_prob: float = 0.0
    refused: bool = False
    rng: random.Random = field(default_factory=lambda: random.Random(0))

    @staticmethod
    def parse(spec: str, rank: int = 0) -> "FaultPlan":
        plan = FaultPlan()
        for item in filter(None, (s.strip() for s in (spec or "").split(","))):
            parts = item.split("@")
            head, quals = parts[0], dict(q.split("=", 1) for q in parts[1:] if "=" in q)
            if "rank" in quals and int(quals["rank"]) != rank:
                continue
            if head == "worker_exit":
                plan.exit_step = int(quals["step"])
            elif head == "raise":
                plan.raise_step = int(quals["step"])
            elif head.startswith("slow_rank_ms="):
                plan.slow_ms = float(head.split("=", 1)[1])
            elif head.startswith("rpc_drop="):
                plan.drop_prob = float(head.split("=", 1)[1])
            else:
                raise ValueError(f"unknown fault {item!r}")
        return plan

    @staticmethod
    def from_env(rank: int = 0) -> Optional["FaultPlan"]:
        spec = os.environ.get("XLLM_FAULT", "")
        return FaultPlan.parse(spec, rank) if spec else None

    def before_step(self, step: int, sleep: Callable[[float], None] = time.sleep, multicast_bound: bool = False):
        """`multicast_bound`: this rank's memory is bound to an NVLink multicast object (a fused
        communicator with a multimem mapping, NVLS).  A rank must not leave while that is so - the
        other ranks' multimem accesses would fault - so the hooks that end the rank are refused: they
        log once and the step goes on.  Run such experiments with XLLM_TP_MULTIMEM=0 and
        NCCL_NVLS_ENABLE=0."""
        if self.slow_ms > 0:
            sleep(self.slow_ms / 1e3)
        leaving = (self.exit_step is not None and step >= self.exit_step) or \
                  (self.raise_step is not None and step == self.raise_step)
        if leaving and multicast_bound:
            if not self.refused:
                self.refused = True
                import logging
                logging.getLogger("xllm_b200.fault").warning(
                    "XLLM_FAULT worker_exit / raise refused at step %d: this rank's memory is bound to an NVLink "
                    "multicast object; set XLLM_TP_MULTIMEM=0 and NCCL_NVLS_ENABLE=0 to use these hooks", step)
            return
        if self.exit_step is not None and step >= self.exit_step:
            raise SystemExit(f"XLLM_FAULT: worker_exit at step {step}")
        if self.raise_step is not None and step == self.raise_step:
            raise RuntimeError(f"XLLM_FAULT: raise at step {step}")

    def drop(self) -> bool:
        return self.drop_prob > 0 and self.rng.random() < self.drop_prob


class DeviceWatchdog:
    """Polls error words.  `sources`: name -> callable returning an int (0 = fine)."""

    def __init__(self, sources: Optional[Dict[str, Callable[[], int]]] = None, on_unhealthy: Optional[Callable[[str], None]] = None):
        self.sources = dict(sources or {})
        self.on_unhealthy = on_unhealthy
        self.reasons: List[str] = []

    @staticmethod
    def for_engine(engine, on_unhealthy=None) -> "DeviceWatchdog":
        src: Dict[str, Callable[[], int]] = {}
        if engine.device.type == "cuda":
            from ..ops import _lib, gemm_tcgen05
            src["gemm"] = gemm_tcgen05.error_status
            src["attention"] = lambda: int(_lib.load().xllm_fmha_error_status())
        comm = getattr(engine.ps, "comm", None)
        if comm is not None:
            src["tp_comm"] = comm.error_status
        return DeviceWatchdog(src, on_unhealthy)

    def check(self) -> bool:
        """True when everything is fine; otherwise records the reasons and calls `on_unhealthy`."""
        bad = []
        for name, fn in self.sources.items():
            try:
                v = int(fn())
            except Exception as e:          # a source that cannot be read is itself a finding
                bad.append(f"{name}: status unreadable ({e})")
                continue
            if v != 0:
                bad.append(f"{name}: a bounded wait expired (status {v})")
        if bad:
            self.reasons.extend(bad)
            if self.on_unhealthy is not None:
                self.on_unhealthy("; ".join(bad))
        return not bad
