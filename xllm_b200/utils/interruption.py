"""Interruption bus and device monitor: the small common services of the reference
(xllm/core/common/interruption_bus.h, device_monitor.h).

`InterruptionBus` is a process-wide publish / subscribe point for "stop what you are doing" events
(shutdown signal, a watchdog's verdict, an admin request): subscribers are called in order of
registration, a failing subscriber does not stop the others, and late subscribers learn of an
interruption that already happened.

`DeviceMonitor` READS the GPUs' state through NVML (utilisation, memory, clocks, throttle reasons, power)
and publishes it as gauges; it never writes a setting.  Without NVML (CPU boxes, tests) it reads from an
injected fake with the same four calls.
"""
from __future__ import annotations

import signal
import threading
import time
from typing import Callable, Dict, List, Optional


class InterruptionBus:
    _instance: Optional["InterruptionBus"] = None

    def __init__(self):
        self._subs: List[Callable[[str], None]] = []
        self._lock = threading.Lock()
        self.reason: Optional[str] = None
        self.failures: List[str] = []

    @classmethod
    def instance(cls) -> "InterruptionBus":
        if cls._instance is None:
            cls._instance = InterruptionBus()
        return cls._instance

    def subscribe(self, fn: Callable[[str], None]):
        with self._lock:
            self._subs.append(fn)
            reason = self.reason
        if reason is not None:
            self._call(fn, reason)

    def publish(self, reason: str) -> int:
        with self._lock:
            if self.reason is not None:
                return 0
            self.reason = reason
            subs = list(self._subs)
        for fn in subs:
            self._call(fn, reason)
        return len(subs)

    def _call(self, fn, reason):
        try:
            fn(reason)
        except Exception as e:  # one subscriber must not silence the others
            self.failures.append(f"{getattr(fn, '__name__', fn)}: {type(e).__name__}: {e}")

    @property
    def interrupted(self) -> bool:
        return self.reason is not None

    def reset(self):
        with self._lock:
            self.reason = None
            self.failures.clear()

    def install_signal_handlers(self, signals=(signal.SIGTERM, signal.SIGINT)):
        for s in signals:
            signal.signal(s, lambda signum, _f: self.publish(f"signal {signal.Signals(signum).name}"))


class DeviceMonitor:
    """Read-only view of the GPUs.  `nvml` is any object with nvmlDeviceGetCount / HandleByIndex /
    UtilizationRates / MemoryInfo (pynvml's module by default)."""

    def __init__(self, nvml=None, publish: Optional[Callable[[str, float], None]] = None):
        self.nvml = nvml
        self.ok = False
        if nvml is None:
            try:
                import pynvml
                pynvml.nvmlInit()
                self.nvml, self.ok = pynvml, True
            except Exception:
                self.nvml = None
        else:
            self.ok = True
        self.publish = publish
        self._thread = None
        self._stop = threading.Event()
        self.last: List[Dict[str, float]] = []

    def sample(self) -> List[Dict[str, float]]:
        if not self.ok:
            return []
        n = self.nvml.nvmlDeviceGetCount()
        out = []
        for i in range(n):
            h = self.nvml.nvmlDeviceGetHandleByIndex(i)
            u = self.nvml.nvmlDeviceGetUtilizationRates(h)
            m = self.nvml.nvmlDeviceGetMemoryInfo(h)
            row = {"index": float(i), "gpu_util": float(u.gpu), "mem_util": float(u.memory), "mem_used": float(m.used),
                   "mem_total": float(m.total)}
            for key, fn, arg in (("sm_mhz", "nvmlDeviceGetClockInfo", 1), ("power_mw", "nvmlDeviceGetPowerUsage", None)):
                f = getattr(self.nvml, fn, None)
                if f is not None:
                    try:
                        row[key] = float(f(h, arg) if arg is not None else f(h))
                    except Exception:
                        pass
            out.append(row)
        self.last = out
        if self.publish and out:
            self.publish("xllm_gpu_num", float(n))
            self.publish("xllm_gpu_utilization", sum(r["gpu_util"] for r in out) / len(out))
        return out

    def start(self, period_seconds: float = 1.0):
        def loop():
            while not self._stop.wait(period_seconds):
                try:
                    self.sample()
                except Exception:
                    pass
        self._thread = threading.Thread(target=loop, daemon=True, name="xllm-device-monitor")
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
