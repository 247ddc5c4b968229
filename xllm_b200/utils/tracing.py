"""Tracing helpers: NVTX ranges, profiler back ends and the request trace log.

* `nvtx_range(name)`: a range in the Nsight timeline when CUDA is present, free otherwise
  (the reference: RAII NvtxRange, xllm/core/platform/cuda/cuda_utils.h:28-33).
* `Profiler(backend)`: "torch" records a Kineto trace (CPU + CUDA activities) and writes
  `xllm_rank{r}_{pid}_{ts}.pt.trace.json`; "cuda" brackets the window with cudaProfilerStart / Stop so
  that an external profiler started with a capture range records only it (the reference:
  platform/torch_profiler.cpp:60-137, platform/cuda_profiler.cpp:23-60, flag `--profile_backend`).
* `TraceLog`: per-request event lines (arrival, first token, finish, with timings) into a rotating
  file; when disabled a call costs one attribute test (the reference: util/verbose_trace_logger.h).
"""
from __future__ import annotations

import contextlib
import json
import logging
import logging.handlers
import os
import time

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class Profiler:
    def __init__(self, backend: str = "torch", rank: int = 0):
        if backend not in ("torch", "cuda"):
            raise ValueError(f"unknown profile backend {backend!r}")
        self.backend, self.rank = backend, rank
        self._prof = None
        self.active = False

    def start(self):
        if self.active:
            return
        if self.backend == "torch":
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._prof = torch.profiler.profile(activities=acts)
            self._prof.__enter__()
        elif torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
        self.active = True

    def stop(self, profile_dir: str = ".") -> str:
        """Returns the path of the trace ("" for the cuda back end: the external profiler owns the file)."""
        if not self.active:
            return ""
        self.active = False
        if self.backend == "torch":
            self._prof.__exit__(None, None, None)
            os.makedirs(profile_dir, exist_ok=True)
            path = os.path.join(profile_dir, f"xllm_rank{self.rank}_{os.getpid()}_{int(time.time())}.pt.trace.json")
            self._prof.export_chrome_trace(path)
            self._prof = None
            return path
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        return ""


class TraceLog:
    def __init__(self, path: str = "", max_bytes: int = 64 << 20, backups: int = 3):
        self.enabled = bool(path)
        self._log = None
        if self.enabled:
            self._log = logging.getLogger(f"xllm_b200.trace.{id(self)}")
            self._log.setLevel(logging.INFO)
            self._log.propagate = False
            h = logging.handlers.RotatingFileHandler(path, maxBytes=max_bytes, backupCount=backups)
            h.setFormatter(logging.Formatter("%(message)s"))
            self._log.addHandler(h)
            self._handler = h

    def event(self, request_id: str, what: str, **fields):
        if not self.enabled:
            return
        self._log.info(json.dumps(dict(ts=round(time.time(), 6), request_id=request_id, event=what, **fields)))

    def close(self):
        if self.enabled:
            self._handler.close()
            self._log.removeHandler(self._handler)
            self.enabled = False
