"""Host-side platform services: NUMA placement of a rank next to its GPU, and the process-wide lock that
keeps other threads off the device while a CUDA graph is being captured.

Parity: xllm/core/platform/numa_utils.h (is_numa_available, get_num_numa_nodes, get_device_numa_node,
bind_process_to_numa_node, bind_thread_to_numa_node, get_current_numa_node) and the graph-capture lock of
the CUDA-graph executor (core/runtime/cuda_graph_executor_impl.cpp).

The topology is read from sysfs (`/sys/devices/system/node`, `/sys/bus/pci/devices/<bdf>/numa_node`), the
binding is `sched_setaffinity` on the process or the calling thread; every function takes the sysfs root as
an argument so that the logic is testable on a fake tree.  With one NUMA node (or none visible) everything
is a no-op that reports so.
"""
from __future__ import annotations

import os
import threading
from contextlib import contextmanager
from typing import List, Optional

_SYS = "/sys"


def _read(path: str) -> Optional[str]:
    try:
        with open(path) as f:
            return f.read().strip()
    except OSError:
        return None


def parse_cpulist(text: str) -> List[int]:
    """'0-3,8,10-11' -> [0, 1, 2, 3, 8, 10, 11]."""
    cpus: List[int] = []
    for part in (text or "").split(","):
        part = part.strip()
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.extend(range(int(lo), int(hi or lo) + 1))
    return cpus


def numa_nodes(sys_root: str = _SYS) -> List[int]:
    base = os.path.join(sys_root, "devices/system/node")
    try:
        return sorted(int(n[4:]) for n in os.listdir(base) if n.startswith("node") and n[4:].isdigit())
    except OSError:
        return []


def is_numa_available(sys_root: str = _SYS) -> bool:
    return len(numa_nodes(sys_root)) > 1


def node_cpus(node: int, sys_root: str = _SYS) -> List[int]:
    return parse_cpulist(_read(os.path.join(sys_root, f"devices/system/node/node{node}/cpulist")) or "")


def pci_bus_id(device_index: int) -> Optional[str]:
    """'0000:1b:00.0' of a CUDA device (lower case, as sysfs spells it), or None without a GPU."""
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        props = torch.cuda.get_device_properties(device_index)
        return f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
    except Exception:
        return None


def device_numa_node(device_index: int, sys_root: str = _SYS, bus_id: Optional[str] = None) -> int:
    """NUMA node the GPU hangs off, -1 when the platform does not say."""
    bus_id = bus_id or pci_bus_id(device_index)
    if not bus_id:
        return -1
    text = _read(os.path.join(sys_root, "bus/pci/devices", bus_id.lower(), "numa_node"))
    try:
        return int(text) if text is not None else -1
    except ValueError:
        return -1


def current_numa_node(sys_root: str = _SYS) -> int:
    """Node of the CPUs this thread may run on when they all belong to one node, else -1."""
    allowed = set(os.sched_getaffinity(0))
    for n in numa_nodes(sys_root):
        cpus = set(node_cpus(n, sys_root))
        if allowed and allowed <= cpus:
            return n
    return -1


def bind_to_numa_node(node: int, sys_root: str = _SYS, thread_only: bool = False, setter=None) -> List[int]:
    """Restricts the process (or the calling thread) to the node's CPUs that it was allowed before; returns
    the CPU list it ended up with ([] = nothing changed).  Memory follows by first touch."""
    cpus = set(node_cpus(node, sys_root))
    if not cpus:
        return []
    pid = threading.get_native_id() if thread_only else 0
    setter = setter or os.sched_setaffinity
    allowed = set(os.sched_getaffinity(0))
    target = sorted(cpus & allowed) or sorted(cpus)
    try:
        setter(pid, target)
    except OSError:
        return []
    return target


def bind_rank_to_device(device_index: int, sys_root: str = _SYS, bus_id: Optional[str] = None, setter=None) -> List[int]:
    """What a rank does at start-up (`XLLM_NUMA_BIND=0` turns it off): sit on the CPUs of its GPU's node so
    that pinned staging buffers and the scheduler thread are local to the PCIe root of the device."""
    if os.environ.get("XLLM_NUMA_BIND", "1") == "0" or not is_numa_available(sys_root):
        return []
    node = device_numa_node(device_index, sys_root, bus_id)
    if node < 0:
        return []
    return bind_to_numa_node(node, sys_root, setter=setter)


# ------------------------------------------------------------------------------------------ capture lock
_CAPTURE = threading.RLock()
_capturing = threading.local()


@contextmanager
def graph_capture():
    """Held by the model runner around warm-up + capture of a CUDA graph.  Anything another thread of the
    process wants to launch meanwhile (a second engine served by the same process, an image pipeline, the
    KV push of a PD pair) takes `device_work()` first and so waits: a launch from another thread on a
    capturing device would either fail the capture or be recorded into it."""
    with _CAPTURE:
        depth = getattr(_capturing, "depth", 0)
        _capturing.depth = depth + 1
        try:
            yield
        finally:
            _capturing.depth = depth


@contextmanager
def device_work():
    """For threads other than the engine loop: excludes graph capture for the duration of the block."""
    with _CAPTURE:
        yield


def capturing() -> bool:
    return getattr(_capturing, "depth", 0) > 0
