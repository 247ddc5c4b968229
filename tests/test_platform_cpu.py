"""NUMA placement against a fake sysfs tree, and the graph-capture lock."""
import os
import threading
import time

from xllm_b200.utils import platform as plat


def _fake_sys(tmp_path, nodes):
    for n, cpus in nodes.items():
        d = tmp_path / "devices/system/node" / f"node{n}"
        d.mkdir(parents=True)
        (d / "cpulist").write_text(cpus + "\n")
    dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    return str(tmp_path)


def test_numa_topology_and_binding(tmp_path):
    assert plat.parse_cpulist("0-3,8,10-11") == [0, 1, 2, 3, 8, 10, 11]
    me = sorted(os.sched_getaffinity(0))
    half = max(1, len(me) // 2)
    spell = lambda cpus: ",".join(str(c) for c in cpus)
    root = _fake_sys(tmp_path, {0: spell(me[:half]), 1: spell(me[half:] or me[:1])})
    assert plat.numa_nodes(root) == [0, 1] and plat.is_numa_available(root)
    assert plat.node_cpus(0, root) == me[:half]
    assert plat.device_numa_node(0, root, bus_id="0000:1B:00.0") == 1
    assert plat.device_numa_node(0, root, bus_id="0000:ff:00.0") == -1
    calls = []
    got = plat.bind_rank_to_device(0, root, bus_id="0000:1b:00.0", setter=lambda pid, cpus: calls.append((pid, list(cpus))))
    assert got == (me[half:] or me[:1]) and calls == [(0, got)]
    os.environ["XLLM_NUMA_BIND"] = "0"
    try:
        assert plat.bind_rank_to_device(0, root, bus_id="0000:1b:00.0", setter=lambda *a: calls.append(a)) == []
    finally:
        del os.environ["XLLM_NUMA_BIND"]
    single = _fake_sys(tmp_path / "one", {0: spell(me)})
    assert not plat.is_numa_available(single)
    assert plat.bind_rank_to_device(0, single, bus_id="0000:1b:00.0") == []
    assert plat.current_numa_node(single) == 0


def test_capture_lock_excludes_other_threads():
    order = []

    def other():
        with plat.device_work():
            order.append("other")

    with plat.graph_capture():
        assert plat.capturing()
        t = threading.Thread(target=other)
        t.start()
        time.sleep(0.1)
        with plat.graph_capture():          # re-entrant for the capturing thread
            order.append("capture")
    t.join(timeout=5)
    assert order == ["capture", "other"] and not plat.capturing()
