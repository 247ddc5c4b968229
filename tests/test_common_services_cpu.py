"""Rank launcher, interruption bus, device monitor (against a fake NVML)."""
import os
import signal
import subprocess
import sys
import time
from types import SimpleNamespace

from xllm_b200 import launch_server
from xllm_b200.utils.interruption import DeviceMonitor, InterruptionBus

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_launcher_builds_rank_commands():
    cmds = launch_server.build_commands(4, ["--model=/m", "--port=9000"], "127.0.0.1", 19000, python="py")
    assert len(cmds) == 4
    r, argv, env = cmds[2]
    assert r == 2 and argv[:3] == ["py", "-m", "xllm_b200.serve"] and "--nnodes=4" in argv and "--node_rank=2" in argv
    assert "--master_node_addr=127.0.0.1:19000" in argv and env["RANK"] == "2" and env["WORLD_SIZE"] == "4"
    assert "--nnodes=1" not in launch_server.build_commands(1, [], "127.0.0.1", 1)[0][1]


def test_launcher_takes_the_job_down_when_a_rank_exits(tmp_path, monkeypatch):
    """Children are stand-ins: rank 1 exits with code 3 after a moment, rank 0 would run forever."""
    script = tmp_path / "fake_rank.py"
    script.write_text("import os, sys, time\nif os.environ['RANK'] == '1':\n    time.sleep(0.3); sys.exit(3)\ntime.sleep(60)\n")

    def fake_build(nproc, server_args, addr, port, python=sys.executable):
        return [(r, [python, str(script)], {"RANK": str(r)}) for r in range(nproc)]

    monkeypatch.setattr(launch_server, "build_commands", fake_build)
    t0 = time.time()
    code = launch_server.launch(2, [], log_dir=str(tmp_path), grace_seconds=5.0, poll_seconds=0.05)
    assert code == 3 and time.time() - t0 < 20
    assert (tmp_path / "rank0.log").exists() and (tmp_path / "rank1.log").exists()


def test_interruption_bus_orders_isolates_and_remembers():
    bus = InterruptionBus()
    seen = []
    bus.subscribe(lambda r: seen.append(("a", r)))
    bus.subscribe(lambda r: (_ for _ in ()).throw(RuntimeError("boom")))
    bus.subscribe(lambda r: seen.append(("c", r)))
    assert not bus.interrupted
    assert bus.publish("watchdog: rank 3 silent") == 3
    assert seen == [("a", "watchdog: rank 3 silent"), ("c", "watchdog: rank 3 silent")]
    assert bus.interrupted and len(bus.failures) == 1 and "boom" in bus.failures[0]
    assert bus.publish("again") == 0                       # the first reason stands
    bus.subscribe(lambda r: seen.append(("late", r)))       # late subscribers still learn of it
    assert seen[-1] == ("late", "watchdog: rank 3 silent")
    bus.reset()
    assert not bus.interrupted


def test_device_monitor_reads_a_fake_nvml_and_publishes_gauges():
    calls = []
    fake = SimpleNamespace(
        nvmlDeviceGetCount=lambda: 2,
        nvmlDeviceGetHandleByIndex=lambda i: i,
        nvmlDeviceGetUtilizationRates=lambda h: SimpleNamespace(gpu=40 + 20 * h, memory=10),
        nvmlDeviceGetMemoryInfo=lambda h: SimpleNamespace(used=1 << 30, total=180 << 30),
        nvmlDeviceGetClockInfo=lambda h, kind: 1620,
        nvmlDeviceGetPowerUsage=lambda h: 900000)
    out = {}
    mon = DeviceMonitor(fake, publish=lambda k, v: out.__setitem__(k, v))
    rows = mon.sample()
    assert [r["gpu_util"] for r in rows] == [40.0, 60.0] and rows[0]["sm_mhz"] == 1620.0
    assert out == {"xllm_gpu_num": 2.0, "xllm_gpu_utilization": 50.0}
    # nothing in the monitor can write a device setting: it only ever calls Get* functions
    assert all(n.startswith("nvmlDeviceGet") for n in vars(fake))
