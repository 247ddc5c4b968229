"""Heartbeats, registry leases and host-side failure detection (gloo ranks, no GPU involved)."""
import os
import socket
import subprocess
import sys

import pytest
import torch.distributed as dist

from xllm_b200.engine.health import HealthState, HeartbeatMonitor, InstanceInfo, InstanceRegistry, KV

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_monitor_and_registry_with_fake_clock():
    now = [100.0]
    kv = KV(dist.HashStore())
    mons = [HeartbeatMonitor(kv, r, 3, timeout_s=2.0, clock=lambda: now[0]) for r in range(3)]
    for m in mons:
        m.beat()
    assert mons[0].check()
    now[0] += 1.5
    mons[0].beat(); mons[1].beat()            # rank 2 goes silent
    now[0] += 1.0
    state = HealthState()
    mons[0].on_failure.append(state.fail)
    assert mons[0].dead_ranks() == [2] and not mons[0].check()
    assert not state.healthy and "2" in state.reason
    mons[1].leave()
    assert mons[0].dead_ranks() == [1, 2]

    reg = InstanceRegistry(kv, lease_s=5.0, clock=lambda: now[0])
    reg.register(InstanceInfo("p0", "PREFILL", "127.0.0.1:9000", tp_size=4))
    reg.register(InstanceInfo("d0", "DECODE", "127.0.0.1:9001", tp_size=4))
    reg.register(InstanceInfo("d1", "DECODE", "127.0.0.1:9002", tp_size=4))
    assert [i.name for i in reg.list("DECODE")] == ["d0", "d1"]
    assert reg.pick("PREFILL").address == "127.0.0.1:9000"
    now[0] += 4.0
    reg.heartbeat(InstanceInfo("d0", "DECODE", "127.0.0.1:9001", tp_size=4))
    now[0] += 2.0                                  # d1's and p0's leases ran out
    assert [i.name for i in reg.list()] == ["d0"]
    reg.deregister("d0")
    assert reg.list() == [] and reg.pick("DECODE") is None


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("mode", ["leave", "silent"])
def test_rank_that_leaves_between_steps_is_noticed_on_the_host(mode):
    world = 3
    env = dict(os.environ, WORLD_SIZE=str(world), QUITTER="2", QUIT_MODE=mode, HB_PORT=str(_free_port()),
               INIT=f"tcp://127.0.0.1:{_free_port()}", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "mp_heartbeat_worker.py")],
                              env=dict(env, RANK=str(r)), stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
             for r in range(world)]
    outs = [p.communicate(timeout=120) for p in procs]
    assert all(p.returncode == 0 for p in procs), [o[1][-800:] for o in outs]
    for r in (0, 1):
        # steps 0-2 with three ranks, steps 3-5 with the two survivors
        assert f"RANK{r} total={3 * 3 + 3 * 2} alive=[0, 1]" in outs[r][0], outs[r]
