"""ParallelState collectives (all-to-all equal / ragged, wave-planned batched send / receive, broadcast,
all-gather) on gloo ranks, and the wave planner alone."""
import os
import subprocess
import sys

import pytest
import torch

from xllm_b200.parallel.state import plan_p2p_waves

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_wave_planner_cuts_both_directions_at_the_bound():
    t = lambda n: torch.empty(n, dtype=torch.uint8)
    sends = [(t(40), 2), (t(40), 1), (t(10), 1), (t(100), 3)]
    recvs = [(t(30), 1)]
    waves = plan_p2p_waves(sends, recvs, 64)
    assert [[(x.numel(), p) for x, p in s] for s, _ in waves] == [[(40, 1), (10, 1)], [(40, 2)], [(100, 3)]]
    assert [[(x.numel(), p) for x, p in r] for _, r in waves] == [[(30, 1)], [], []]
    assert plan_p2p_waves([], [], 64) == []


@pytest.mark.parametrize("world", [2, 3])
def test_collectives_on_gloo(world):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29670 + world),
           os.path.join(ROOT, "tests", "mp_collectives_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "COLLECTIVES_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
