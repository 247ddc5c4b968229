"""Ulysses / CFG / encoder-DP groups on gloo ranks."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world,cfg", [(2, 1), (4, 2), (4, 1)])
def test_dit_parallel_groups(world, cfg):
    env = dict(os.environ, CFG_SIZE=str(cfg), PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29650 + world + cfg),
           os.path.join(ROOT, "tests", "mp_dit_parallel_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "DIT_PARALLEL_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
