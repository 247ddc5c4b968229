"""Data-parallel attention with expert parallelism: two gloo ranks with different requests, the
experts split over both; the rank that runs out of work keeps joining the MoE collectives with dummy
steps, and every request decodes exactly as on a single full model."""
import json
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_dp_attention_lockstep_and_outputs():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.path.join(ROOT, "tests") + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "mp_dp_attention_worker.py")],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    res = {}
    for line in r.stdout.splitlines():
        if line.startswith("RESULT"):
            _, rank, payload = line.split(" ", 2)
            res[int(rank)] = json.loads(payload)
    assert set(res) == {0, 1}
    for rank in (0, 1):
        assert res[rank]["out"] == res[rank]["want"], res[rank]
    assert res[0]["dp_steps"] == res[1]["dp_steps"]          # both ranks ran the same number of forwards
    assert res[1]["fake"] > 0 and res[0]["fake"] == 0          # rank 1 idled through rank 0's long decode
