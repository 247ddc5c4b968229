"""Context parallelism: zig-zag sharding is balanced and invertible, merged partial attention states
equal full attention, CP prefill and DCP decode over gloo ranks match the single-rank result."""
import os
import socket
import subprocess
import sys

import torch

from xllm_b200.parallel import context_parallel as cp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_zigzag_and_merge():
    shards = cp.zigzag_shards(1000, 4)
    assert sorted(torch.cat(shards).tolist()) == list(range(1000))
    work = [int((s + 1).sum()) for s in shards]           # causal work ~ sum of (position + 1)
    assert max(work) / min(work) < 1.02
    x = torch.randn(1000, 3)
    assert torch.equal(cp.restore_order([x[s] for s in shards], shards), x)
    torch.manual_seed(1)
    q, k, v = torch.randn(5, 4, 8), torch.randn(37, 2, 8), torch.randn(37, 2, 8)
    full, lse = cp.attention_with_lse(q, k, v, 0.3, causal=False)
    cuts = [(0, 10), (10, 11), (11, 37)]
    parts = [cp.attention_with_lse(q, k[a:b], v[a:b], 0.3, causal=False) for a, b in cuts]
    out, lse2 = cp.merge_states([p[0] for p in parts], [p[1] for p in parts])
    assert torch.allclose(out, full, atol=1e-5) and torch.allclose(lse2, lse, atol=1e-5)


def test_cp_and_dcp_over_gloo_ranks():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    world = 3
    env = dict(os.environ, WORLD_SIZE=str(world), INIT=f"tcp://127.0.0.1:{port}",
               PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "mp_cp_worker.py")], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(world)]
    outs = [p.communicate(timeout=120) for p in procs]
    assert all(p.returncode == 0 for p in procs), [o[1][-800:] for o in outs]
    assert all(f"CP_OK {r}" in outs[r][0] for r in range(world))
