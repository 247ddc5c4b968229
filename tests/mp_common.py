"""Shared harness of the multi-GPU test workers (tests/mp_*.py).

A worker's checks run inside `guarded(body)`.  Pass / fail is made collective: every rank computes
its own verdict, the ranks agree on the minimum over a gloo (CPU) group, synchronise their devices,
pass a barrier and tear the process group down together, and only then does a failing rank report
and exit non-zero.  No rank leaves while another one may still be inside a collective or a
flag-wait kernel that needs it, and none leaves while its symmetric memory is still in use by a peer.
"""
import sys
import traceback

import torch
import torch.distributed as dist


def guarded(body):
    """body() -> message printed by rank 0 when every rank passed."""
    err = None
    msg = None
    try:
        msg = body()
    except BaseException:  # noqa: BLE001 - the verdict must reach the agreement below whatever happened
        err = traceback.format_exc()
    all_ok = err is None
    rank = 0
    if dist.is_initialized():
        rank = dist.get_rank()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        g = dist.new_group(backend="gloo")
        t = torch.tensor([0 if err else 1], dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=g)
        all_ok = bool(t.item())
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dist.barrier(group=g)
        dist.destroy_process_group()
    if err is not None:
        # on stdout as well: the launcher's own report fills the tail of stderr
        print(f"[rank {rank}] FAILED\n{err}", flush=True)
        sys.stderr.write(f"[rank {rank}] FAILED\n{err}\n")
        sys.stderr.flush()
    if all_ok and rank == 0 and msg:
        print(msg, flush=True)
    sys.exit(0 if all_ok else 1)
