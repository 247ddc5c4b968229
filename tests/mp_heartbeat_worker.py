"""Worker for test_health_cpu.py: gloo ranks step together; one rank leaves between steps and the
others must notice on the host (store) before entering the next collective."""
import os
import sys
import time

import torch
import torch.distributed as dist

from xllm_b200.engine.health import HeartbeatMonitor, KV


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    quitter = int(os.environ["QUITTER"])
    mode = os.environ.get("QUIT_MODE", "leave")
    dist.init_process_group("gloo", rank=rank, world_size=world, init_method=os.environ["INIT"])
    store = dist.TCPStore("127.0.0.1", int(os.environ["HB_PORT"]), world, rank == 0, wait_for_workers=False)
    mon = HeartbeatMonitor(KV(store), rank, world, timeout_s=2.0)   # generous: a loaded test host must not look like a dead rank
    alive = list(range(world))
    group = dist.group.WORLD
    total = 0
    for step in range(6):
        mon.beat(step)
        if rank == quitter and step == 3:
            if mode == "leave":
                mon.leave()
            # a rank leaves only between steps: nothing of its own is in flight
            os._exit(0)
        # give the quitter's announcement (or silence) time to show up, then look before launching
        deadline = time.time() + (0.3 if mode == "leave" else 3.0)
        while step >= 3 and time.time() < deadline:
            mon.beat(step)                    # a live rank keeps beating while it waits
            time.sleep(0.05)
        mon.beat(step)
        dead = [r for r in mon.dead_ranks() if r in alive]
        if dead:
            alive = [r for r in alive if r not in dead]
            group = None                      # survivors stop using the old group; host-only from here
        if group is not None:
            t = torch.ones(1)
            dist.all_reduce(t, group=group)
            total += int(t.item())
        else:
            total += len(alive)
    print(f"RANK{rank} total={total} alive={alive}", flush=True)
    # rank 0 hosts the store: it leaves last, or the others' final beats meet a closed socket
    store.set(f"done{rank}", "1")
    if rank == 0:
        import datetime
        try:
            store.wait([f"done{r}" for r in alive], datetime.timedelta(seconds=20))
        except Exception:
            pass
    os._exit(0)


if __name__ == "__main__":
    main()
