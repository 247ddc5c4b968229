"""Keeping the schedulers of a multi-rank job in lock step.

Every rank runs the same deterministic scheduler, so the only thing non-zero ranks need from rank 0
is the stream of control events (new requests, aborts, pause/resume) in the order rank 0 applied
them, once per engine step.  Rank 0 broadcasts the list of events of a step over the process
group's object broadcast; the others apply it and step.  This replaces the reference's per-step
`ExecuteModel` RPC with serialized ForwardInput (xllm/core/distributed_runtime/remote_worker.cpp:165,
comm_channel.cpp:288-643) by a few bytes of control traffic.
"""
from __future__ import annotations

import torch.distributed as dist


def _bcast(obj, ps):
    ctl = getattr(ps, "ctl", None)
    if ctl is not None:                                   # ranks of one host: shared-memory ring, no collective
        if ps.rank == 0:
            ctl.send(obj)
            return obj
        return ctl.recv()
    box = [obj]
    dist.broadcast_object_list(box, src=getattr(ps, "leader", 0), group=ps.world_group)
    return box[0]


def _open_control(ps):
    """Both roles call this once, at the same point: the control channel of the instance."""
    if not hasattr(ps, "ctl"):
        from .shm_channel import open_for_group
        ps.ctl = open_for_group(ps)


def lead_ranks(server, ps):
    """Wrap rank 0's engine so that add_request / abort / pause / resume / step are mirrored."""
    eng = server.engine
    _open_control(ps)
    log = []
    orig_add, orig_abort, orig_pause, orig_resume, orig_step = eng.add_request, eng.abort, eng.pause, eng.resume, eng.step

    def add_request(*a, **kw):
        ok = orig_add(*a, **kw)
        if ok:
            log.append(("add", a, kw))
        return ok

    def abort(rid):
        log.append(("abort", (rid,), {}))
        return orig_abort(rid)

    def pause(mode="KEEP"):
        log.append(("pause", (mode,), {}))
        return orig_pause(mode)

    def resume():
        log.append(("resume", (), {}))
        return orig_resume()

    def step():
        _bcast(("step", list(log)), ps)
        log.clear()
        return orig_step()

    eng.add_request, eng.abort, eng.pause, eng.resume, eng.step = add_request, abort, pause, resume, step
    orig_shutdown = server.shutdown

    def shutdown():
        _bcast(("stop", []), ps)
        orig_shutdown()
        if getattr(ps, "ctl", None) is not None:
            import time
            time.sleep(0.2)                               # the followers read the stop before the segment goes
            ps.ctl.close()
            ps.ctl = None

    server.shutdown = shutdown


def follow_rank0(engine, ps) -> int:
    """Loop of a non-zero rank: apply rank 0's control events, then run the same step."""
    _open_control(ps)
    while True:
        kind, events = _bcast(None, ps)
        if kind == "stop":
            if getattr(ps, "ctl", None) is not None:
                ps.ctl.close()
            return 0
        for name, a, kw in events:
            getattr(engine, {"add": "add_request"}.get(name, name))(*a, **kw)
        engine.step()
