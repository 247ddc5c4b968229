"""Process-group topology: one process per GPU, groups derived from (world, dp, ep, cp).

Parity with the reference's CollectiveCommunicator / ParallelArgs
(xllm/core/framework/parallel_state/collective_communicator.cpp:317-639, parallel_args.h): per rank
a `world` group, a `tp` group of size world/dp (contiguous ranks), a strided `dp` group, and for MoE
a contiguous `moe_tp` group of size world/ep and a strided `moe_ep` group of size ep.  Groups are
``torch.distributed`` groups (NCCL on GPUs, gloo on CPU ranks); the fused sm_100a communication
kernels use symmetric-memory buffers registered per group (``xllm_b200.parallel.symm``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist


def tp_group_ranks(world: int, dp: int) -> List[List[int]]:
    tp = world // dp
    return [list(range(i * tp, (i + 1) * tp)) for i in range(dp)]


def dp_group_ranks(world: int, dp: int) -> List[List[int]]:
    tp = world // dp
    return [list(range(i, world, tp)) for i in range(tp)]


def moe_tp_group_ranks(world: int, ep: int) -> List[List[int]]:
    mtp = world // ep
    return [list(range(i * mtp, (i + 1) * mtp)) for i in range(ep)]


def moe_ep_group_ranks(world: int, ep: int) -> List[List[int]]:
    mtp = world // ep
    return [list(range(i, world, mtp)) for i in range(mtp)]


def cp_rank_layout(world: int, dp: int, cp: int):
    """rank = dp_idx * (cp * tp) + cp_idx * tp + tp_idx (the reference's CP layout,
    parallel_state/npu_cp_plan.h:34-120).  Returns (tp_groups, cp_groups)."""
    per_dp = world // dp
    tp = per_dp // cp
    tp_groups, cp_groups = [], []
    for d in range(dp):
        base = d * per_dp
        for c in range(cp):
            tp_groups.append([base + c * tp + t for t in range(tp)])
        for t in range(tp):
            cp_groups.append([base + c * tp + t for c in range(cp)])
    return tp_groups, cp_groups


@dataclass
class ParallelState:
    rank: int = 0
    world_size: int = 1
    dp_size: int = 1
    ep_size: int = 1
    cp_size: int = 1
    device: torch.device = field(default_factory=lambda: torch.device("cpu"))
    world_group: Optional[object] = None
    tp_group: Optional[object] = None
    dp_group: Optional[object] = None
    moe_tp_group: Optional[object] = None
    moe_ep_group: Optional[object] = None
    cp_group: Optional[object] = None
    tp_ranks: List[int] = field(default_factory=lambda: [0])
    comm: Optional[object] = None  # fused-kernel communicator (symmetric memory), set by symm.attach
    # a job may hold several independent serving instances (prefill / decode pairs): `rank` and
    # `world_size` above are those of THIS instance, the job-wide ones are below
    instance: int = 0
    n_instances: int = 1
    global_rank: int = 0
    job_group: Optional[object] = None
    leader: int = 0                # job rank of this instance's rank 0 (source of in-instance broadcasts)

    @property
    def tp_size(self) -> int:
        return self.world_size // self.dp_size // self.cp_size

    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp_size

    @property
    def dp_rank(self) -> int:
        return self.rank // (self.tp_size * self.cp_size)

    @property
    def moe_tp_size(self) -> int:
        return self.world_size // self.ep_size

    @property
    def ep_rank(self) -> int:
        return self.rank // self.moe_tp_size

    @property
    def moe_tp_rank(self) -> int:
        return self.rank % self.moe_tp_size

    # ------------------------------------------------------------------ collectives (library path)
    def all_reduce(self, x, group=None):
        g = group if group is not None else self.tp_group
        if g is None or dist.get_world_size(g) == 1:
            return x
        dist.all_reduce(x, group=g)
        return x

    def all_gather(self, x, dim=-1, group=None):
        g = group if group is not None else self.tp_group
        if g is None or dist.get_world_size(g) == 1:
            return x
        n = dist.get_world_size(g)
        x = x.contiguous()
        if x.dim() == 0:
            x = x.view(1)
        # concatenated along dim 0: the one output form every backend takes (gloo refuses the stacked one)
        flat = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(flat, x, group=g)
        out = flat.view((n,) + tuple(x.shape))
        if dim == 0:
            return out.reshape((n * x.shape[0],) + tuple(x.shape[1:]))
        d = dim % x.dim()
        return torch.cat(list(out.unbind(0)), dim=d)

    def reduce_scatter(self, x, group=None):
        """Sum across the group, each rank keeps its dim-0 shard (dim 0 must divide)."""
        g = group if group is not None else self.tp_group
        if g is None or dist.get_world_size(g) == 1:
            return x
        n = dist.get_world_size(g)
        out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=g)
        return out

    def broadcast(self, x, src=0, group=None):
        g = group if group is not None else self.world_group
        if g is None or dist.get_world_size(g) == 1:
            return x
        dist.broadcast(x, src=src, group=g)
        return x

    def barrier(self):
        if self.world_group is not None and self.world_size > 1:
            dist.barrier(group=self.world_group)

    def all_to_all_single(self, x, out_splits=None, in_splits=None, group=None):
        """Rank r's i-th dim-0 slice goes to rank i (equal slices, or `in_splits` / `out_splits` rows per
        peer).  Backends without a native all-to-all (gloo) run it as one exchange per peer pair."""
        g = group if group is not None else self.world_group
        if g is None or dist.get_world_size(g) == 1:
            return x
        n, me = dist.get_world_size(g), dist.get_rank(g)
        x = x.contiguous()
        if in_splits is None:
            in_splits = [x.shape[0] // n] * n
        if out_splits is None:
            out_splits = list(in_splits) if len(set(in_splits)) == 1 else None
            if out_splits is None:
                counts = torch.tensor(in_splits, dtype=torch.int64, device=x.device)
                gathered = [torch.empty_like(counts) for _ in range(n)]
                dist.all_gather(gathered, counts, group=g)
                out_splits = [int(c[me]) for c in gathered]
        out = torch.empty((sum(out_splits),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        if dist.get_backend(g) != "gloo":
            dist.all_to_all_single(out, x, out_splits, in_splits, group=g)
            return out
        ins, outs = list(x.split(in_splits)), list(out.split(out_splits))
        outs[me].copy_(ins[me])
        self.batch_send_recv([(ins[p], p) for p in range(n) if p != me], [(outs[p], p) for p in range(n) if p != me], group=g)
        return out

    def send(self, x, dst: int, group=None, tag: int = 0):
        g = group if group is not None else self.world_group
        dist.send(x.contiguous(), dst=dist.get_global_rank(g, dst) if g is not None else dst, group=g, tag=tag)

    def recv(self, x, src: int, group=None, tag: int = 0):
        g = group if group is not None else self.world_group
        dist.recv(x, src=dist.get_global_rank(g, src) if g is not None else src, group=g, tag=tag)
        return x

    def batch_send_recv(self, sends, recvs, group=None, max_wave_bytes: int = 256 << 20):
        """`sends` / `recvs`: [(tensor, peer rank in the group)].  The transfers are issued in waves of at most
        `max_wave_bytes` each way (a bound on staging memory; xllm's ProcessGroup::batch_isend_irecv with its
        p2p wave planning) and every wave is waited for before the next starts."""
        g = group if group is not None else self.world_group
        glob = (lambda r: dist.get_global_rank(g, r)) if g is not None else (lambda r: r)
        for wave in plan_p2p_waves(sends, recvs, max_wave_bytes):
            ops = [dist.P2POp(dist.isend, t.contiguous(), glob(p), g) for t, p in wave[0]] + \
                  [dist.P2POp(dist.irecv, t, glob(p), g) for t, p in wave[1]]
            if ops:
                for w in dist.batch_isend_irecv(ops):
                    w.wait()


def plan_p2p_waves(sends, recvs, max_wave_bytes: int):
    """Splits matched send / receive lists into waves whose payload stays under the bound per direction.
    Entry i of a rank's send list to peer p pairs with entry i of p's receive list from this rank, so both
    sides must cut at the same places: the cut depends only on the sizes, walked in peer order."""
    def nbytes(t):
        return t.numel() * t.element_size()

    def waves(items):
        out, cur, used = [], [], 0
        for t, p in sorted(items, key=lambda it: it[1]):
            b = nbytes(t)
            if cur and used + b > max_wave_bytes:
                out.append(cur)
                cur, used = [], 0
            cur.append((t, p))
            used += b
        if cur:
            out.append(cur)
        return out

    ws, wr = waves(sends), waves(recvs)
    n = max(len(ws), len(wr))
    return [(ws[i] if i < len(ws) else [], wr[i] if i < len(wr) else []) for i in range(n)]


_SINGLE = ParallelState()


def single() -> ParallelState:
    return _SINGLE


def init_parallel(dp_size: int = 1, ep_size: int = 1, cp_size: int = 1, backend: Optional[str] = None,
                  timeout_s: float = 600.0, instances: int = 1) -> ParallelState:
    """Join the job described by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT.
    With `instances` > 1 the job's ranks are cut into that many equal, contiguous slices and every
    slice becomes an independent instance (its own world / TP / DP / EP groups): the prefill and
    decode halves of a disaggregated deployment started by one launcher."""
    import datetime

    job_world = int(os.environ.get("WORLD_SIZE", "1"))
    job_rank = int(os.environ.get("RANK", "0"))
    assert job_world % instances == 0, (job_world, instances)
    world = job_world // instances
    inst, rank = divmod(job_rank, world)
    local = int(os.environ.get("LOCAL_RANK", str(job_rank)))
    use_cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if job_world == 1:
        return ParallelState(device=device)
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        kw = {}
        if backend == "nccl":
            kw["device_id"] = device
        dist.init_process_group(backend=backend, rank=job_rank, world_size=job_world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    assert world % (dp_size * cp_size) == 0 and world % ep_size == 0
    st = ParallelState(rank=rank, world_size=world, dp_size=dp_size, ep_size=ep_size, cp_size=cp_size,
                       device=device, instance=inst, n_instances=instances, global_rank=job_rank,
                       job_group=dist.group.WORLD, leader=inst * world)

    def make(groups):
        # `groups` are rank lists of ONE instance; every process of the job creates the groups of
        # every instance (group creation is collective over the job) and keeps its own
        mine = (None, [rank])
        for j in range(instances):
            for ranks in groups:
                job_ranks = [j * world + r for r in ranks]
                g = dist.new_group(job_ranks) if len(job_ranks) > 1 else None
                if job_rank in job_ranks:
                    mine = (g, ranks)
        return mine

    if instances == 1:
        st.world_group = dist.group.WORLD
    else:
        st.world_group, _ = make([list(range(world))])
    if world == 1:
        return st

    if cp_size > 1:
        tp_groups, cp_groups = cp_rank_layout(world, dp_size, cp_size)
        st.tp_group, st.tp_ranks = make(tp_groups)
        st.cp_group, _ = make(cp_groups)
    else:
        st.tp_group, st.tp_ranks = make(tp_group_ranks(world, dp_size))
    if dp_size > 1:
        st.dp_group, _ = make(dp_group_ranks(world, dp_size))
    if ep_size > 1:
        st.moe_tp_group, _ = make(moe_tp_group_ranks(world, ep_size))
        st.moe_ep_group, _ = make(moe_ep_group_ranks(world, ep_size))
    return st


def process_group_test(st: ParallelState) -> bool:
    """Start-up probe: an all-reduce and an all-gather of a [10, 10] tensor on the world group
    (the reference does the same before loading weights: llm_engine.cpp:164-186)."""
    if st.world_size == 1:
        return True
    x = torch.ones(10, 10, device=st.device, dtype=torch.float32)
    dist.all_reduce(x, group=st.world_group)
    ok = bool((x == st.world_size).all().item())
    out = torch.empty(st.world_size * 10, 10, device=st.device)
    dist.all_gather_into_tensor(out, torch.full((10, 10), float(st.rank), device=st.device), group=st.world_group)
    ok = ok and bool((out[::10, 0].cpu() == torch.arange(st.world_size, dtype=torch.float32)).all().item())
    return ok
