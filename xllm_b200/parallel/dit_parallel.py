"""Parallel groups of diffusion transformers and vision towers: Ulysses sequence parallelism,
classifier-free-guidance (CFG) parallelism, encoder data parallelism.

Parity: the DiT groups of the reference's parallel state (xllm/core/framework/parallel_state/
parallel_state.cpp:300-444: `sp` (Ulysses) groups, `cfg` groups, TP of the VAE / text encoder) and the
encoder-DP mode of its communicator (collective_communicator.cpp:332-348).

Rank layout of a job of `world` ranks: rank = cfg_rank * sp_size + sp_rank.  The `sp` group of a rank
holds the ranks that share its CFG branch (contiguous), the `cfg` group the ranks that hold the same
sequence shard of the other branch (strided).

  * Ulysses: activations are sharded along the SEQUENCE; around attention an all-to-all turns the
    layout into "all of the sequence, 1/sp of the HEADS" and back, so attention itself is local and
    exact.  On CUDA the all-to-all runs over peer memory in one kernel when a symmetric workspace is
    attached (`AllToAll`), else through the process group.
  * CFG parallel: the conditional and the unconditional branch of a guided step run on different ranks
    and are combined after an all-gather of the two velocity predictions.
  * Encoder DP: the items of a batch (images of a request batch) are dealt to the ranks, every rank
    encodes its share, results are all-gathered back in order (ragged lengths padded for the wire).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


# ------------------------------------------------------------------------------------------ layout
def sp_group_ranks(world: int, cfg_size: int) -> List[List[int]]:
    sp = world // cfg_size
    return [list(range(c * sp, (c + 1) * sp)) for c in range(cfg_size)]


def cfg_group_ranks(world: int, cfg_size: int) -> List[List[int]]:
    sp = world // cfg_size
    return [list(range(s, world, sp)) for s in range(sp)]


@dataclass
class DitParallelState:
    rank: int = 0
    world_size: int = 1
    cfg_size: int = 1
    sp_group: Optional[object] = None
    cfg_group: Optional[object] = None
    world_group: Optional[object] = None
    a2a: Optional[object] = None          # peer-memory all-to-all (CUDA), see AllToAll

    @property
    def sp_size(self) -> int:
        return self.world_size // self.cfg_size

    @property
    def sp_rank(self) -> int:
        return self.rank % self.sp_size

    @property
    def cfg_rank(self) -> int:
        return self.rank // self.sp_size


def init_dit_parallel(cfg_size: int = 1, rank: Optional[int] = None, world: Optional[int] = None) -> DitParallelState:
    """Create the groups on top of an initialised default process group."""
    if not dist.is_initialized():
        return DitParallelState()
    rank = dist.get_rank() if rank is None else rank
    world = dist.get_world_size() if world is None else world
    assert world % cfg_size == 0 and cfg_size in (1, 2), (world, cfg_size)
    st = DitParallelState(rank=rank, world_size=world, cfg_size=cfg_size, world_group=dist.group.WORLD)
    for ranks in sp_group_ranks(world, cfg_size):
        g = dist.new_group(ranks) if len(ranks) > 1 else None
        if rank in ranks:
            st.sp_group = g
    for ranks in cfg_group_ranks(world, cfg_size):
        g = dist.new_group(ranks) if len(ranks) > 1 else None
        if rank in ranks:
            st.cfg_group = g
    return st


# ------------------------------------------------------------------------------------------ Ulysses
def all_to_all(x: torch.Tensor, group, scatter_dim: int, gather_dim: int, a2a=None) -> torch.Tensor:
    """Splits `scatter_dim` into n parts, sends part r to rank r, concatenates what arrives along
    `gather_dim` (n = group size).  Both dims must divide / be equal across ranks."""
    n = dist.get_world_size(group) if group is not None else 1
    if n == 1:
        return x
    if a2a is not None and x.is_cuda:
        return a2a(x, scatter_dim, gather_dim)
    parts = [p.contiguous() for p in x.chunk(n, dim=scatter_dim)]
    if dist.get_backend(group) == "gloo":
        # gloo has no all-to-all: gather every rank's tensor and keep the parts addressed to this rank
        me = dist.get_rank(group)
        everything = [torch.empty_like(x) for _ in range(n)]
        dist.all_gather(everything, x.contiguous(), group=group)
        return torch.cat([t.chunk(n, dim=scatter_dim)[me] for t in everything], dim=gather_dim)
    recv = [torch.empty_like(parts[0]) for _ in range(n)]
    dist.all_to_all(recv, parts, group=group)
    return torch.cat(recv, dim=gather_dim)


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, st: DitParallelState,
                      attn_fn: Optional[Callable] = None) -> torch.Tensor:
    """q, k, v: [B, heads, T_local, d] (this rank's shard of the sequence) -> [B, heads, T_local, d].
    heads must be divisible by the sp size."""
    attn_fn = attn_fn or torch.nn.functional.scaled_dot_product_attention
    if st.sp_group is None or st.sp_size == 1:
        return attn_fn(q, k, v)
    assert q.shape[1] % st.sp_size == 0, "Ulysses needs heads % sp_size == 0"
    # sequence-sharded -> head-sharded: scatter heads (dim 1), gather sequence (dim 2)
    qh, kh, vh = (all_to_all(t, st.sp_group, 1, 2, st.a2a) for t in (q, k, v))
    oh = attn_fn(qh, kh, vh)
    # back: scatter sequence, gather heads
    return all_to_all(oh, st.sp_group, 2, 1, st.a2a)


def shard_sequence(x: torch.Tensor, st: DitParallelState, dim: int = 1) -> torch.Tensor:
    if st.sp_size == 1:
        return x
    assert x.shape[dim] % st.sp_size == 0
    return x.chunk(st.sp_size, dim=dim)[st.sp_rank].contiguous()


def gather_sequence(x: torch.Tensor, st: DitParallelState, dim: int = 1) -> torch.Tensor:
    if st.sp_group is None or st.sp_size == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(st.sp_size)]
    dist.all_gather(parts, x.contiguous(), group=st.sp_group)
    return torch.cat(parts, dim=dim)


class AllToAll:
    """The Ulysses exchange over peer memory (CUDA): one kernel (`a2a_permute_kernel`, comm.cu) stores
    every element straight into its place in the destination rank's receive area, in the head-sharded
    (or sequence-sharded) layout, and one flag exchange completes the call.  Attach to a
    DitParallelState as `st.a2a`; used by `all_to_all` for bf16 4-D tensors with scatter / gather dims
    (1, 2) or (2, 1), anything else goes through the process group."""

    def __init__(self, group, rank: int, world: int, device, max_bytes: int):
        import torch.distributed._symmetric_memory as symm_mem
        from ..ops import _lib
        from ..ops._lib import I, L, P
        _lib.register_signature("xllm_a2a_permute", [P, P, P, L, L, L, P, P, I, I, I, I, I, I, I, P])
        self.group, self.rank, self.world, self.device = group, rank, world, device
        self.half = (int(max_bytes) + 255) & ~255
        self.buf = symm_mem.empty(2 * self.half, dtype=torch.uint8, device=device)
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.peer_ptrs = self.hdl.buffer_ptrs_dev
        self.signal_ptrs = self.hdl.signal_pad_ptrs_dev
        self.sig_off = self.hdl.signal_pad_size // 8 + 160       # its own 32-slot group in the upper half of the pad
        self.state = torch.zeros(2, dtype=torch.int32, device=device)
        self.err = torch.zeros(1, dtype=torch.int32, device=device)
        self.calls = 0
        self.hdl.barrier()

    def __call__(self, x: torch.Tensor, scatter_dim: int, gather_dim: int) -> torch.Tensor:
        ok = (x.dim() == 4 and x.dtype == torch.bfloat16 and (scatter_dim, gather_dim) in ((1, 2), (2, 1))
              and x.shape[3] % 8 == 0 and x.numel() * 2 <= self.half)
        if not ok:
            parts = [p.contiguous() for p in x.chunk(self.world, dim=scatter_dim)]
            recv = [torch.empty_like(parts[0]) for _ in range(self.world)]
            dist.all_to_all(recv, parts, group=self.group)
            return torch.cat(recv, dim=gather_dim)
        from ..ops import _count, _lib
        from ..ops._lib import check, ptr, stream
        x = x.contiguous()
        d0, d1, d2, E = x.shape
        mode = 0 if scatter_dim == 1 else 1
        check(_lib.load().xllm_a2a_permute(ptr(x), self.peer_ptrs, self.signal_ptrs, 0, self.half, self.sig_off,
                                           ptr(self.state), ptr(self.err), d0, d1, d2, E, mode, self.rank, self.world,
                                           stream()), "a2a_permute")
        _count()
        self.calls += 1
        half = (self.calls & 1) * self.half               # the kernel's epoch is the call count
        shape = (d0, d1 // self.world, d2 * self.world, E) if mode == 0 else (d0, d1 * self.world, d2 // self.world, E)
        n = d0 * d1 * d2 * E
        # copy out: the area is reused by the call after next
        return self.buf[half: half + 2 * n].view(torch.bfloat16).view(shape).clone()

    def error_status(self) -> int:
        v = int(self.err.item())
        if v:
            self.err.zero_()
        return v


# ------------------------------------------------------------------------------------------ CFG parallel
def cfg_combine(branch_out: torch.Tensor, st: DitParallelState, guidance_scale: float) -> torch.Tensor:
    """Every rank holds the prediction of ITS branch (cfg_rank 0: conditional, 1: unconditional);
    returns uncond + scale * (cond - uncond) on every rank."""
    if st.cfg_group is None or st.cfg_size == 1:
        return branch_out
    both = [torch.empty_like(branch_out) for _ in range(2)]
    dist.all_gather(both, branch_out.contiguous(), group=st.cfg_group)
    cond, uncond = both[0], both[1]
    return uncond + guidance_scale * (cond - uncond)


# ------------------------------------------------------------------------------------------ encoder DP
def encoder_dp(items: Sequence, encode: Callable[[Sequence], List[torch.Tensor]], group, rank: int,
               world: int) -> List[torch.Tensor]:
    """`encode(list of items) -> list of [n_i, D] tensors`.  Item i is encoded by rank i % world; every
    rank returns the results of ALL items in order."""
    if group is None or world == 1:
        return encode(list(items))
    mine = [i for i in range(len(items)) if i % world == rank]
    outs = encode([items[i] for i in mine]) if mine else []
    ref = outs[0] if outs else None
    # agree on the feature width / dtype and on every item's row count
    meta = torch.zeros(len(items) + 1, dtype=torch.int64)
    for i, o in zip(mine, outs):
        meta[i] = o.shape[0]
    meta[-1] = ref.shape[1] if ref is not None else 0
    dev = ref.device if ref is not None else torch.device("cpu")
    meta = meta.to(dev) if dist.get_backend(group) == "nccl" else meta
    gathered = [torch.empty_like(meta) for _ in range(world)]
    dist.all_gather(gathered, meta, group=group)
    rows = torch.stack([g[:-1] for g in gathered]).max(0).values.tolist()
    width = int(max(int(g[-1]) for g in gathered))
    per_rank = max(sum(rows[i] for i in range(len(items)) if i % world == r) for r in range(world))
    dtype = ref.dtype if ref is not None else torch.float32
    buf = torch.zeros(max(per_rank, 1), width, dtype=dtype, device=meta.device if meta.is_cuda else dev)
    if outs:
        buf[: sum(o.shape[0] for o in outs)] = torch.cat(outs, 0)
    allb = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(allb, buf, group=group)
    result: List[Optional[torch.Tensor]] = [None] * len(items)
    for r in range(world):
        off = 0
        for i in range(len(items)):
            if i % world == r:
                result[i] = allb[r][off: off + rows[i]]
                off += rows[i]
    return result  # type: ignore[return-value]
