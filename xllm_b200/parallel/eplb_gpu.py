"""Expert re-placement on the GPUs: the worker side of expert-parallel load balancing.

`ExpertStore` keeps the expert weights of one MoE layer in symmetric memory, twice (an active and a
spare buffer).  A new placement is prepared by PULLING, for every local slot, the weights of its new
expert from whichever rank holds that expert now (`xllm_peer_copy`: plain peer loads, one kernel per
tensor) into the spare buffer; once every rank has done so (a group barrier) the layer switches to
the spare buffer at a step boundary.  Placements here are permutations (every expert exactly once):
the router's rows are permuted the same way, so that the router emits PHYSICAL slot ids and
everything downstream of it (counts, dispatch, grouped GEMMs, combine) is untouched.

Parity: EplbExecutor's prepare / activate with a spare weight buffer
(xllm/core/framework/eplb/eplb_executor.cpp, llm_engine.cpp:1259-1302); the policy is
`parallel/eplb.py`.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch
import torch.distributed as dist

from .eplb import balanced_placement


class ExpertStore:
    def __init__(self, block, group, rank: int, world: int):
        import torch.distributed._symmetric_memory as symm_mem
        from ..ops import _lib
        from ..ops._lib import L, P
        _lib.register_signature("xllm_peer_copy", [P, P, L, P])
        assert not block.fp8 and block.args.n_group == 1, "re-placement supports bf16 experts and ungrouped routing"
        self.block, self.group, self.rank, self.world = block, group, rank, world
        w1, w2 = block.w_gate_up, block.w_down
        self.e_local, self.E = w1.shape[0], w1.shape[0] * world
        self.n1, self.n2 = w1[0].numel(), w2[0].numel()
        esz = w1.element_size()
        # one half = [gate_up of every local slot | down of every local slot], both contiguous
        self.b1, self.b2 = self.n1 * esz, self.n2 * esz
        assert self.b1 % 16 == 0 and self.b2 % 16 == 0
        self.off2 = (self.e_local * self.b1 + 255) & ~255
        self.half = (self.off2 + self.e_local * self.b2 + 255) & ~255
        self.buf = symm_mem.empty(2 * self.half, dtype=torch.uint8, device=w1.device)
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.active = 0
        self.shape1, self.shape2, self.dtype = tuple(w1.shape), tuple(w2.shape), w1.dtype
        v1, v2 = self._views(0)
        v1.copy_(w1)
        v2.copy_(w2)
        self._install()
        # physical slot p (= rank * e_local + s) holds logical expert placement[p]
        self.placement: List[int] = list(range(self.E))
        self.gate_logical = block.gate.weight.detach().clone()
        self.bias_logical = block.bias.detach().clone() if getattr(block, "bias", None) is not None else None
        self.load = torch.zeros(self.E, dtype=torch.float32, device=w1.device)   # tokens per PHYSICAL slot
        self.moved_bytes = 0
        self.hdl.barrier()

    # ---- buffers
    def _views(self, half: int):
        """(gate_up [e_local, 2I, H], down [e_local, H, I]) of one buffer half."""
        base = half * self.half
        v1 = self.buf[base: base + self.e_local * self.b1].view(self.dtype).view(self.shape1)
        v2 = self.buf[base + self.off2: base + self.off2 + self.e_local * self.b2].view(self.dtype).view(self.shape2)
        return v1, v2

    def _install(self):
        v1, v2 = self._views(self.active)
        b = self.block
        b.w_gate_up, b.w_down = v1, v2
        b._params["experts.gate_up"], b._params["experts.down"] = v1, v2

    # ---- statistics
    def logical_load(self) -> np.ndarray:
        phys = self.load.cpu().numpy()
        out = np.zeros(self.E)
        for p, e in enumerate(self.placement):
            out[e] += phys[p]
        return out

    # ---- re-placement (collective: every rank of the group calls these in the same order)
    def plan(self, min_gain: float = 0.05) -> Optional[List[int]]:
        """All-reduces the loads, returns the new placement (the same on every rank) or None."""
        total = self.load.clone()
        dist.all_reduce(total, group=self.group)
        phys = total.cpu().numpy()
        load = np.zeros(self.E)
        for p, e in enumerate(self.placement):
            load[e] += phys[p]
        if load.sum() <= 0:
            return None
        per_rank = lambda pl: np.array([sum(load[e] for e in pl[r * self.e_local:(r + 1) * self.e_local])
                                        for r in range(self.world)])
        cur = per_rank(self.placement)
        rows = balanced_placement(load, self.world, 0)
        new = [e for row in rows for e in row]
        nl = per_rank(new)
        if cur.max() / max(cur.mean(), 1e-9) - nl.max() / max(nl.mean(), 1e-9) < min_gain:
            return None
        return new

    def prepare(self, new_placement: List[int]):
        from ..ops import _lib
        from ..ops._lib import check, stream
        lib = _lib.load()
        where = {e: p for p, e in enumerate(self.placement)}
        spare = 1 - self.active
        mine = int(self.hdl.buffer_ptrs[self.rank])
        for s in range(self.e_local):
            e = new_placement[self.rank * self.e_local + s]
            src_rank, src_slot = divmod(where[e], self.e_local)
            peer = int(self.hdl.buffer_ptrs[src_rank])
            for off, nb in ((0, self.b1), (self.off2, self.b2)):
                src = peer + self.active * self.half + off + src_slot * nb
                dst = mine + spare * self.half + off + s * nb
                check(lib.xllm_peer_copy(dst, src, nb, stream()), "peer_copy")
            if src_rank != self.rank:
                self.moved_bytes += self.b1 + self.b2
        torch.cuda.current_stream().synchronize()
        dist.barrier(group=self.group)          # every rank has read what it needs from the active buffers

    def activate(self, new_placement: List[int]):
        self.active = 1 - self.active
        self.placement = list(new_placement)
        self._install()
        perm = torch.tensor(new_placement, dtype=torch.long, device=self.gate_logical.device)
        self.block.gate.weight.copy_(self.gate_logical[perm])
        if self.bias_logical is not None:
            self.block.bias.copy_(self.bias_logical[perm])
        self.load.zero_()
        torch.cuda.current_stream().synchronize()
        dist.barrier(group=self.group)          # nobody prepares the next placement before all have switched

    def rebalance(self, min_gain: float = 0.05) -> bool:
        new = self.plan(min_gain)
        if new is None:
            return False
        self.prepare(new)
        self.activate(new)
        return True
