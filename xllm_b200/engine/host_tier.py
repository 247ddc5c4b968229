"""Host-memory tier of the KV prefix cache.

Parity: `HierarchyBlockManagerPool` / `HierarchyKVCacheTransfer` (xllm/core/framework/block/
hierarchy_block_manager_pool.h:42, kv_cache_transfer/hierarchy_kv_cache_transfer.*): KV blocks that
the device prefix cache evicts are kept in (pinned) host memory under the same chained block hash;
a later request whose prefix misses on the device but hits on the host gets those blocks copied back
before it is scheduled, so it skips their prefill.

Data movement per step is two batched copies at most: one gather of the evicted blocks (device ->
pinned host, issued right after scheduling and before the step's kernels overwrite the blocks) and
one scatter of the promoted blocks (host -> device, at admission).  With 180 GB of HBM the device
tier is large; the host tier matters for long shared prefixes (system prompts, RAG corpora).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import List, Sequence, Tuple

import torch


class HostKVTier:
    def __init__(self, kv_caches, num_host_blocks: int, block_manager, rt, block_size: int):
        self.kv = kv_caches
        self.bm = block_manager
        self.rt = rt
        self.block_size = block_size
        self.n = int(num_host_blocks)
        k0 = kv_caches[0][0]
        self.device = k0.device
        shape = (len(kv_caches), 2, self.n) + tuple(k0.shape[1:])
        pin = k0.is_cuda
        self.store = torch.empty(shape, dtype=k0.dtype, pin_memory=pin)
        self.free: List[int] = list(range(self.n - 1, -1, -1))
        self.index: "OrderedDict[Tuple[int, int], int]" = OrderedDict()   # hash -> host slot, LRU order
        self.saved = self.loaded = self.dropped = 0
        self.bm.set_track_evictions(True)

    # ------------------------------------------------------------------ device -> host
    def save_evicted(self):
        """Call after scheduling a step and before running it."""
        ev = self.bm.take_evictions()
        if not ev:
            return 0
        blocks, slots = [], []
        for b, lo, hi in ev:
            key = (lo, hi)
            if key in self.index:
                self.index.move_to_end(key)
                continue
            if not self.free:
                old, slot = self.index.popitem(last=False)
                self.free.append(slot)
                self.dropped += 1
            slot = self.free.pop()
            self.index[key] = slot
            blocks.append(b)
            slots.append(slot)
        if not blocks:
            return 0
        bi = torch.as_tensor(blocks, dtype=torch.long, device=self.device)
        si = torch.as_tensor(slots, dtype=torch.long)
        for l, (k, v) in enumerate(self.kv):
            self.store[l, 0, si] = k[bi].to("cpu", non_blocking=False)
            self.store[l, 1, si] = v[bi].to("cpu", non_blocking=False)
        self.saved += len(blocks)
        return len(blocks)

    # ------------------------------------------------------------------ host -> device
    def prefetch(self, tokens: Sequence[int], extra: int = 0) -> int:
        """Promote the host-resident continuation of the device-resident prefix of `tokens`.
        Returns the number of blocks copied to the device."""
        chain = self.rt.block_hash_chain([int(t) for t in tokens], self.block_size, extra)
        max_blocks = (len(tokens) - 1) // self.block_size
        blocks, slots = [], []
        for lo, hi in chain[:max_blocks]:
            if self.bm.lookup(lo, hi) >= 0:
                continue
            slot = self.index.get((lo, hi))
            if slot is None:
                break
            b = self.bm.insert_cached(lo, hi)
            if b < 0:
                break
            self.index.move_to_end((lo, hi))
            blocks.append(b)
            slots.append(slot)
        # taking blocks for the promotion may itself have evicted colder ones
        self.save_evicted()
        if not blocks:
            return 0
        bi = torch.as_tensor(blocks, dtype=torch.long, device=self.device)
        si = torch.as_tensor(slots, dtype=torch.long)
        for l, (k, v) in enumerate(self.kv):
            k[bi] = self.store[l, 0, si].to(self.device, non_blocking=True)
            v[bi] = self.store[l, 1, si].to(self.device, non_blocking=True)
        self.loaded += len(blocks)
        return len(blocks)

    def stats(self):
        return {"host_blocks": self.n, "host_used": len(self.index), "saved": self.saved, "loaded": self.loaded,
                "dropped": self.dropped}
