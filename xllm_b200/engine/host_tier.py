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

import os
from collections import OrderedDict
from typing import List, Optional, Sequence, Tuple

import torch


class KVCacheStore:
    """Third tier: blocks the host tier drops go to a store that outlives the process and can be shared by the
    instances of a node (`enable_kvcache_store`; the reference's Mooncake-store client,
    xllm/core/framework/kv_cache_transfer/kv_cache_store.*).  Interface: put / get / contains by block
    hash; a block is one contiguous byte string (all layers, K then V)."""

    def put(self, key: Tuple[int, int], blob: torch.Tensor) -> bool:
        raise NotImplementedError

    def get(self, key: Tuple[int, int], out: torch.Tensor) -> bool:
        raise NotImplementedError

    def contains(self, key: Tuple[int, int]) -> bool:
        raise NotImplementedError


class MemoryKVStore(KVCacheStore):
    def __init__(self, capacity_blocks: int = 1 << 30):
        self.cap = capacity_blocks
        self.data: "OrderedDict[Tuple[int, int], torch.Tensor]" = OrderedDict()

    def put(self, key, blob):
        self.data[key] = blob.clone()
        self.data.move_to_end(key)
        while len(self.data) > self.cap:
            self.data.popitem(last=False)
        return True

    def get(self, key, out):
        t = self.data.get(key)
        if t is None:
            return False
        out.copy_(t)
        self.data.move_to_end(key)
        return True

    def contains(self, key):
        return key in self.data


class DirectoryKVStore(KVCacheStore):
    """One file per block under a directory (a tmpfs or NVMe mount), named by the block hash and the cache
    geometry; written to a temporary name and renamed, so that concurrent instances only ever see whole
    blocks.  `capacity_bytes` is enforced by deleting the least recently used files."""

    def __init__(self, path: str, geometry: str, capacity_bytes: int = 0):
        self.dir = os.path.join(path, geometry)
        os.makedirs(self.dir, exist_ok=True)
        self.cap = capacity_bytes

    def _file(self, key):
        return os.path.join(self.dir, f"{key[0] & (2 ** 64 - 1):016x}{key[1] & (2 ** 64 - 1):016x}.kv")

    def put(self, key, blob):
        f = self._file(key)
        if os.path.exists(f):
            os.utime(f)
            return True
        tmp = f"{f}.{os.getpid()}.tmp"
        try:
            with open(tmp, "wb") as fh:
                fh.write(blob.contiguous().view(torch.uint8).numpy().tobytes())
            os.replace(tmp, f)
        except OSError:
            return False
        if self.cap > 0:
            self._trim()
        return True

    def _trim(self):
        files = [(e.stat().st_atime, e.stat().st_size, e.path) for e in os.scandir(self.dir) if e.name.endswith(".kv")]
        total = sum(sz for _, sz, _ in files)
        for _, sz, path in sorted(files):
            if total <= self.cap:
                break
            try:
                os.unlink(path)
                total -= sz
            except OSError:
                pass

    def get(self, key, out):
        f = self._file(key)
        try:
            with open(f, "rb") as fh:
                raw = fh.read()
        except OSError:
            return False
        flat = out.view(torch.uint8).view(-1)
        if len(raw) != flat.numel():
            return False                                  # another geometry or a torn file: treat as a miss
        flat.copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
        os.utime(f)
        return True

    def contains(self, key):
        return os.path.exists(self._file(key))


class HostKVTier:
    def __init__(self, kv_caches, num_host_blocks: int, block_manager, rt, block_size: int,
                 store: Optional[KVCacheStore] = None):
        self.ext = store
        self.ext_saved = self.ext_loaded = 0
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
        total = 0

        def flush():
            nonlocal total
            if not blocks:
                return
            bi = torch.as_tensor(blocks, dtype=torch.long, device=self.device)
            si = torch.as_tensor(slots, dtype=torch.long)
            for l, (k, v) in enumerate(self.kv):
                self.store[l, 0, si] = k[bi].to("cpu", non_blocking=False)
                self.store[l, 1, si] = v[bi].to("cpu", non_blocking=False)
            total += len(blocks)
            blocks.clear()
            slots.clear()

        for b, lo, hi in ev:
            key = (lo, hi)
            if key in self.index:
                self.index.move_to_end(key)
                continue
            if not self.free and not self._drop_lru(protect=slots):
                flush()                                    # more evictions than host slots: fill them, then recycle
                self._drop_lru()
            slot = self.free.pop()
            self.index[key] = slot
            blocks.append(b)
            slots.append(slot)
        flush()
        self.saved += total
        return total

    def _drop_lru(self, protect=()) -> bool:
        """Frees the coldest host slot that is not in `protect`; with an external store its block moves there
        instead of vanishing.  False when every slot is protected."""
        for key, slot in self.index.items():
            if slot in protect:
                continue
            del self.index[key]
            if self.ext is not None and self.ext.put(key, self.store[:, :, slot]):
                self.ext_saved += 1
            self.free.append(slot)
            self.dropped += 1
            return True
        return False

    def _from_store(self, key, protect=()) -> Optional[int]:
        """Host slot holding `key` after fetching it from the external store (None: not there, or no host
        slot can be freed because all of them wait to be copied to the device)."""
        if self.ext is None or not self.ext.contains(key):
            return None
        if not self.free and not self._drop_lru(protect):
            return None
        slot = self.free.pop()
        buf = torch.empty(self.store[:, :, slot].shape, dtype=self.store.dtype)
        if not self.ext.get(key, buf):
            self.free.append(slot)
            return None
        self.store[:, :, slot] = buf
        self.index[key] = slot
        self.ext_loaded += 1
        return slot

    # ------------------------------------------------------------------ host -> device
    def prefetch(self, tokens: Sequence[int], extra: int = 0) -> int:
        """Promote the host-resident (or store-resident) continuation of the device-resident prefix of
        `tokens`.  Returns the number of blocks copied to the device."""
        chain = self.rt.block_hash_chain([int(t) for t in tokens], self.block_size, extra)
        max_blocks = (len(tokens) - 1) // self.block_size
        blocks, slots = [], []
        total = 0

        def flush():
            nonlocal total
            if not blocks:
                return
            bi = torch.as_tensor(blocks, dtype=torch.long, device=self.device)
            si = torch.as_tensor(slots, dtype=torch.long)
            for l, (k, v) in enumerate(self.kv):
                k[bi] = self.store[l, 0, si].to(self.device, non_blocking=True)
                v[bi] = self.store[l, 1, si].to(self.device, non_blocking=True)
            if self.device.type == "cuda":
                torch.cuda.current_stream().synchronize()     # the host slots may be reused right away
            total += len(blocks)
            blocks.clear()
            slots.clear()

        for lo, hi in chain[:max_blocks]:
            if self.bm.lookup(lo, hi) >= 0:
                continue
            slot = self.index.get((lo, hi))
            if slot is None:
                slot = self._from_store((lo, hi), protect=slots)
                if slot is None and slots and self.ext is not None and self.ext.contains((lo, hi)):
                    flush()                                # every host slot was waiting for its copy: copy, then retry
                    slot = self._from_store((lo, hi))
            if slot is None:
                break
            b = self.bm.insert_cached(lo, hi)
            if b < 0:
                break
            self.index.move_to_end((lo, hi))
            blocks.append(b)
            slots.append(slot)
        flush()
        # taking blocks for the promotion may itself have evicted colder ones
        self.save_evicted()
        self.loaded += total
        return total

    def stats(self):
        return {"host_blocks": self.n, "host_used": len(self.index), "saved": self.saved, "loaded": self.loaded,
                "dropped": self.dropped, "store_saved": self.ext_saved, "store_loaded": self.ext_loaded}
