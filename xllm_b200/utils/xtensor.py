"""Tensors over virtual address ranges whose physical pages come from a pool shared by all models
on a device (csrc/runtime/vmm.h).

    pool = VmmPool(device=0, page_bytes=2 << 20, max_pages=4096)
    kv = pool.range(64 << 30)              # reserves addresses only
    kv.ensure(8 << 30)                     # maps the first 8 GiB
    t = kv.tensor((n_blocks, heads, 16, 128), torch.bfloat16)
    kv.release_all()                       # sleep: pages go back to the pool, `t` keeps its address
    kv.ensure(8 << 30)                     # wake up (contents are whatever the pages held)

Parity: the reference's XTensor allocator and physical page pool
(xllm/core/framework/xtensor/xtensor_allocator.cpp, phy_page_pool.cpp), used there so that several
models can share one device and swap in and out without re-capturing graphs.  On a machine without a
CUDA driver the pool runs on a host-memory emulation with the same semantics.
"""
from __future__ import annotations

import ctypes
import math

import torch


class _CudaView:
    def __init__(self, ptr, shape, dtype):
        code = {torch.float32: "<f4", torch.float16: "<f2", torch.bfloat16: "<u2", torch.uint8: "|u1",
                torch.int32: "<i4", torch.int64: "<i8", torch.float8_e4m3fn: "|u1"}[dtype]
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": code, "data": (int(ptr), False), "version": 3,
                                         "strides": None}


class VmmRange:
    def __init__(self, pool: "VmmPool", virt_bytes: int):
        from .. import _rt
        self.pool = pool
        self.x = _rt.XTensor(pool.p, int(virt_bytes))

    ptr = property(lambda self: self.x.ptr)
    virt_bytes = property(lambda self: self.x.virt_bytes)
    mapped_bytes = property(lambda self: self.x.mapped_bytes)

    def ensure(self, nbytes: int):
        self.x.ensure(int(nbytes))

    def map_range(self, offset: int, nbytes: int):
        self.x.map_range(int(offset), int(nbytes))

    def unmap_range(self, offset: int, nbytes: int):
        self.x.unmap_range(int(offset), int(nbytes))

    def release_all(self):
        self.x.release_all()

    def tensor(self, shape, dtype=torch.uint8, offset: int = 0) -> torch.Tensor:
        """A tensor over [offset, offset + numel * itemsize) of the range.  It is valid while those
        bytes are mapped; across release_all() / ensure() it keeps its address."""
        n = math.prod(shape)
        item = torch.empty((), dtype=dtype).element_size()
        if offset + n * item > self.virt_bytes:
            raise ValueError("tensor does not fit the reserved range")
        if self.pool.fake:
            buf = (ctypes.c_char * (n * item)).from_address(self.ptr + offset)
            return torch.frombuffer(buf, dtype=dtype, count=n).view(*shape)
        view = _CudaView(self.ptr + offset, shape, dtype)
        t = torch.as_tensor(view, device=torch.device("cuda", self.pool.device))
        return t.view(dtype) if t.dtype != dtype else t


class VmmPool:
    def __init__(self, device: int = 0, page_bytes: int = 2 << 20, max_pages: int = 1024, fake=None):
        from .. import _rt
        if fake is None:
            fake = not (torch.cuda.is_available() and _rt.vmm_cuda_available())
        self.fake = bool(fake)
        self.device = device
        if not self.fake:
            torch.zeros(1, device=torch.device("cuda", device))    # the driver calls want an initialised device
        self.p = _rt.PhyPagePool(device, int(page_bytes), int(max_pages), self.fake)

    page_bytes = property(lambda self: self.p.page_bytes)
    pages_in_use = property(lambda self: self.p.pages_in_use)
    pages_free = property(lambda self: self.p.pages_free)
    pages_created = property(lambda self: self.p.pages_created)

    def range(self, virt_bytes: int) -> VmmRange:
        return VmmRange(self, virt_bytes)

    def trim(self) -> int:
        return self.p.trim()


_SHARED = {}


def shared_pool(device, page_bytes: int = 2 << 20, max_pages: int = 0, fake=None) -> VmmPool:
    """The page pool of a device, shared by every engine of the process (several models on one GPU
    take turns on the same physical pages: one sleeps, another wakes up)."""
    dev = torch.device(device)
    key = (dev.type, dev.index or 0)
    if key not in _SHARED:
        if not max_pages:
            if dev.type == "cuda" and torch.cuda.is_available():
                max_pages = int(torch.cuda.get_device_properties(dev).total_memory // page_bytes)
            else:
                max_pages = 4096
        _SHARED[key] = VmmPool(dev.index or 0, page_bytes, max_pages, fake=fake if dev.type == "cuda" else True)
    return _SHARED[key]
