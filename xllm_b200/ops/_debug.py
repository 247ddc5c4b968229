"""`XLLM_BOUNDS_CHECK=1`: every index tensor handed to a kernel is range-checked on the host side of the
launch (token ids against the vocabulary, cache slots against the cache, block-table entries against the
number of blocks, lengths against the table width, positions against the rotary table), and a violation
raises with the operator's name instead of becoming an out-of-range access on the device.

Parity: the reference's debug builds run its kernels under a memory checker; here the check sits at the
operator boundary, costs one reduction + one device-to-host read per index tensor (so it is a debugging
mode, off by default), and works the same on CPU tensors, which is how it is tested.
"""
from __future__ import annotations

import os

import torch


class BoundsError(IndexError):
    pass


def enabled() -> bool:
    return os.environ.get("XLLM_BOUNDS_CHECK", "0") == "1"


def check_range(t, lo: int, hi: int, what: str, allow_negative_skip: bool = False):
    """Every element of `t` in [lo, hi); with `allow_negative_skip` negative entries mean "skip" and pass."""
    if t is None or t.numel() == 0 or not enabled():
        return
    mn, mx = int(t.min()), int(t.max())
    if mx >= hi or (mn < lo and not allow_negative_skip):
        raise BoundsError(f"{what}: values span [{mn}, {mx}], allowed [{lo}, {hi})")


def check_block_table(block_table, lens, n_blocks: int, page: int, what: str):
    """The entries a kernel will read (the first ceil(len / page) of every row) name existing blocks, and
    no length runs past the table."""
    if not enabled() or block_table is None or block_table.numel() == 0:
        return
    width = block_table.shape[1]
    need = (lens.to(torch.int64) + page - 1) // page
    if int(need.max()) > width:
        raise BoundsError(f"{what}: a sequence of {int(lens.max())} tokens needs {int(need.max())} blocks, the table has {width}")
    used = torch.arange(width, device=block_table.device)[None, :] < need[:, None]
    vals = block_table.to(torch.int64)
    bad = used & ((vals < 0) | (vals >= n_blocks))
    if bool(bad.any()):
        r, c = [int(x[0]) for x in torch.nonzero(bad, as_tuple=True)]
        raise BoundsError(f"{what}: block_table[{r}, {c}] = {int(vals[r, c])}, the cache has {n_blocks} blocks")
