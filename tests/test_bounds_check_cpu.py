"""XLLM_BOUNDS_CHECK=1: out-of-range index tensors raise at the operator boundary; valid ones pass and the
mode costs nothing when off."""
import pytest
import torch

from xllm_b200 import ops
from xllm_b200.ops import _debug
from xllm_b200.ops import reference as ref


def _cache(nb=4, nkv=2, page=16, d=32):
    return torch.randn(nb, nkv, page, d), torch.randn(nb, nkv, page, d)


def test_bounds_mode(monkeypatch):
    kc, vc = _cache()
    q = torch.randn(2, 4, 32)
    good_bt = torch.tensor([[1, 2], [3, 0]], dtype=torch.int32)
    lens = torch.tensor([20, 5], dtype=torch.int32)
    bad_bt = torch.tensor([[1, 9], [3, 0]], dtype=torch.int32)            # block 9 of a 4-block cache, and it is used
    unused_bad = torch.tensor([[1, 2], [3, 77]], dtype=torch.int32)      # the second row needs one block only
    # off: nothing is checked at the boundary (the CPU reference would index out of range by itself)
    monkeypatch.delenv("XLLM_BOUNDS_CHECK", raising=False)
    ops.paged_decode_attention(q, kc, vc, unused_bad, lens, 0.2)
    monkeypatch.setenv("XLLM_BOUNDS_CHECK", "1")
    ops.paged_decode_attention(q, kc, vc, good_bt, lens, 0.2)
    ops.paged_decode_attention(q, kc, vc, unused_bad, lens, 0.2)          # entries beyond a row's length are never read
    with pytest.raises(_debug.BoundsError, match=r"block_table\[0, 1\] = 9"):
        ops.paged_decode_attention(q, kc, vc, bad_bt, lens, 0.2)
    with pytest.raises(_debug.BoundsError, match="needs 3 blocks"):
        ops.paged_decode_attention(q, kc, vc, good_bt, torch.tensor([40, 5], dtype=torch.int32), 0.2)
    cu = torch.tensor([0, 1, 2], dtype=torch.int32)
    with pytest.raises(_debug.BoundsError):
        ops.paged_prefill_attention(q, kc, vc, bad_bt, cu, lens, 1, 0.2)
    with pytest.raises(_debug.BoundsError, match="cu_q"):
        ops.paged_prefill_attention(q, kc, vc, good_bt, torch.tensor([0, 1, 5], dtype=torch.int32), lens, 1, 0.2)
    # rotary + cache write: positions beyond the table, slots beyond the cache; -1 slots mean "skip"
    cs = ref.build_cos_sin_cache(32, 64, 1e4, None, "cpu")
    qkv = torch.randn(3, (4 + 2 * 2) * 32)
    pos = torch.tensor([0, 1, 2])
    ops.rope_kv_write(qkv, 4, 2, 32, pos, cs, 32, torch.tensor([5, -1, 63], dtype=torch.int32), kc, vc)
    with pytest.raises(_debug.BoundsError, match="slots"):
        ops.rope_kv_write(qkv, 4, 2, 32, pos, cs, 32, torch.tensor([5, 6, 64], dtype=torch.int32), kc, vc)
    with pytest.raises(_debug.BoundsError, match="positions"):
        ops.rope_kv_write(qkv, 4, 2, 32, torch.tensor([0, 1, 64]), cs, 32, torch.tensor([5, 6, 7], dtype=torch.int32), kc, vc)
    with pytest.raises(_debug.BoundsError, match="gather_rows"):
        ops.gather_rows(torch.randn(4, 8), torch.tensor([0, 4]))
    with pytest.raises(_debug.BoundsError, match="embedding"):
        ops.embedding(torch.tensor([3, -2]), torch.randn(10, 4))
