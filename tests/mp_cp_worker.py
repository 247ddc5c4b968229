"""Worker for test_context_parallel_cpu.py (gloo ranks)."""
import os

import torch
import torch.distributed as dist

from xllm_b200.parallel import context_parallel as cp


def main():
    dist.init_process_group("gloo", init_method=os.environ["INIT"], rank=int(os.environ["RANK"]),
                            world_size=int(os.environ["WORLD_SIZE"]))
    r, W = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)                       # the same full problem on every rank
    T, H, Hkv, D = 203, 4, 2, 16
    q, k, v = torch.randn(T, H, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    scale = D ** -0.5
    full, _ = cp.attention_with_lse(q, k, v, scale)
    # ---- CP prefill: zig-zag shards, KV all-gather
    shards = cp.zigzag_shards(T, W)
    mine = shards[r]
    o_local = cp.cp_prefill_attention(q[mine], k[mine], v[mine], mine, scale, dist.group.WORLD)
    assert torch.allclose(o_local, full[mine], atol=1e-5), (o_local - full[mine]).abs().max()
    parts = [torch.empty(len(s), H, D) for s in shards]
    for i in range(W):
        buf = o_local.contiguous() if i == r else parts[i]
        dist.broadcast(buf, src=i)
        parts[i] = buf
    assert torch.allclose(cp.restore_order(parts, shards), full, atol=1e-5)
    # ---- DCP decode: the last token attends to KV striped over the ranks
    kpos = torch.arange(T)[r::W]
    o = cp.dcp_decode_attention(q[-1:], k[kpos], v[kpos], kpos, scale, dist.group.WORLD)
    assert torch.allclose(o, full[-1:], atol=1e-5)
    print(f"CP_OK {r}", flush=True)
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
