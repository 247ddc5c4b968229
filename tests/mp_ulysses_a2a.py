"""torchrun worker (2+ GPUs): the peer-memory Ulysses all-to-all against the process-group form, and
Ulysses attention over it against single-GPU attention."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from xllm_b200.parallel import dit_parallel as dp  # noqa: E402
from xllm_b200.parallel.state import init_parallel  # noqa: E402


def main():
    ps = init_parallel()
    n, rank, dev = ps.world_size, ps.rank, ps.device
    st = dp.init_dit_parallel(1, rank, n)
    a2a = dp.AllToAll(st.sp_group, rank, n, dev, max_bytes=64 << 20)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    for shape, (sd, gd) in (((2, 8 * n, 96, 128), (1, 2)), ((2, 4, 64 * n, 128), (2, 1)), ((1, 2 * n, 3, 64), (1, 2)),
                            ((3, 5, 7 * n, 8), (2, 1))):
        for _ in range(3):                                   # consecutive calls alternate the receive halves
            x = torch.randn(shape, device=dev, generator=g).to(torch.bfloat16)
            want = dp.all_to_all(x, st.sp_group, sd, gd, None)
            got = a2a(x, sd, gd)
            assert got.shape == want.shape and torch.equal(got, want), (shape, sd, gd)
    assert a2a.error_status() == 0
    # attention through it
    st.a2a = a2a
    g2 = torch.Generator(device=dev).manual_seed(7)           # the same full tensors on every rank
    B, H, T, D = 2, 4 * n, 64 * n, 128
    q, k, v = (torch.randn(B, H, T, D, device=dev, generator=g2).to(torch.bfloat16) for _ in range(3))
    want = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float())
    sh = lambda t: dp.shard_sequence(t, st, dim=2)
    got = dp.ulysses_attention(sh(q), sh(k), sh(v), st)
    assert torch.allclose(got.float(), sh(want), atol=3e-2, rtol=3e-2)
    # timing: peer-memory form against NCCL all_to_all + cat, q-sized tensor of a 4096-token, 24-head, 128-dim step
    x = torch.randn(1, 24 if 24 % n == 0 else 8 * n, 4096 // n, 128, device=dev, generator=g).to(torch.bfloat16)

    def timed(fn, reps=20):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    us_peer = timed(lambda: a2a(x, 1, 2))
    us_nccl = timed(lambda: dp.all_to_all(x, st.sp_group, 1, 2, None))
    return f"ULYSSES_A2A_OK world={n} {tuple(x.shape)} bf16: peer-memory kernel {us_peer:.1f} us, NCCL all_to_all + cat {us_nccl:.1f} us"


if __name__ == "__main__":
    from mp_common import guarded
    guarded(main)
