"""Worker for test_tp_gpu.py: the one-shot fused all-reduce (+residual +RMSNorm), the vocabulary-sharded
arg-max and the logits gather, against torch.distributed; eager and replayed from a CUDA graph."""
import os

import torch
import torch.distributed as dist

from xllm_b200 import ops
from xllm_b200.ops import reference as ref
from xllm_b200.parallel import symm
from xllm_b200.parallel.state import init_parallel


def main():
    ps = init_parallel(timeout_s=120)
    H = int(os.environ.get("HIDDEN", "4096"))
    Vs = 4096 + 64
    comm = symm.attach(ps, 4096, H, vocab_shard=Vs, max_sample_rows=256)
    assert comm is not None
    dev, W, r = ps.device, ps.world_size, ps.rank
    torch.manual_seed(1234)  # same stream on every rank
    for T in (1, 7, 256, 768, 2048):
        assert comm.begin_forward(T), "these sizes take the one-shot form"
        parts = [torch.randn(T, H, device=dev, dtype=torch.bfloat16) for _ in range(W)]
        res = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
        w = (torch.randn(H, device=dev) * 0.1 + 1).to(torch.bfloat16)
        total = sum(p.float() for p in parts)
        comm.partial_buffer(T).copy_(parts[r])
        got = comm.allreduce(T)
        assert torch.allclose(got.float(), total, atol=0.06, rtol=0.02), (T, (got.float() - total).abs().max())
        # sum + residual + norm, several calls in a row: the partial buffers alternate
        residual = res.clone()
        for it in range(3):
            comm.partial_buffer(T).copy_(parts[r])
            want_res = (total + (res if it == 0 else prev).float()).to(torch.bfloat16)
            want, _ = ref.rmsnorm(want_res, w, 1e-6)
            got = comm.allreduce_norm(T, residual, w, 1e-6)
            assert torch.allclose(residual.float(), want_res.float(), atol=0.07, rtol=0.02), (T, it)
            assert torch.allclose(got.float(), want.float(), atol=0.08, rtol=0.03), (T, it, (got.float() - want.float()).abs().max())
            prev = want_res
        comm.end_forward()
        assert comm.error_status() == 0, T

    # vocabulary-sharded arg-max: rank k holds columns [k * Vs, (k + 1) * Vs)
    B = 200
    full = torch.randn(B, W * Vs, device=dev, dtype=torch.bfloat16)
    full[3, 5] = full[3, W * Vs - 2] = 50.0          # a tie across ranks: the lowest index wins
    local = full[:, r * Vs:(r + 1) * Vs].contiguous()
    for _ in range(3):                                 # consecutive calls alternate the pair slots
        ids = comm.argmax(local, Vs, r * Vs)
    want_ids = full.float().argmax(-1)
    want_ids[3] = 5
    assert torch.equal(ids, want_ids), (ids[:8], want_ids[:8])
    # gather of the shards into full rows
    g = comm.gather_logits(local)
    assert g is not None and torch.equal(g[:, : W * Vs], full)
    assert comm.error_status() == 0

    # the same kernels replayed from a CUDA graph (epochs advance on the device)
    T = 64
    part = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    residual = torch.zeros(T, H, device=dev, dtype=torch.bfloat16)
    w = torch.ones(H, device=dev, dtype=torch.bfloat16)

    def step():
        comm.begin_forward(T)
        comm.partial_buffer(T).copy_(part)
        a = comm.allreduce(T)
        comm.partial_buffer(T).copy_(part)
        b = comm.allreduce_norm(T, residual, w, 1e-6)
        comm.end_forward()
        return a, b, comm.argmax(local, Vs, r * Vs)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        step()
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        a, b, ids2 = step()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    tot = part.float().clone()
    dist.all_reduce(tot)
    assert torch.allclose(a.float(), tot, atol=0.06, rtol=0.02)
    assert torch.equal(ids2, want_ids)
    assert comm.error_status() == 0

    # device time per call, max over ranks (CUDA events, back-to-back calls inside one graph so that
    # launch gaps do not count)
    def timeit(fn, n=20):
        gph = torch.cuda.CUDAGraph()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            fn()
        torch.cuda.current_stream().wait_stream(s)
        with torch.cuda.graph(gph):
            for _ in range(n):
                fn()
        gph.replay()
        ts = []
        for _ in range(5):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            gph.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / n)
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e3

    rows = []
    for T in (16, 256, 768, 2048):
        residual = torch.zeros(T, H, device=dev, dtype=torch.bfloat16)
        y = torch.randn(T, H, device=dev, dtype=torch.bfloat16)

        def one():
            comm.begin_forward(T)
            comm.allreduce_norm(T, residual, w, 1e-6)
            comm.allreduce_norm(T, residual, w, 1e-6)
            comm.end_forward()

        def two():
            comm.oneshot = False
            b0, e0, S = comm.shard(T)
            comm.allreduce_norm(T, residual[:S], w, 1e-6)
            comm.allreduce_norm(T, residual[:S], w, 1e-6)

        def lib():
            dist.all_reduce(y)
            ops.rmsnorm(y, w, 1e-6, residual=residual)
            dist.all_reduce(y)
            ops.rmsnorm(y, w, 1e-6, residual=residual)

        rows.append((T, timeit(one) / 2, timeit(two) / 2, timeit(lib) / 2))
    ta = timeit(lambda: comm.argmax(local, Vs, r * Vs))
    assert comm.error_status() == 0
    table = "; ".join(f"T={T}: one-shot {a:.1f} us, two-shot {b:.1f} us, NCCL+norm {c:.1f} us" for T, a, b, c in rows)
    return (f"ONESHOT_OK world={W} H={H} multimem={int(comm.mc_base != 0)} per all-reduce+norm: {table}; "
            f"arg-max over shards ({B} rows) {ta:.1f} us")


if __name__ == "__main__":
    from mp_common import guarded
    guarded(main)
