"""Worker for test_tp_gpu.py: fused all-reduce(+residual+RMSNorm) against torch.distributed."""
import torch
import torch.distributed as dist

from xllm_b200.ops import reference as ref
from xllm_b200.parallel import symm
from xllm_b200.parallel.state import init_parallel


def main():
    ps = init_parallel()
    H = 4096
    comm = symm.attach(ps, 4096, H)
    assert comm is not None
    torch.manual_seed(1234)  # same stream on every rank
    for T in (1, 7, 256, 1000, 4096):
        parts = [torch.randn(T, H, device=ps.device, dtype=torch.bfloat16) for _ in range(ps.world_size)]
        res_full = torch.randn(T, H, device=ps.device, dtype=torch.bfloat16)
        w = (torch.randn(H, device=ps.device) * 0.1 + 1).to(torch.bfloat16)
        total = sum(p.float() for p in parts)
        # plain sum
        comm.partial_buffer(T).copy_(parts[ps.rank])
        got = comm.allreduce(T).clone()
        assert torch.allclose(got.float(), total, atol=0.06, rtol=0.02), (T, (got.float() - total).abs().max())
        # sum + residual + norm (twice in a row on the same buffers)
        b, e, S = comm.shard(T)
        shard = torch.zeros(S, H, device=ps.device, dtype=torch.bfloat16)
        shard[: e - b] = res_full[b:e]
        for _ in range(2):
            comm.partial_buffer(T).copy_(parts[ps.rank])
            want_res = (total + res_full.float()).to(torch.bfloat16)
            want, _ = ref.rmsnorm(want_res, w, 1e-6)
            got = comm.allreduce_norm(T, shard, w, 1e-6).clone()
            assert torch.allclose(shard[: e - b].float(), want_res[b:e].float(), atol=0.07, rtol=0.02)
            assert torch.allclose(got.float(), want.float(), atol=0.08, rtol=0.03), (T, (got.float() - want.float()).abs().max())
            res_full = want_res
        assert comm.error_status() == 0
    # inside a CUDA graph
    T = 64
    part = torch.randn(T, H, device=ps.device, dtype=torch.bfloat16)
    comm.partial_buffer(T).copy_(part)
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        comm.allreduce(T)
    torch.cuda.current_stream().wait_stream(s)
    with torch.cuda.graph(g):
        y = comm.allreduce(T)
    for _ in range(3):
        comm.partial_buffer(T).copy_(part)
        g.replay()
    torch.cuda.synchronize()
    tot = part.float().clone()
    dist.all_reduce(tot)
    assert torch.allclose(y.float(), tot, atol=0.06, rtol=0.02)
    assert comm.error_status() == 0
    return "ALLREDUCE_NORM_OK multimem=%d world=%d" % (int(comm.mc_base != 0), ps.world_size)


if __name__ == "__main__":
    from mp_common import guarded
    guarded(main)
