"""Worker for test_collectives_cpu.py: the process-group helpers of ParallelState on gloo ranks."""
import torch
import torch.distributed as dist

from xllm_b200.parallel.state import init_parallel


def main():
    ps = init_parallel()
    r, n = ps.rank, ps.world_size
    # equal all-to-all: slice i of rank r goes to rank i
    x = torch.arange(n * 2 * 3, dtype=torch.float32).view(n * 2, 3) + 1000 * r
    y = ps.all_to_all_single(x)
    want = torch.cat([(torch.arange(n * 2 * 3, dtype=torch.float32).view(n * 2, 3) + 1000 * p)[2 * r: 2 * r + 2] for p in range(n)])
    assert torch.equal(y, want), (r, y, want)
    # ragged: rank r sends (p + 1) rows to peer p and so receives (r + 1) rows from everyone
    rows = sum(p + 1 for p in range(n))
    z = torch.full((rows, 2), float(r))
    out = ps.all_to_all_single(z, in_splits=[p + 1 for p in range(n)])
    assert out.shape[0] == n * (r + 1)
    assert torch.equal(out, torch.cat([torch.full((r + 1, 2), float(p)) for p in range(n)]))
    # point to point ring, in waves of at most 64 bytes
    nxt, prv = (r + 1) % n, (r - 1) % n
    payload = [torch.full((8,), float(r * 10 + i)) for i in range(5)]            # 5 x 32 bytes -> 3 waves
    inbox = [torch.empty(8) for _ in range(5)]
    ps.batch_send_recv([(t, nxt) for t in payload], [(t, prv) for t in inbox], max_wave_bytes=64)
    assert all(torch.equal(t, torch.full((8,), float(prv * 10 + i))) for i, t in enumerate(inbox))
    b = torch.full((4,), float(r))
    ps.broadcast(b, src=n - 1)
    assert torch.equal(b, torch.full((4,), float(n - 1)))
    g = ps.all_gather(torch.tensor([[float(r)]]), dim=0, group=ps.world_group)
    assert g.view(-1).tolist() == [float(p) for p in range(n)]
    ps.barrier()
    if r == 0:
        print("COLLECTIVES_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
