"""gloo worker: Ulysses attention, CFG parallel and encoder DP against their single-process forms."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from xllm_b200.parallel import dit_parallel as dp  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    cfg_size = int(os.environ.get("CFG_SIZE", "1"))
    st = dp.init_dit_parallel(cfg_size)
    g = torch.Generator().manual_seed(0)
    B, H, T, D = 2, 8, 32, 16
    q, k, v = (torch.randn(B, H, T, D, generator=g) for _ in range(3))
    want = torch.nn.functional.scaled_dot_product_attention(q, k, v)
    # every CFG branch shards the same sequence over its sp group
    sh = lambda t: dp.shard_sequence(t, st, dim=2)
    got = dp.ulysses_attention(sh(q), sh(k), sh(v), st)
    assert torch.allclose(got, sh(want), atol=1e-5), "ulysses shard differs"
    full = dp.gather_sequence(got, st, dim=2)
    assert torch.allclose(full, want, atol=1e-5)
    # CFG: branch 0 = cond, branch 1 = uncond
    cond, uncond = torch.randn(3, 5, generator=g), torch.randn(3, 5, generator=g)
    mine = cond if st.cfg_rank == 0 else uncond
    out = dp.cfg_combine(mine, st, 4.0)
    if cfg_size == 2:
        assert torch.allclose(out, uncond + 4.0 * (cond - uncond), atol=1e-6)
    else:
        assert torch.equal(out, mine)
    # encoder DP: 7 "images" of different sizes
    items = [torch.randn(n, 6, generator=g) for n in (3, 9, 1, 4, 4, 7, 2)]
    enc = lambda xs: [x * 2 + 1 for x in xs]
    res = dp.encoder_dp(items, enc, dist.group.WORLD, rank, world)
    assert all(torch.equal(r, x * 2 + 1) for r, x in zip(res, items))
    # the compact DiT: sequence-parallel blocks and CFG-parallel guidance reproduce one process
    from xllm_b200.dit.model import TinyDiT
    torch.manual_seed(5)
    model = TinyDiT(size=8, heads=4).eval()
    noise = torch.randn(2, 4, 8, 8, generator=g)
    cond = torch.randn(2, model.dim, generator=g)
    want_img = model.sample(noise, steps=4, cond=cond, guidance_scale=3.0)
    got_img = model.sample(noise, steps=4, cond=cond, guidance_scale=3.0, st=st)
    assert torch.allclose(got_img, want_img, atol=1e-4), float((got_img - want_img).abs().max())
    assert dp.sp_group_ranks(8, 2) == [[0, 1, 2, 3], [4, 5, 6, 7]] and dp.cfg_group_ranks(8, 2)[1] == [1, 5]
    dist.barrier()
    if rank == 0:
        print("DIT_PARALLEL_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
