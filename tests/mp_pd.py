"""torchrun worker, 2 GPUs: rank 0 is a prefill instance, rank 1 a decode instance.  Each owns an
engine with its KV cache in peer-mapped memory; the prompt's KV is pushed layer by layer during
the prefill forward, the control messages go over a socket.  The tokens must equal those of one
engine; then the push kernel is timed against one peer copy per block."""
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from xllm_b200.api.llm import LLM, SamplingParams  # noqa: E402
from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine  # noqa: E402
from xllm_b200.engine.model_runner import ModelRunner  # noqa: E402
from xllm_b200.engine.pd_service import Channel, DecodeService, PDLink, PeerPush, PrefillService  # noqa: E402
from xllm_b200.models import ModelArgs, create_model  # noqa: E402
from xllm_b200.parallel.state import init_parallel, single  # noqa: E402

NUM_BLOCKS = 4096


def main():
    ps = init_parallel(instances=2)
    assert ps.world_size == 1 and ps.n_instances == 2
    role = "prefill" if ps.instance == 0 else "decode"
    dev = ps.device
    args = ModelArgs(model_type="qwen3", vocab_size=32000, hidden_size=1024, num_hidden_layers=3,
                     num_attention_heads=8, num_key_value_heads=2, head_dim=128, intermediate_size=3072,
                     tie_word_embeddings=False, max_position_embeddings=4096)
    model = create_model(args, torch.bfloat16, dev, single())
    model.init_random(seed=7)                      # the same weights in both processes
    kv_bytes = ModelRunner.kv_bytes_per_block(args, 2, 16, torch.bfloat16) * NUM_BLOCKS
    link = PDLink(ps.job_group, dev, kv_bytes)
    cfg = EngineConfig(model="t", device=str(dev), dtype="bfloat16", block_size=16, num_blocks=NUM_BLOCKS,
                       max_seqs_per_batch=8, max_tokens_per_batch=256, max_model_len=1024, enable_graph=True,
                       enable_prefix_cache=False)
    port = int(os.environ.get("MASTER_PORT", "29571")) + 17
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 32000, (int(n),), generator=g).tolist() for n in (40, 300, 9, 77, 512)]
    msg = ""
    phase1_error = None
    try:
        if role == "prefill":
            srv = Channel.listen("127.0.0.1", port)
            base = LLM.__new__(LLM)
            base.engine = LLMEngine(cfg, ps=single(), model=model, model_args=args)
            base.tokenizer = None
            want = [o.outputs[0].token_ids for o in base.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0,
                                                                                            ignore_eos=True))]
            eng = LLMEngine(cfg, ps=single(), model=model, model_args=args, hold_finished_blocks=True,
                            kv_allocator=link.allocator())
            assert eng.runner.kv_tensor.data_ptr() == link.buf.data_ptr()
            ch = Channel.accept(srv, 120.0)
            svc = PrefillService(eng, ch, PeerPush(link, eng.runner, peer_rank=1))
            for i, pr in enumerate(prompts):
                assert svc.add_request(f"r{i}", pr, max_tokens=12, temperature=0.0, ignore_eos=True)
            got = {f"r{i}": [] for i in range(len(prompts))}

            def on(ev):
                if ev.token >= 0:
                    got[ev.request_id].append(int(ev.token))

            assert svc.run_until_done(on, max_seconds=120.0)
            svc.close()
            res = [got[f"r{i}"] for i in range(len(prompts))]
            # chunked prefill (256-token budget) pushed 300- and 512-token prompts over several steps
            assert res == want, (want, res)
            assert not svc.failed and svc.handed_over == len(prompts)
            assert eng.scheduler.block_stats(0).num_used == 0
            msg = f"tokens equal, {svc.t.pushed_bytes >> 10} KiB pushed in {svc.epoch} steps"
        else:
            eng = LLMEngine(cfg, ps=single(), model=model, model_args=args, kv_allocator=link.allocator())
            ch = Channel.connect("127.0.0.1", port, 120.0)
            svc = DecodeService(eng, ch, PeerPush(link, eng.runner, peer_rank=0))
            assert svc.serve(120.0)
            assert svc.adopted == len(prompts) and svc.failed_waits == 0
            assert eng.scheduler.block_stats(0).num_used == 0 and eng.scheduler.num_reserved() == 0
    except BaseException as e:  # noqa: BLE001 - both ranks must reach the collectives below
        phase1_error = e
    torch.cuda.synchronize()
    dist.barrier()

    # ---- push bandwidth: 2048 blocks of 32 KiB per plane (K and V: 128 MiB), block ids shuffled
    from xllm_b200.engine.kv_transfer import KVPusher, PushTarget
    nb, heads, page, d = 2048, 8, 16, 128
    plane = nb * heads * page * d * 2
    assert 2 * plane <= link.kv_bytes
    k = link.buf[:plane].view(torch.bfloat16).view(nb, heads, page, d)
    v = link.buf[plane:2 * plane].view(torch.bfloat16).view(nb, heads, page, d)
    if role == "prefill":
        k.copy_(torch.randn(nb, heads, page, d, device=dev).to(torch.bfloat16))
        v.copy_(torch.randn(nb, heads, page, d, device=dev).to(torch.bfloat16))
    else:
        k.zero_()
        v.zero_()
    torch.cuda.synchronize()
    dist.barrier()
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(1))
    bw = {}
    if role == "prefill":
        pairs = torch.stack([torch.arange(nb), perm], 1).to(torch.int32).to(dev)
        pusher = KVPusher([(k, v)], 16, dev)
        base_ptr = link.peer_base(1)
        target = PushTarget([(base_ptr, base_ptr + plane)], pusher.block_bytes, base_ptr + link.kv_bytes)
        peer_k = link.hdl.get_buffer(1, (nb, heads, page, d), torch.bfloat16, 0)
        peer_v = link.hdl.get_buffer(1, (nb, heads, page, d), torch.bfloat16, plane // 2)
        pl = perm.tolist()

        def timed(fn, reps=5):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps

        def per_block():
            for s, t in enumerate(pl):
                peer_k[t].copy_(k[s], non_blocking=True)
                peer_v[t].copy_(v[s], non_blocking=True)

        ms_push = timed(lambda: pusher.push_layer(0, pairs, target, 1000))
        ms_copy = timed(per_block, reps=2)
        ms_big = timed(lambda: (peer_k.copy_(k, non_blocking=True), peer_v.copy_(v, non_blocking=True)))
        gb = 2 * plane / 1e9
        bw = dict(push_gbs=gb / ms_push * 1e3, per_block_copy_gbs=gb / ms_copy * 1e3, one_copy_gbs=gb / ms_big * 1e3)
        pusher.push_layer(0, pairs, target, 1001)       # leave the shuffled image for the check below
    torch.cuda.synchronize()
    dist.barrier()
    if role == "decode":
        # what arrived is the prefill side's data at the shuffled block ids: check through a checksum
        # exchanged over the process group
        sums = (k.float().sum((1, 2, 3)), v.float().sum((1, 2, 3)))
    else:
        sums = (k.float().sum((1, 2, 3))[torch.argsort(perm.to(dev))], v.float().sum((1, 2, 3))[torch.argsort(perm.to(dev))])
    both = [torch.empty_like(sums[0]) for _ in range(2)]
    dist.all_gather(both, sums[0])
    assert torch.equal(both[0], both[1]), "pushed K blocks differ"
    dist.all_gather(both, sums[1])
    assert torch.equal(both[0], both[1]), "pushed V blocks differ"
    if phase1_error is not None:
        raise phase1_error
    if role == "prefill":
        msg += " | push %.0f GB/s, one copy per block %.0f GB/s, one big copy %.0f GB/s" % (
            bw["push_gbs"], bw["per_block_copy_gbs"], bw["one_copy_gbs"])
    return "PD_OK " + msg


if __name__ == "__main__":
    from mp_common import guarded
    guarded(main)
