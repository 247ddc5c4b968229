"""Engine features on a GPU (bf16, CUDA kernels): speculative decoding, beam search, PD pair, host
tier, constrained decoding and the VLM path.  Exact-equality checks are made against runs that use
the same kernels; where two paths differ in kernels (one-pass verification uses the prefill kernel,
plain decoding the decode kernel) a small number of late divergences on near-tie logits is allowed."""
import numpy as np
import pytest
import torch

from xllm_b200 import LLM, SamplingParams

pytestmark = pytest.mark.gpu

KW = dict(devices="cuda:0", dtype="bfloat16", block_size=16, num_blocks=256, max_seqs_per_batch=8, max_tokens_per_batch=256)


def _prompts(seed=0):
    g = torch.Generator().manual_seed(seed)
    base = torch.randint(0, 32000, (12,), generator=g).tolist()
    return [base * 3, torch.randint(0, 32000, (40,), generator=g).tolist(), (base[:5] * 6)[:29]]


def _close(a, b, min_prefix=4):
    n = 0
    for x, y in zip(a, b):
        if x != y:
            break
        n += 1
    return n >= min(min_prefix, len(a))


def test_speculative_ngram_on_gpu():
    sp = SamplingParams(max_tokens=24, temperature=0.0, ignore_eos=True)
    plain = [o.outputs[0].token_ids for o in LLM("tiny", enable_schedule_overlap=False, **KW).generate(_prompts(), sp)]
    llm = LLM("tiny", enable_schedule_overlap=False, num_speculative_tokens=3, **KW)
    got = [o.outputs[0].token_ids for o in llm.generate(_prompts(), sp)]
    assert all(len(g) == 24 for g in got)
    assert all(_close(a, b) for a, b in zip(plain, got)), (plain, got)
    assert llm.engine.spec.steps > 0


def test_beam_search_width_one_is_greedy_on_gpu():
    llm = LLM("tiny", enable_prefix_cache=False, **KW)
    p = _prompts(1)[1]
    greedy = llm.generate([p], SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))[0].outputs[0].token_ids
    one = llm.beam_search([p], beam_width=1, max_tokens=8, ignore_eos=True)[0][0].token_ids
    assert _close(greedy, one, 6)
    wide = llm.beam_search([p], beam_width=4, max_tokens=8, ignore_eos=True)[0]
    assert len(wide) == 4 and wide[0].score >= wide[-1].score
    assert llm.engine.scheduler.block_manager(0).num_used_blocks == 0


def test_pd_pair_and_host_tier_on_gpu():
    from xllm_b200.engine.disagg import PDCoordinator, make_pd_pair
    kw = dict(device="cuda:0", dtype="bfloat16", block_size=16, num_blocks=128, max_seqs_per_batch=8,
              max_tokens_per_batch=128, enable_prefix_cache=False)
    prompts = _prompts(2)
    want = [o.outputs[0].token_ids for o in LLM("tiny", enable_prefix_cache=False, **KW).generate(
        prompts, SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True))]
    p, d = make_pd_pair("tiny", **kw)
    pd = PDCoordinator(p, d)
    for i, pr in enumerate(prompts):
        pd.add_request(f"r{i}", pr, max_tokens=10, temperature=0.0, ignore_eos=True)
    got = {f"r{i}": [] for i in range(len(prompts))}
    pd.run_until_done(lambda ev: got[ev.request_id].append(ev.token) if ev.token >= 0 else None)
    assert all(_close(w, got[f"r{i}"], 6) for i, w in enumerate(want)), (want, got)
    # host tier
    llm = LLM("tiny", devices="cuda:0", dtype="bfloat16", block_size=16, num_blocks=14, max_seqs_per_batch=2,
              max_tokens_per_batch=128, enable_prefix_cache=True, host_kv_blocks=64)
    g = torch.Generator().manual_seed(2)
    a = torch.randint(0, 32000, (100,), generator=g).tolist()
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    first = llm.generate([a], sp)[0].outputs[0].token_ids
    for _ in range(3):
        llm.generate([torch.randint(0, 32000, (120,), generator=g).tolist()], sp)
    again = llm.generate([a], sp)[0].outputs[0].token_ids
    assert again == first and llm.engine.host_tier.stats()["loaded"] >= 6


def test_vlm_on_gpu_matches_cpu_tokens():
    from test_vlm_cpu import IMG, VEND, VSTART, _args
    from xllm_b200.api.vlm import VLM
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
    from xllm_b200.multimodal import Qwen2VLImageProcessor
    rng = np.random.default_rng(1)
    img = (rng.random((80, 100, 3)) * 255).astype(np.uint8)
    reqs = [dict(prompt_token_ids=[11, 12, VSTART, IMG, VEND, 13, 14, 15], images=[img])]
    outs = {}
    for dev, dt in (("cpu", "float32"), ("cuda:0", "bfloat16")):
        vlm = VLM.__new__(VLM)
        vlm.engine = LLMEngine(EngineConfig(model="v", device=dev, dtype=dt, num_blocks=64, enable_graph=False,
                                            max_tokens_per_batch=16, enable_schedule_overlap=False),
                               model_args=_args(head_dim=64, hidden=256, sections=(8, 12, 12)))
        vlm.tokenizer = None
        if dev == "cpu":
            vlm.engine.model.init_random(std=0.05, seed=3)
            cpu_params = dict(vlm.engine.model.named_params())
        else:   # the same weights on the GPU (random generators differ between devices)
            vlm.engine.model.copy_params_from(cpu_params)
        vlm.processor = Qwen2VLImageProcessor(14, 2, 2, min_pixels=56 * 56, max_pixels=112 * 112)
        vlm.image_token_id = IMG
        outs[dev] = vlm.generate_mm(reqs, SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True))[0]
    assert len(outs["cuda:0"]) == 5 and outs["cuda:0"][:2] == outs["cpu"][:2], outs


def test_vmm_pool_maps_device_memory_and_keeps_addresses():
    """The page pool on the real driver: map on demand, compute on the mapped tensor, give the pages
    back, map again at the same address, let a second range reuse the pages."""
    from xllm_b200.utils.xtensor import VmmPool
    pool = VmmPool(device=0, page_bytes=2 << 20, max_pages=8)
    assert not pool.fake and pool.p.driver == "cuda"
    pb = pool.page_bytes
    r = pool.range(8 * pb)
    r.ensure(3 * pb)
    t = r.tensor((3 * pb // 2,), torch.bfloat16)
    assert t.is_cuda and t.data_ptr() == r.ptr
    t.fill_(1.0)
    assert float(t.float().sum()) == t.numel()
    y = torch.ones(4, 8, device="cuda", dtype=torch.bfloat16) @ r.tensor((8, 16), torch.bfloat16)
    assert float(y.float().sum()) == 4 * 8 * 16
    torch.cuda.synchronize()
    addr = r.ptr
    r.release_all()
    assert pool.pages_in_use == 0 and pool.pages_free == 3
    other = pool.range(4 * pb)
    other.ensure(2 * pb)                                # reuses two of the pages
    assert pool.pages_created == 3
    r.ensure(pb)
    assert r.ptr == addr and pool.pages_in_use == 3
    r.tensor((16,), torch.float32).zero_()
    torch.cuda.synchronize()
    other.release_all()
    r.release_all()
    assert pool.trim() == 3


def test_mla_latent_cache_on_gpu_matches_materialised_form():
    from test_deepseek_cpu import _args
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
    args = _args()

    def make(**kw):
        llm = LLM.__new__(LLM)
        llm.engine = LLMEngine(EngineConfig(model="d", device="cuda:0", dtype="bfloat16", num_blocks=128, enable_graph=False,
                                            max_tokens_per_batch=64, **kw), model_args=args)
        llm.tokenizer = None
        return llm

    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (12, 70, 33)]
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    a, b = make(), make(mla_latent_cache=True)
    for (_, t), (_, u) in zip(a.engine.model.named_params(), b.engine.model.named_params()):
        u.copy_(t)
    want = [o.outputs[0].token_ids for o in a.generate(prompts, sp)]
    got = [o.outputs[0].token_ids for o in b.generate(prompts, sp)]
    assert [w[:2] for w in want] == [x[:2] for x in got], (want, got)      # bf16: later near ties may differ
    assert b.engine.runner.kv_caches[0][0].shape[1] == 1


def test_qwen3_next_hybrid_on_gpu_matches_cpu_tokens():
    """Linear-attention state slots, gated attention and the MoE on the GPU against the CPU engine
    with the same weights (bf16 against fp32: the first tokens must agree)."""
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
    from xllm_b200.models import ModelArgs
    args = ModelArgs(model_type="qwen3_next", vocab_size=1000, hidden_size=256, num_hidden_layers=4, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=64, intermediate_size=512, qk_norm=True, partial_rotary_factor=0.25,
                     rope_theta=10000.0, max_position_embeddings=512, tie_word_embeddings=False,   # dense MLPs: no routing ties
                     extra=dict(linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=32,
                                linear_value_head_dim=32, linear_conv_kernel_dim=4, full_attention_interval=4))
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (9, 50, 21)]
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    from xllm_b200.api.embedding import hidden_states
    outs, params, logits = {}, None, {}
    for dev, dt in (("cpu", "float32"), ("cuda:0", "bfloat16")):
        llm = LLM.__new__(LLM)
        llm.engine = LLMEngine(EngineConfig(model="n", device=dev, dtype=dt, num_blocks=64, enable_graph=False,
                                            max_tokens_per_batch=32), model_args=args)
        llm.tokenizer = None
        if params is None:
            llm.engine.model.init_random(std=0.05, seed=5)
            params = dict(llm.engine.model.named_params())
        else:
            llm.engine.model.copy_params_from(params)
        outs[dev] = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
        # teacher-forced logits over prompt + the CPU continuation, one pass
        logits[dev] = [llm.engine.model.logits(hidden_states(llm.engine, p + c)).float().cpu()
                       for p, c in zip(prompts, outs["cpu"])]
    # bf16 against fp32 on nearly flat logits: first tokens agree, logits agree closely over whole sequences
    assert [o[:1] for o in outs["cuda:0"]] == [o[:1] for o in outs["cpu"]], outs
    for a, b in zip(logits["cpu"], logits["cuda:0"]):
        assert float((a - b).abs().mean() / a.std()) < 0.08
    # and on the GPU itself the decode path (state kernel, paged decode attention) must reproduce what
    # the one-pass prefill predicts at the same positions
    hit = tot = 0
    for p, c, lg in zip(prompts, outs["cuda:0"], logits["cuda:0"]):
        if c == outs["cpu"][prompts.index(p)]:
            pred = lg[len(p) - 1: len(p) - 1 + len(c)].argmax(-1).tolist()
            hit += sum(int(x == y) for x, y in zip(pred, c))
            tot += len(c)
    assert tot >= 10 and hit >= 0.8 * tot, (hit, tot, outs)


def test_flux_transformer_on_device_matches_cpu():
    """The Flux-family transformer in bf16 on the GPU (linears on the tcgen05 GEMM) against the same weights in
    fp32 on the CPU."""
    from xllm_b200.dit.flux import FluxArgs, FluxTransformer, image_ids, pack_latents
    from xllm_b200.ops import launches
    args = FluxArgs(in_channels=16, num_layers=2, num_single_layers=2, attention_head_dim=32, num_attention_heads=4,
                    joint_attention_dim=64, pooled_projection_dim=32, axes_dims_rope=(8, 12, 12))
    cpu = FluxTransformer(args)
    cpu.init_random(std=0.05, seed=1)
    gpu = FluxTransformer(args, dtype=torch.bfloat16, device="cuda")
    gpu.load_weights(cpu.p.items())
    g = torch.Generator().manual_seed(0)
    lat = pack_latents(torch.randn(2, 4, 16, 16, generator=g))
    text, pooled, t = torch.randn(2, 12, 64, generator=g), torch.randn(2, 32, generator=g), torch.tensor([0.8, 0.3])
    gd = torch.tensor([3.5, 3.5])
    want = cpu.forward(lat, text, pooled, t, image_ids(16, 16), torch.zeros(12, 3), gd)
    n0 = launches()
    got = gpu.forward(lat.cuda(), text.cuda(), pooled.cuda(), t.cuda(), image_ids(16, 16, "cuda"), torch.zeros(12, 3, device="cuda"),
                      gd.cuda())
    assert launches() > n0                                    # the hand-written GEMM ran
    err = (got.float().cpu() - want).abs().max().item()
    assert err < 0.05 * max(1.0, want.abs().max().item()), err
