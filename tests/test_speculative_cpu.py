"""Speculative decoding (n-gram drafter + one-pass verification) on the tiny CPU model: the token
stream must be identical to plain greedy decoding, and repetitive text must be accepted in bulk."""
import numpy as np
import pytest
import torch

from xllm_b200 import LLM, SamplingParams
from xllm_b200.engine.speculative import NgramDrafter


def _llm(**kw):
    return LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=128, max_seqs_per_batch=8,
               max_tokens_per_batch=256, enable_graph=False, enable_schedule_overlap=False, **kw)


def test_ngram_drafter_finds_latest_match():
    d = NgramDrafter(3, max_ngram=3)
    toks = np.array([5, 6, 7, 8, 9, 1, 2, 6, 7, 3, 4, 6, 7], dtype=np.int32)
    assert d.propose_one(toks).tolist() == [3, 4, 6]       # latest "6 7" is followed by 3 4 6
    assert d.propose_one(np.array([1, 2, 3], dtype=np.int32)).tolist() == [3, 3, 3]  # no match: repeat


def test_speculative_greedy_equals_plain_greedy():
    g = torch.Generator().manual_seed(3)
    base = torch.randint(0, 32000, (12,), generator=g).tolist()
    prompts = [base * 3, torch.randint(0, 32000, (40,), generator=g).tolist(), (base[:5] * 6)[:29]]
    sp = SamplingParams(max_tokens=24, temperature=0.0, ignore_eos=True)
    plain = [o.outputs[0].token_ids for o in _llm().generate(prompts, sp)]
    for k in (1, 3):
        llm = _llm(num_speculative_tokens=k)
        outs = llm.generate(prompts, sp)
        assert [o.outputs[0].token_ids for o in outs] == plain
        assert all(len(o.outputs[0].token_ids) == 24 for o in outs)
        assert llm.engine.spec.steps > 0


def test_speculative_accepts_repetition_and_stops_mid_row():
    # a model-free check of the multi-token bookkeeping: a stop token inside an accepted run ends
    # the sequence there and drops the rest of the run
    llm = _llm(num_speculative_tokens=3)
    eng = llm.engine
    prompt = list(range(100, 120))
    eng.add_request("r", prompt, temperature=0.0, max_tokens=50, stop_token_ids=[777], eos_token_id=-1)
    got = []
    while eng.has_unfinished():
        batches = eng.scheduler.schedule()
        if not batches:
            break
        b = batches[0]
        if b.n_prefill > 0:
            evs = eng._finish(eng.runner.execute(b))
        else:
            evs = eng.scheduler.process_output_multi(b.batch_id, np.array([1, 2, 777, 4], dtype=np.int64),
                                                     np.array([4], dtype=np.int32))
        got += [e.token for e in evs if e.token >= 0]
    assert got[1:] == [1, 2, 777] and len(got) == 4


def test_mtp_drafter_on_deepseek_matches_plain_greedy():
    """DeepSeek-style model + its MTP layer as the drafter (own paged KV cache, hidden states of the
    verified rows): the token stream must not depend on whether drafts are accepted."""
    from test_deepseek_cpu import _args
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine

    def make(**kw):
        llm = LLM.__new__(LLM)
        llm.engine = LLMEngine(EngineConfig(model="d", device="cpu", dtype="float32", num_blocks=96, enable_graph=False,
                                            max_tokens_per_batch=24, enable_schedule_overlap=False, **kw), model_args=_args())
        llm.tokenizer = None
        return llm

    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (9, 40, 17)]   # 40 > 24: chunked prefill
    sp = SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True)
    plain = [o.outputs[0].token_ids for o in make().generate(prompts, sp)]
    llm = make(num_speculative_tokens=1, speculative_method="mtp")
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == plain
    spec = llm.engine.spec
    assert spec.steps > 0 and spec.proposed > 0
    assert len(spec.drafter.draft) > 0
    # a drafter that already knows the answer gets everything accepted, so two tokens per step
    llm2 = make(num_speculative_tokens=1, speculative_method="mtp")
    truth = {tuple(p): t for p, t in zip(prompts, plain)}

    class Oracle:
        k = 1
        def propose(self, batch, n, **_):
            out = np.zeros((n, 1), dtype=np.int64)
            for i in range(n):
                h = batch.history(i, 0).tolist()
                for p, t in truth.items():
                    if tuple(h[: len(p)]) == p:
                        j = len(h) - len(p)
                        out[i, 0] = t[j] if j < len(t) else 0
            return out
        def observe(self, *a, **kw): pass
        def after_execute(self, *a, **kw): pass

    llm2.engine.spec.drafter = Oracle()
    got2 = [o.outputs[0].token_ids for o in llm2.generate(prompts, sp)]
    assert got2 == plain and llm2.engine.spec.acceptance_rate > 0.9


def test_mtp_chained_drafts_match_plain_greedy():
    """Three draft tokens per step from one MTP layer chained on its own output: the stream is the
    plain greedy one, and every proposal is k tokens wide."""
    from test_deepseek_cpu import _args
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine

    def make(**kw):
        llm = LLM.__new__(LLM)
        llm.engine = LLMEngine(EngineConfig(model="d", device="cpu", dtype="float32", num_blocks=96, enable_graph=False,
                                            max_tokens_per_batch=24, enable_schedule_overlap=False, **kw), model_args=_args())
        llm.tokenizer = None
        return llm

    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (15, 16, 33)]   # 16: a block boundary
    sp = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
    plain = [o.outputs[0].token_ids for o in make().generate(prompts, sp)]
    llm = make(num_speculative_tokens=3, speculative_method="mtp")
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == plain
    d = llm.engine.spec.drafter
    assert d.k == 3 and all(len(v) == 3 for v in d.draft.values())


def test_eagle3_head_drafts_and_stream_is_unchanged():
    """EAGLE-3 head on a tiny dense model: the target exposes three auxiliary hidden states, the head
    drafts two tokens per step over its draft vocabulary (mapped through d2t), and the verified stream
    equals plain greedy decoding."""
    def make(**kw):
        return LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=96, max_seqs_per_batch=8,
                   max_tokens_per_batch=64, enable_graph=False, enable_schedule_overlap=False, **kw)

    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 32000, (n,), generator=g).tolist() for n in (7, 30, 70)]
    sp = SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True)
    plain = [o.outputs[0].token_ids for o in make().generate(prompts, sp)]
    llm = make(num_speculative_tokens=2, speculative_method="eagle3")
    eng = llm.engine
    H = eng.args.hidden_size
    eng.eagle3.d2t.copy_(torch.full_like(eng.eagle3.d2t, 3))       # draft id d stands for target id d + 3
    eng.eagle3.d2t[-3:] = 0
    got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    assert got == plain
    assert eng.model.last_aux.shape[-1] == 3 * H
    assert eng.spec.steps > 0 and all(len(v) == 2 for v in eng.spec.drafter.draft.values())
    ids = torch.tensor([0, 5, 100])
    assert eng.eagle3.to_target_ids(ids).tolist() == [3, 8, 103]


def _mtp_engine(args, **kw):
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
    llm = LLM.__new__(LLM)
    llm.engine = LLMEngine(EngineConfig(model="m", device="cpu", dtype="float32", num_blocks=96, enable_graph=False,
                                        max_tokens_per_batch=64, enable_schedule_overlap=False, **kw), model_args=args)
    llm.tokenizer = None
    return llm


def test_mimo_and_qwen35_mtp_layers_load_by_checkpoint_names_and_draft_losslessly(tmp_path):
    """The MTP layer of MiMo (`model.mtp_layers.0.*`, input [hidden | token]) and of Qwen3.5
    (`mtp.*`, layer under `mtp.layers.0.`): their tensors are found in a checkpoint by the family's
    names, and speculative decoding with them returns the plain greedy stream."""
    from xllm_b200.models import ModelArgs
    from xllm_b200.models.deepseek import MTPDraft, mtp_kind_of
    from xllm_b200.utils.loader import iterate_weights, save_file
    mimo = ModelArgs(model_type="mimo", vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=16, intermediate_size=128, attention_bias=True, qk_norm=False,
                     tie_word_embeddings=False, max_position_embeddings=512)
    q35 = ModelArgs(model_type="qwen3_5", vocab_size=512, hidden_size=64, num_hidden_layers=4, num_attention_heads=4,
                    num_key_value_heads=2, head_dim=16, intermediate_size=128, tie_word_embeddings=False,
                    max_position_embeddings=512, partial_rotary_factor=0.25,
                    extra={"full_attention_interval": 2, "linear_num_value_heads": 4, "linear_num_key_heads": 2,
                           "linear_key_head_dim": 16, "linear_value_head_dim": 16, "linear_conv_kernel_dim": 4})
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 500, (n,), generator=g).tolist() for n in (9, 33)]
    sp = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
    for args, kind, marker in ((mimo, "mimo", "model.mtp_layers.0.token_layernorm.weight"),
                               (q35, "qwen3_5", "mtp.layers.0.self_attn.q_proj.weight")):
        assert mtp_kind_of(args) == kind
        if kind == "mimo":
            plain = [o.outputs[0].token_ids for o in _mtp_engine(args).generate(prompts, sp)]
            llm = _mtp_engine(args, num_speculative_tokens=1, speculative_method="mtp")
            eng = llm.engine
            got = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
            assert got == plain and eng.spec.proposed > 0
        else:
            # a hybrid target keeps recurrent state that rejected drafts would have advanced: the engine
            # refuses to speculate on it; the layer itself is built and run directly
            with pytest.raises(ValueError, match="recurrent state"):
                _mtp_engine(args, num_speculative_tokens=1, speculative_method="mtp")
            eng = _mtp_engine(args).engine
            eng.mtp = MTPDraft(eng.args, eng.model, eng.dtype, eng.device, eng.ps)
            eng.mtp.init_random(seed=3)
            from xllm_b200.models.layers import AttentionMetadata
            T = 12
            k0, v0 = (torch.zeros_like(t) for t in eng.runner.kv_caches[1])
            meta = AttentionMetadata(n_decode=0, n_prefill=1, slots=torch.arange(16, 16 + T, dtype=torch.int32),
                                     block_table=torch.tensor([[1]], dtype=torch.int32), kv_lens=torch.tensor([T], dtype=torch.int32),
                                     cu_q=torch.tensor([0, T], dtype=torch.int32), max_q_len=T, max_kv_len=T)
            h = eng.mtp.forward(torch.arange(T), torch.randn(T, 64), torch.arange(T), meta, k0, v0)
            assert h.shape == (T, 64) and torch.isfinite(h).all() and eng.mtp.logits(h).shape[-1] == 512
        assert eng.mtp.kind == kind
        # export under checkpoint names, load into a fresh layer, compare every tensor
        tensors = {}
        a = eng.mtp.layer.self_attn
        for n, t in eng.mtp.named_params():
            t = t.detach().clone()
            if ".qkv_proj." in n:                      # fused in memory, three tensors in a checkpoint
                nq = t.shape[0] - 2 * a.nkv * a.d
                for part, rows in zip(("q_proj", "k_proj", "v_proj"), t.split([nq, a.nkv * a.d, a.nkv * a.d])):
                    tensors[eng.mtp.checkpoint_name(n.replace("qkv_proj", part))] = rows.contiguous()
            elif ".gate_up_proj." in n:
                for part, rows in zip(("gate_proj", "up_proj"), t.chunk(2)):
                    tensors[eng.mtp.checkpoint_name(n.replace("gate_up_proj", part))] = rows.contiguous()
            else:
                tensors[eng.mtp.checkpoint_name(n)] = t
        assert marker in tensors, sorted(tensors)[:8]
        tensors["model.embed_tokens.weight"] = torch.zeros(4, 4)               # unrelated tensors are ignored
        d = tmp_path / kind
        d.mkdir()
        save_file(tensors, str(d / "model-00001-of-00001.safetensors"), {"format": "pt"})
        fresh = MTPDraft(eng.args, eng.model, eng.dtype, eng.device, eng.ps)
        fresh.init_random(seed=99)
        used = fresh.load_from_checkpoint(iterate_weights(str(d)))
        mine, theirs = dict(fresh.named_params()), dict(eng.mtp.named_params())
        assert used >= len(mine) - 2 and all(torch.equal(mine[n], theirs[n]) for n in mine), kind
