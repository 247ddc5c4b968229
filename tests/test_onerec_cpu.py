"""OneRec (T5-layout encoder-decoder recommender) against HuggingFace's T5: encoder states, decoder logits,
greedy items, beam scores, padded batches and a catalogue."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from xllm_b200.engine.rec import ItemTrie  # noqa: E402
from xllm_b200.models.onerec import OneRecModel, relative_bucket  # noqa: E402


def _hf(tmp_path, ff):
    cfg = transformers.T5Config(vocab_size=300, d_model=64, d_kv=16, d_ff=128, num_layers=3, num_decoder_layers=2, num_heads=4,
                                relative_attention_num_buckets=8, relative_attention_max_distance=20, feed_forward_proj=ff,
                                tie_word_embeddings=True, decoder_start_token_id=0, pad_token_id=0, eos_token_id=1,
                                dropout_rate=0.0)
    torch.manual_seed(0)
    hf = transformers.T5ForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():                  # the default init leaves the logits nearly flat
            if "layer_norm" not in n:
                p.mul_(3.0)
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    return hf


@pytest.mark.parametrize("ff", ["relu", "gated-gelu"])
def test_onerec_matches_t5(tmp_path, ff):
    hf = _hf(tmp_path, ff)
    m = OneRecModel.from_pretrained(str(tmp_path))
    assert m.args.feed_forward_proj == ff and m.args.num_decoder_layers == 2
    g = torch.Generator().manual_seed(1)
    hist = [torch.randint(2, 300, (n,), generator=g).tolist() for n in (23, 9, 40)]
    # one request, no padding: encoder states and decoder logits
    ids = torch.tensor([hist[0]])
    dec = torch.tensor([[0, 17, 45]])
    with torch.no_grad():
        want = hf(input_ids=ids, decoder_input_ids=dec)
    enc = m.encode(ids)
    assert (enc - want.encoder_last_hidden_state).abs().max() < 2e-4
    logits = m.decode(dec, m.cross_kv(enc))
    assert (logits - want.logits[:, -1]).abs().max() < 2e-3
    # greedy item = HF greedy generation, per request, from ONE padded batch here
    got = m.recommend(hist, beam_width=1, num_steps=3)
    for h, items in zip(hist, got):
        with torch.no_grad():
            ref = hf.generate(torch.tensor([h]), max_new_tokens=3, do_sample=False, eos_token_id=None)[0, 1:].tolist()
        assert items[0].token_ids == ref
    # beams: distinct, sorted, and every score is the teacher-forced log-probability under HF
    beams = m.recommend(hist, beam_width=5, num_steps=3)
    for h, items in zip(hist, beams):
        assert len(items) == 5 and len({tuple(i.token_ids) for i in items}) == 5
        assert all(items[i].logprob >= items[i + 1].logprob for i in range(4))
        for it in items[:3]:
            with torch.no_grad():
                lg = hf(input_ids=torch.tensor([h]), decoder_input_ids=torch.tensor([[0] + it.token_ids[:-1]])).logits[0]
            lp = torch.log_softmax(lg.float(), -1)
            want_lp = sum(float(lp[i, t]) for i, t in enumerate(it.token_ids))
            assert abs(want_lp - it.logprob) < 5e-3
    assert beams[0][0].logprob >= got[0][0].logprob - 1e-4
    # catalogue
    items = [tuple(torch.randint(2, 300, (3,), generator=g).tolist()) for _ in range(20)]
    only = m.recommend(hist[:1], beam_width=6, num_steps=3, trie=ItemTrie(items, 300))[0]
    assert len(only) == 6 and all(tuple(i.token_ids) in set(items) for i in only)


def test_relative_buckets_match_t5():
    from transformers.models.t5.modeling_t5 import T5Attention
    rel = torch.arange(-40, 41)[None, :] - torch.zeros(1, 1, dtype=torch.long)
    for bi in (True, False):
        want = T5Attention._relative_position_bucket(rel, bidirectional=bi, num_buckets=16, max_distance=32)
        assert torch.equal(relative_bucket(rel, bi, 16, 32), want)
