"""JSON-object grammar: validator against json.loads on prefixes, and constrained decoding of the
tiny model over a synthetic vocabulary."""
import json

import torch

from xllm_b200.engine.grammar import GrammarFilter, JsonObjectValidator


def _ok_prefix(s):
    v = JsonObjectValidator()
    return all(v.feed(c) for c in s), v


def test_validator_accepts_every_prefix_of_valid_objects_and_rejects_bad_steps():
    good = ['{"a": 1, "b": [true, false, null, -0.5e+3, "x\\n\\u00e9"], "c": {"d": {}}, "e": []}',
            ' {"k":"v"} ', '{}', '{"a":[[1,2],[3]],"b":0}']
    for g in good:
        json.loads(g)
        for i in range(1, len(g) + 1):
            ok, v = _ok_prefix(g[:i])
            assert ok, g[:i]
        assert v.complete
    bad = ['[', '{1', '{"a" 1', '{"a":01', '{"a":1,}', '{"a":tru3', '{"a":1}}', '{"a":"\x01', '{"a":1.e', 'x', '{"a":--1']
    for b in bad:
        ok, _ = _ok_prefix(b)
        assert not ok, b


def test_filter_keeps_random_logits_inside_the_grammar():
    pieces = ['{', '}', '[', ']', ':', ',', '"', ' ', 'a', 'b', '"key"', '"v"', '1', '23', '.5', 'true', 'false', 'null',
              '{"', '":', '",', 'e', '-', '\\', 'tr', 'ue', '}}', ']]', '\n']
    vocab = [pieces[i % len(pieces)] for i in range(512)]
    EOS = 511
    vocab[EOS] = ""
    gf = GrammarFilter(vocab, top_n=32, eos_token_id=EOS)
    g = torch.Generator().manual_seed(0)
    for trial in range(5):
        rid = f"r{trial}"
        gf.start(rid)
        text = ""
        for step in range(200):
            logits = torch.randn(512, generator=g)
            if step > 20:
                logits[[i for i, p in enumerate(vocab) if p in ('}', ']', '"', '1', 'null')]] += 4.0  # nudge to close
            gf.filter_row(rid, logits)
            tok = int(torch.argmax(logits))
            assert torch.isfinite(logits[tok])
            if tok == EOS:
                break
            gf.advance(rid, tok)
            text += vocab[tok]
            ok, _ = _ok_prefix(text)
            assert ok, text
        if gf.is_complete(rid):
            assert isinstance(json.loads(text), dict)


def test_engine_json_object_requests_emit_valid_json():
    from xllm_b200 import LLM
    llm = LLM("tiny", devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=4,
              max_tokens_per_batch=128, enable_graph=False, enable_schedule_overlap=False)
    eng = llm.engine
    pieces = ['{', '}', '[', ']', ':', ',', '"k"', '"v"', ' ', '1', '2', 'true', 'null', 'x', 'y', '{"a"', '"b":']
    vocab = [pieces[i % len(pieces)] for i in range(eng.args.vocab_size)]
    EOS = 7
    vocab[EOS] = ""
    eng.set_grammar_vocab(vocab, eos_token_id=EOS, top_n=48)
    g = torch.Generator().manual_seed(1)
    texts = {}
    for i in range(3):
        eng.add_request(f"j{i}", torch.randint(0, 32000, (20,), generator=g).tolist(), temperature=0.8, top_k=40,
                        max_tokens=60, eos_token_id=EOS, json_object=True, seed=i)
        texts[f"j{i}"] = ""
    eng.add_request("free", torch.randint(0, 32000, (20,), generator=g).tolist(), temperature=0.0, max_tokens=8,
                    ignore_eos=True)
    done = {}
    while eng.has_unfinished():
        for ev in eng.step():
            if ev.request_id in texts and ev.token >= 0 and ev.token != EOS:
                texts[ev.request_id] += vocab[ev.token]
            if ev.request_finished:
                done[ev.request_id] = ev.finish_reason
    for rid, t in texts.items():
        ok, v = _ok_prefix(t)
        assert ok, (rid, t)
        if v.complete:
            assert isinstance(json.loads(t), dict)
    assert not eng.grammar.state          # validators are dropped when their request ends
