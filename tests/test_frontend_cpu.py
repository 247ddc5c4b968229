"""C++ front end on CPU: JSON, flags, safetensors, tokenizer (vs the HF `tokenizers` library),
incremental decoding with stop strings, chat templates, reasoning and tool-call parsers."""
import json
import os

import pytest
import torch

from xllm_b200 import _rt


def test_json_roundtrip_and_partial_completion():
    text = '{"a": [1, 2.5, true, null, "x\\n\\u00e9\\ud83d\\ude00"], "b": {"c": -3e2}}'
    assert _rt.json_loads(text) == json.loads(text)
    assert json.loads(_rt.json_roundtrip(text)) == json.loads(text)
    with pytest.raises(RuntimeError):
        _rt.json_loads('{"a": }')
    assert json.loads(_rt.complete_partial_json('{"name": "f", "arguments": {"city": "Par')) == \
        {"name": "f", "arguments": {"city": "Par"}}
    assert json.loads(_rt.complete_partial_json('{"a": [1, 2, {"b": 3}, ')) == {"a": [1, 2, {"b": 3}]}
    assert json.loads(_rt.complete_partial_json('{"a": 1, "b"')) == {"a": 1}


def test_flags_reference_names_defaults_json_override(tmp_path):
    f = _rt.FlagRegistry()
    # names and defaults of the reference's launch flags
    assert f.get_int("port") == 8010 and f.get_int("block_size") == 128
    assert f.get_int("max_tokens_per_batch") == 10240 and f.get_int("max_seqs_per_batch") == 1024
    assert f.get_bool("enable_prefix_cache") and f.get_bool("enable_chunked_prefill")
    assert abs(f.get_double("max_memory_utilization") - 0.8) < 1e-9
    assert not f.get_bool("enable_schedule_overlap")
    rest = f.parse_args(["--model=/m", "--port", "9000", "--noenable_prefix_cache", "--enable_schedule_overlap", "x"])
    assert rest == ["x"]
    assert f.get("model") == "/m" and f.get_int("port") == 9000
    assert not f.get_bool("enable_prefix_cache") and f.get_bool("enable_schedule_overlap")
    assert f.validate() == []
    dumped = json.loads(f.to_json())
    assert dumped == {"model": "/m", "port": 9000, "enable_prefix_cache": False, "enable_schedule_overlap": True}
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps({"port": 7000, "block_size": 16}))
    g = _rt.FlagRegistry()
    g.parse_args(["--model", "/m", "--port=9000", f"--config_json_file={cfg}"])
    assert g.get_int("port") == 7000 and g.get_int("block_size") == 16  # the file wins
    with pytest.raises(ValueError):
        _rt.FlagRegistry().parse_args(["--no_such_flag=1"])
    bad = _rt.FlagRegistry()
    bad.parse_args(["--block_size=24"])
    assert any("model" in m for m in bad.validate()) and any("block_size" in m for m in bad.validate())
    assert "SchedulerConfig" in bad.help()
    # cross-flag rules of the reference's option check
    for args, word in ((["--cp_size=2"], "cp_size"), (["--backend=tts"], "backend"), (["--task=classify"], "task"),
                       (["--backend=rec", "--task=embed"], "rec"), (["--enable_eplb"], "enable_eplb"),
                       (["--beam_width=4", "--num_speculative_tokens=2", "--draft_model=/d"], "beam_width"),
                       (["--kv_cache_transfer_mode=COPY"], "kv_cache_transfer_mode"),
                       (["--max_seqs_per_batch=512", "--max_tokens_per_batch=256"], "max_seqs_per_batch"),
                       (["--host_blocks_factor=1.5"], "host_blocks_factor")):
        r = _rt.FlagRegistry()
        r.parse_args(["--model=/m"] + args)
        assert any(word in m for m in r.validate()), (args, r.validate())
    ok = _rt.FlagRegistry()
    ok.parse_args(["--model=/m", "--backend=rec", "--enable_eplb", "--ep_size=2", "--nnodes=2"])
    assert ok.validate() == []


def test_safetensors_roundtrip(tmp_path):
    from xllm_b200.utils.loader import iterate_weights, save_file
    tensors = {"a.weight": torch.randn(5, 7), "b": torch.arange(12, dtype=torch.int64).view(3, 4),
               "c": torch.randn(4, 4).to(torch.bfloat16), "empty": torch.empty(0, 3)}
    save_file(tensors, str(tmp_path / "model-00001-of-00001.safetensors"), {"format": "pt"})
    got = dict(iterate_weights(str(tmp_path)))
    assert set(got) == set(tensors)
    for k, v in tensors.items():
        assert got[k].dtype == v.dtype and tuple(got[k].shape) == tuple(v.shape)
        assert torch.equal(got[k], v)


def _make_tokenizer(tmp_path, digits_single=True):
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    pat = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(pat), behavior="isolated"),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    corpus = ["Hello world, this is a test of the tokenizer! It's 2024 and we've got 12345 numbers.",
              "def foo(x):\n    return x + 1\n\n\nprint(foo(41))", "Ünïcödé tëxt — 你好，世界 🙂 and   spaces\t\ttabs",
              "The quick brown fox jumps over the lazy dog. " * 4, "<|im_start|>user\nhi<|im_end|>"]
    trainer = trainers.BpeTrainer(vocab_size=600, special_tokens=["<|im_start|>", "<|im_end|>", "<|endoftext|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(corpus * 3, trainer)
    path = tmp_path / "tokenizer.json"
    tok.save(str(path))
    return tok, str(path), corpus


def test_bpe_tokenizer_matches_hf_tokenizers(tmp_path):
    hf, path, corpus = _make_tokenizer(tmp_path)
    mine = _rt.BpeTokenizer()
    mine.load_hf_file(path)
    assert mine.vocab_size == hf.get_vocab_size()
    extra = ["a  b   c", " leading space", "trailing space ", "line1\nline2\r\n\r\nline3", "don't can't I'LL",
             "x=1;y=22;z=333", "<|im_start|>system\nYou are<|im_end|>\n<|im_start|>assistant\n", "", " ", "\n\n",
             "naïve café 東京 ünder", "tabs\t\tand  \n  mixed"]
    for text in corpus + extra:
        want = hf.encode(text, add_special_tokens=False).ids
        got = mine.encode(text)
        assert got == want, (text, got, want)
        assert mine.decode(got, False) == text
    assert mine.decode(mine.encode("<|im_start|>hi<|im_end|>"), True) == "hi"


def test_incremental_decoder_utf8_and_stop_strings(tmp_path):
    hf, path, _ = _make_tokenizer(tmp_path)
    tok = _rt.BpeTokenizer()
    tok.load_hf_file(path)
    text = "你好，世界 🙂 done. STOP here"
    ids = tok.encode(text)
    dec = _rt.IncrementalDecoder(tok, [], True)
    pieces = []
    for t in ids:
        s, stopped = dec.push(t)
        assert not stopped
        s.encode("utf-8")  # never a broken code point
        assert "�" not in s
        pieces.append(s)
    assert "".join(pieces) + dec.flush() == text
    dec = _rt.IncrementalDecoder(tok, ["STOP", "never"], True)
    out, hit = "", False
    for t in ids:
        s, stopped = dec.push(t)
        out += s
        if stopped:
            hit = True
            break
    assert hit and out == "你好，世界 🙂 done. "


def test_chat_templates():
    M = _rt.ChatMessage
    t = _rt.ChatTemplate("chatml")
    s = t.apply([M("system", "be brief"), M("user", "hi")], "", True, True)
    assert s == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    s = t.apply([M("user", "hi")], "", True, False)
    assert s.endswith("<|im_start|>assistant\n<think>\n\n</think>\n\n")
    tools = json.dumps([{"type": "function", "function": {"name": "get_weather", "parameters": {}}}])
    s = t.apply([M("user", "weather?"), M("assistant", "", json.dumps([{"function": {"name": "get_weather", "arguments": "{\"c\": 1}"}}])),
                 M("tool", "sunny")], tools, True, True)
    assert "<tools>" in s and "get_weather" in s and "<tool_response>\nsunny\n</tool_response>" in s
    assert '<tool_call>\n{"name": "get_weather", "arguments": {"c": 1}}\n</tool_call>' in s
    assert _rt.ChatTemplate("llama3").apply([M("user", "hi")], "", True, True) == \
        "<|begin_of_text|><|start_header_id|>user<|end_header_id|>\n\nhi<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n"
    assert _rt.ChatTemplate.detect_family("qwen3", "") == "chatml"
    assert _rt.ChatTemplate.detect_family("x", "{{ '<|start_header_id|>' }}") == "llama3"


def test_reasoning_parser_streaming():
    p = _rt.ReasoningParser("qwen3", False)
    text = "<think>step 1\nstep 2</think>\n\nThe answer is 4."
    r, c = "", ""
    for i in range(0, len(text), 3):
        dr, dc = p.push(text[i:i + 3])
        r += dr
        c += dc
    dr, dc = p.flush()
    assert (r + dr, c + dc) == ("step 1\nstep 2", "The answer is 4.")
    p = _rt.ReasoningParser("deepseek-r1", False)
    dr, dc = p.push("thinking...</think>done")
    assert (dr, dc) == ("thinking...", "done")


@pytest.mark.parametrize("kind,text,name,args", [
    ("qwen25", 'Sure.\n<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris", "n": 2}}\n</tool_call>',
     "get_weather", {"city": "Paris", "n": 2}),
    ("qwen3_coder", '<tool_call>\n<function=run>\n<parameter=cmd>\nls -l\n</parameter>\n<parameter=n>\n3\n</parameter>\n</function>\n</tool_call>',
     "run", {"cmd": "ls -l", "n": 3}),
    ("deepseekv3", '<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>get_weather\n```json\n{"city": "Paris"}\n```<｜tool▁call▁end｜><｜tool▁calls▁end｜>',
     "get_weather", {"city": "Paris"}),
    ("kimi_k2", '<|tool_calls_section_begin|><|tool_call_begin|>functions.get_weather:0<|tool_call_argument_begin|>{"city": "Paris"}<|tool_call_end|><|tool_calls_section_end|>',
     "get_weather", {"city": "Paris"}),
    ("glm45", '<tool_call>get_weather\n<arg_key>city</arg_key>\n<arg_value>Paris</arg_value>\n<arg_key>n</arg_key>\n<arg_value>2</arg_value>\n</tool_call>',
     "get_weather", {"city": "Paris", "n": 2}),
])
def test_tool_call_parsers(kind, text, name, args):
    p = _rt.ToolCallParser(kind)
    assert p.has_tool_call(text)
    content, calls = p.parse(text)
    assert len(calls) == 1 and calls[0][1] == name and json.loads(calls[0][2]) == args
    if kind == "qwen25":
        assert content == "Sure."
    # streaming in small pieces gives the same name and argument text
    sp = _rt.ToolCallParser(kind)
    got_name, got_args, got_content = "", "", ""
    for i in range(0, len(text), 5):
        c, cs = sp.push(text[i:i + 5])
        got_content += c
        for _, n, a in cs:
            got_name = got_name or n
            got_args += a
    assert got_name == name and json.loads(got_args) == args
