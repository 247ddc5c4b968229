"""Wire formats: the message classes are real protobuf messages, the PD channel's frames round-trip,
and the committed .proto text matches the schema."""
import os

from xllm_b200 import proto


def test_messages_serialize_and_parse():
    r = proto.CompletionRequest(model="m", prompt_tokens=[1, 2, 3], stream=True)
    r.sampling.max_tokens = 16
    r.sampling.stop_sequences.add().seq_tokens.extend([7, 8])
    back = proto.CompletionRequest.FromString(r.SerializeToString())
    assert back.model == "m" and list(back.prompt_tokens) == [1, 2, 3] and back.sampling.max_tokens == 16
    assert list(back.sampling.stop_sequences[0].seq_tokens) == [7, 8]
    assert not back.sampling.HasField("seed")            # proto3 optional: absent is not zero
    back.sampling.seed = 0
    assert proto.SamplingFields.FromString(back.sampling.SerializeToString()).HasField("seed")
    resp = proto.ChatResponse(id="x", choices=[proto.ChatChoice(index=0, message=proto.ChatMessage(role="assistant", content="hi"))])
    assert proto.ChatResponse.FromString(resp.SerializeToString()).choices[0].message.content == "hi"


def test_pd_frames_round_trip():
    frames = [
        {"op": "hello", "block_size": 16, "n_layers": 3, "n_kv_heads": 2, "head_dim": 128, "dtype": "torch.bfloat16", "tp": 1, "planes": 2},
        {"op": "hello_ack", "ok": True, "reason": "", "num_blocks": 4096, "transport": "peer_push"},
        {"op": "reserve", "rid": "r1", "n_tokens": 41},
        {"op": "reserved", "rid": "r1", "blocks": [5, 6, 7]},
        {"op": "reserved", "rid": "r2", "blocks": []},
        {"op": "kv", "layer": 1, "blocks": [5, 6], "k": b"\x00\x01\xff" * 100, "v": b"abc"},
        {"op": "first", "rid": "r1", "tokens": list(range(41)), "num_prompt": 40, "epoch": 9,
         "sampling": {"max_tokens": 12, "temperature": 0.0, "top_p": 1.0, "top_k": -1, "ignore_eos": True,
                      "stop_token_ids": [3], "stop_sequences": [[1, 2], [9]], "seed": None}},
        {"op": "adopted", "rid": "r1", "ok": False, "reason": "kv of layer 2 did not arrive"},
        {"op": "gen", "rid": "r1", "token": 77, "logprob": -0.5, "finished": True, "reason": "length"},
        {"op": "cancel", "rid": "r1"}, {"op": "bye"},
    ]
    for f in frames:
        g = proto.decode(proto.encode(f))
        assert g["op"] == f["op"]
        for k, v in f.items():
            if k == "sampling":
                for sk, sv in v.items():
                    if sv is not None:
                        assert g["sampling"][sk] == sv, (sk, g["sampling"])
                assert "seed" not in g["sampling"]
            else:
                assert g[k] == v, (f["op"], k)


def test_committed_proto_text_is_current():
    path = os.path.join(os.path.dirname(proto.__file__), "xllm_b200.proto")
    assert open(path).read() == proto.proto_source()
    assert "message DisaggRequest {" in proto.proto_source() and "repeated int32 prompt_tokens = 3;" in proto.proto_source()
