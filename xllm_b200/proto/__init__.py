"""Wire formats: protobuf messages of the services, built at import time.

The schema below is the single source: it is turned into real protobuf descriptors through
`descriptor_pb2` (no protoc needed), and `proto_source()` renders it as `.proto` text for other
languages (`xllm_b200.proto`, next to this file, is that text).  Field names follow the reference's
protos where the meaning is the same (xllm/proto/disagg_pd.proto, completion.proto, chat.proto,
common.proto, xllm_service.proto), so that a client written against those finds the same names; the
message set is this engine's own.

    from xllm_b200 import proto
    m = proto.DisaggRequest(req_id="r1", tokens_num=40, prompt_tokens=[1, 2, 3])
    data = m.SerializeToString(); proto.DisaggRequest.FromString(data)
    proto.encode({"op": "reserve", "rid": "r1", "n_tokens": 40})  # the PD channel's frames
"""
from __future__ import annotations

from typing import Dict, List, Tuple

from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

PACKAGE = "xllm_b200.proto"

# (name, type, number[, "repeated" | "optional"]) per field; types are protobuf scalar names or message names
SCHEMA: Dict[str, List[Tuple]] = {
    # ---- common
    "Status": [("ok", "bool", 1), ("code", "int32", 2), ("message", "string", 3)],
    "Usage": [("prompt_tokens", "int32", 1), ("completion_tokens", "int32", 2), ("total_tokens", "int32", 3)],
    "StopSequence": [("seq_tokens", "int32", 1, "repeated")],
    "SamplingFields": [
        ("max_tokens", "int32", 1), ("temperature", "float", 2), ("top_p", "float", 3), ("top_k", "int64", 4),
        ("frequency_penalty", "float", 5), ("presence_penalty", "float", 6), ("repetition_penalty", "float", 7),
        ("ignore_eos", "bool", 8), ("eos_token_id", "int32", 9, "optional"), ("stop_token_ids", "int32", 10, "repeated"),
        ("stop_sequences", "StopSequence", 11, "repeated"), ("seed", "uint64", 12, "optional"),
        ("logprobs", "bool", 13), ("top_logprobs", "int64", 14), ("n", "int32", 15)],
    # ---- OpenAI-style API bodies (binary form of the JSON routes)
    "CompletionRequest": [
        ("model", "string", 1), ("prompt", "string", 2), ("prompt_tokens", "int32", 3, "repeated"),
        ("sampling", "SamplingFields", 4), ("stream", "bool", 5), ("echo", "bool", 6), ("request_id", "string", 7),
        ("include_usage", "bool", 8), ("offline", "bool", 9), ("priority", "int32", 10)],
    "CompletionChoice": [("index", "int32", 1), ("text", "string", 2), ("finish_reason", "string", 3),
                         ("token_ids", "int32", 4, "repeated"), ("token_logprobs", "float", 5, "repeated")],
    "CompletionResponse": [("id", "string", 1), ("object", "string", 2), ("created", "int64", 3), ("model", "string", 4),
                           ("choices", "CompletionChoice", 5, "repeated"), ("usage", "Usage", 6)],
    "ChatMessage": [("role", "string", 1), ("content", "string", 2), ("reasoning_content", "string", 3),
                    ("tool_calls_json", "string", 4), ("tool_call_id", "string", 5)],
    "ChatRequest": [("model", "string", 1), ("messages", "ChatMessage", 2, "repeated"), ("sampling", "SamplingFields", 3),
                    ("stream", "bool", 4), ("tools_json", "string", 5), ("request_id", "string", 6),
                    ("enable_thinking", "bool", 7), ("include_usage", "bool", 8)],
    "ChatChoice": [("index", "int32", 1), ("message", "ChatMessage", 2), ("delta", "ChatMessage", 3),
                   ("finish_reason", "string", 4)],
    "ChatResponse": [("id", "string", 1), ("object", "string", 2), ("created", "int64", 3), ("model", "string", 4),
                     ("choices", "ChatChoice", 5, "repeated"), ("usage", "Usage", 6)],
    "EmbeddingRequest": [("model", "string", 1), ("input", "string", 2, "repeated"), ("request_id", "string", 3)],
    "Embedding": [("index", "int32", 1), ("embedding", "float", 2, "repeated")],
    "EmbeddingResponse": [("id", "string", 1), ("model", "string", 2), ("data", "Embedding", 3, "repeated"),
                          ("usage", "Usage", 4)],
    # ---- masters and instance links (admin routes)
    "MasterInfos": [("model_id", "string", 1), ("model_path", "string", 2), ("master_status", "int32", 3),
                    ("num_blocks", "int32", 4), ("max_memory_utilization", "float", 5)],
    "P2PLinkRequest": [("role", "string", 1), ("host", "string", 2), ("port", "uint32", 3), ("timeout", "float", 4)],
    "InstanceInfo": [("name", "string", 1), ("rpc_address", "string", 2), ("type", "string", 3), ("dp_size", "int32", 4),
                     ("tp_size", "int32", 5), ("block_size", "int32", 6), ("num_blocks", "int64", 7),
                     ("lease_seconds", "float", 8)],
    "Heartbeat": [("name", "string", 1), ("time", "double", 2), ("num_running", "int32", 3), ("num_waiting", "int32", 4),
                  ("kv_utilization", "float", 5)],
    # ---- prefill / decode disaggregation (the DisaggPDService conversation)
    "Topology": [("block_size", "int32", 1), ("n_layers", "int32", 2), ("n_kv_heads", "int32", 3), ("head_dim", "int32", 4),
                 ("dtype", "string", 5), ("tp", "int32", 6), ("planes", "int32", 7)],
    "TopologyAck": [("ok", "bool", 1), ("reason", "string", 2), ("num_blocks", "int64", 3), ("transport", "string", 4)],
    "DisaggRequest": [("req_id", "string", 1), ("tokens_num", "int64", 2), ("prompt_tokens", "int32", 3, "repeated"),
                      ("sampling", "SamplingFields", 4), ("stream", "bool", 5), ("offline", "bool", 6)],
    "DisaggResponse": [("req_id", "string", 1), ("status_code", "int32", 2), ("blocks", "int32", 3, "repeated"),
                       ("dp_rank", "int32", 4)],
    "KVBlocks": [("layer", "int32", 1), ("blocks", "int32", 2, "repeated"), ("k", "bytes", 3), ("v", "bytes", 4)],
    "FirstGeneration": [("req_id", "string", 1), ("tokens", "int32", 2, "repeated"), ("num_prompt", "int32", 3),
                        ("sampling", "SamplingFields", 4), ("epoch", "uint32", 5)],
    "Adopted": [("req_id", "string", 1), ("ok", "bool", 2), ("reason", "string", 3)],
    "Generation": [("req_id", "string", 1), ("token", "int32", 2), ("logprob", "float", 3), ("finished", "bool", 4),
                   ("finish_reason", "string", 5)],
    "Cancel": [("req_id", "string", 1)],
    "Bye": [],
    "Pull": [("free_blocks", "int32", 1), ("max_requests", "int32", 2)],
    # ---- control events rank 0 sends to the other ranks of an instance, once per step
    "ControlEvent": [("kind", "string", 1), ("request_id", "string", 2), ("prompt_tokens", "int32", 3, "repeated"),
                     ("sampling", "SamplingFields", 4), ("mode", "string", 5)],
    "StepEvents": [("step", "int64", 1), ("events", "ControlEvent", 2, "repeated"), ("stop", "bool", 3)],
}

_SCALARS = {
    "double": 1, "float": 2, "int64": 3, "uint64": 4, "int32": 5, "bool": 8, "string": 9, "bytes": 12, "uint32": 13,
}
_TYPE_MESSAGE = 11
_LABEL_OPTIONAL, _LABEL_REPEATED = 1, 3


def _build():
    fd = descriptor_pb2.FileDescriptorProto()
    fd.name = "xllm_b200.proto"
    fd.package = PACKAGE
    fd.syntax = "proto3"
    for name, fields in SCHEMA.items():
        m = fd.message_type.add()
        m.name = name
        for f in fields:
            fname, ftype, num = f[0], f[1], f[2]
            mod = f[3] if len(f) > 3 else ""
            fp = m.field.add()
            fp.name, fp.number = fname, num
            fp.label = _LABEL_REPEATED if mod == "repeated" else _LABEL_OPTIONAL
            if ftype in _SCALARS:
                fp.type = _SCALARS[ftype]
            else:
                fp.type = _TYPE_MESSAGE
                fp.type_name = f".{PACKAGE}.{ftype}"
            if mod == "optional":
                fp.proto3_optional = True
                od = m.oneof_decl.add()
                od.name = "_" + fname
                fp.oneof_index = len(m.oneof_decl) - 1
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    classes = {}
    for name in SCHEMA:
        classes[name] = message_factory.GetMessageClass(pool.FindMessageTypeByName(f"{PACKAGE}.{name}"))
    return fd, classes


FILE_DESCRIPTOR, MESSAGES = _build()
globals().update(MESSAGES)


def proto_source() -> str:
    """The schema as `.proto` text."""
    out = ['syntax = "proto3";', f"package {PACKAGE};", ""]
    for name, fields in SCHEMA.items():
        out.append(f"message {name} {{")
        for f in fields:
            mod = (f[3] + " ") if len(f) > 3 else ""
            out.append(f"  {mod}{f[1]} {f[0]} = {f[2]};")
        out.append("}")
        out.append("")
    return "\n".join(out)


# ------------------------------------------------------------------------------------------ PD channel frames
# op name of the dict protocol (engine/pd_service.py) -> (frame type id, message, dict key -> field)
_SAMPLING_KEYS = {f[0] for f in SCHEMA["SamplingFields"]}
_OPS = {
    "hello": (1, "Topology", {}), "hello_ack": (2, "TopologyAck", {}),
    "reserve": (3, "DisaggRequest", {"rid": "req_id", "n_tokens": "tokens_num"}),
    "reserved": (4, "DisaggResponse", {"rid": "req_id"}),
    "kv": (5, "KVBlocks", {}),
    "first": (6, "FirstGeneration", {"rid": "req_id"}),
    "adopted": (7, "Adopted", {"rid": "req_id"}),
    "gen": (8, "Generation", {"rid": "req_id", "reason": "finish_reason"}),
    "cancel": (9, "Cancel", {"rid": "req_id"}),
    "bye": (10, "Bye", {}),
    "pull": (11, "Pull", {}),
}
_BY_ID = {v[0]: (k, v[1], {b: a for a, b in v[2].items()}) for k, v in _OPS.items()}


def _repeated(field) -> bool:
    r = getattr(field, "is_repeated", None)
    if r is not None:
        return bool(r() if callable(r) else r)
    return field.label == field.LABEL_REPEATED


def _fill_sampling(msg, par: dict):
    for k, v in par.items():
        if v is None or k not in _SAMPLING_KEYS:
            continue
        if k == "stop_sequences":
            for s in v:
                msg.stop_sequences.add().seq_tokens.extend(int(t) for t in s)
        elif k == "stop_token_ids":
            msg.stop_token_ids.extend(int(t) for t in v)
        else:
            setattr(msg, k, v)


def _read_sampling(msg) -> dict:
    out = {}
    for f, v in msg.ListFields():
        if f.name == "stop_sequences":
            out[f.name] = [list(s.seq_tokens) for s in v]
        elif _repeated(f):
            out[f.name] = list(v)
        else:
            out[f.name] = v
    # proto3 scalars at their default are absent from ListFields: the zero values the protocol relies on
    for k in ("temperature", "ignore_eos"):
        out.setdefault(k, getattr(msg, k))
    return out


def encode(d: dict) -> bytes:
    """One frame body of the PD channel: a type byte, then the serialized message."""
    tid, mname, ren = _OPS[d["op"]]
    m = MESSAGES[mname]()
    for k, v in d.items():
        if k == "op" or v is None:
            continue
        k = ren.get(k, k)
        if k == "sampling":
            _fill_sampling(m.sampling, v)
        elif isinstance(v, (list, tuple)):
            getattr(m, k).extend(v)
        else:
            setattr(m, k, v)
    return bytes([tid]) + m.SerializeToString()


def decode(data: bytes) -> dict:
    op, mname, ren = _BY_ID[data[0]]
    m = MESSAGES[mname].FromString(bytes(data[1:]))
    out = {"op": op}
    for f in m.DESCRIPTOR.fields:
        key = ren.get(f.name, f.name)
        if f.name == "sampling":
            if m.HasField("sampling"):
                out[key] = _read_sampling(m.sampling)
        elif _repeated(f):
            out[key] = list(getattr(m, f.name))
        else:
            out[key] = getattr(m, f.name)
    return out
