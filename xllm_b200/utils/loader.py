"""Checkpoint loading: HuggingFace directory -> (name, tensor) stream.

Parity: HFModelLoader + StateDictFromSafeTensor (xllm/core/framework/hf_model_loader.cpp,
state_dict/state_dict.cpp): enumerate `*.safetensors` shards in sorted order (or follow
`model.safetensors.index.json`), mmap each, hand out zero-copy tensors; each module's loader picks
and shards what it needs.  The mmap / header parsing is the C++ `SafeTensorsFile`.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterator, List, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


def shard_files(model_dir: str) -> List[str]:
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        return [os.path.join(model_dir, x) for x in files]
    return sorted(os.path.join(model_dir, x) for x in os.listdir(model_dir) if x.endswith(".safetensors"))


def iterate_file(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    from .. import _rt
    f = _rt.SafeTensorsFile(path)
    buf = f.buffer()
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")  # the mapping is read-only by design; tensors are only copied from
        raw = torch.frombuffer(buf, dtype=torch.uint8) if len(buf) else torch.empty(0, dtype=torch.uint8)
    for name, (dt, shape, begin, end) in f.index().items():
        dtype = _DTYPES[dt]
        if end <= begin:
            t = torch.empty(shape, dtype=dtype)
        else:
            b = raw[begin:end]
            esz = torch.empty((), dtype=dtype).element_size()
            if (b.data_ptr() % esz) != 0:
                b = b.clone()  # a file whose data section is not aligned for this dtype
            t = b.view(dtype).view(*shape)
        t._xllm_keepalive = f  # the mmap lives as long as any tensor cut from it
        yield name, t


def iterate_weights(model_dir: str) -> Iterator[Tuple[str, torch.Tensor]]:
    files = shard_files(model_dir)
    if not files:
        raise FileNotFoundError(f"no *.safetensors under {model_dir}")
    for p in files:
        yield from iterate_file(p)


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Dict[str, str] = None) -> None:
    """Write a safetensors file (used by tests, by `update_weights` round trips and by tools)."""
    header = {}
    if metadata:
        header["__metadata__"] = metadata
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        b = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        off += len(b)
        blobs.append(b)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(len(hj).to_bytes(8, "little"))
        f.write(hj)
        for b in blobs:
            f.write(b)


def dequant_fp8_stream(weights, keep_fp8=None, dtype=torch.bfloat16):
    """Pair every block-scaled fp8 tensor `X.weight` with its `X.weight_scale_inv` (128 x 128 blocks,
    DeepSeek-V3 checkpoints) and yield the bf16 weight; everything else passes through.  Weights named in
    `keep_fp8` (a set of `X.weight` names: layers that execute in fp8) pass through untouched, scales
    included.  `dtype`: type of the dequantised tensors (the model's compute type)."""
    from ..ops import fp8
    pending_w, pending_s = {}, {}
    keep_fp8 = keep_fp8 or ()
    for name, t in weights:
        if name in keep_fp8 or (name.endswith("_scale_inv") and name[: -len("_scale_inv")] in keep_fp8):
            yield name, t
        elif name.endswith(".weight_scale_inv"):
            base = name[: -len("_scale_inv")]
            if base in pending_w:
                yield base, fp8.dequant_block128_ref(pending_w.pop(base), t.float(), dtype)
            else:
                pending_s[base] = t
        elif t.dtype == torch.float8_e4m3fn:
            if name in pending_s:
                yield name, fp8.dequant_block128_ref(t, pending_s.pop(name).float(), dtype)
            else:
                pending_w[name] = t
        else:
            yield name, t
    for name, t in pending_w.items():  # fp8 tensors without scales: plain cast
        yield name, t.to(dtype)
