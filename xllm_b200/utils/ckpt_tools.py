"""Checkpoint utilities (command line: `python -m xllm_b200.utils.ckpt_tools <command> ...`).

    compare  A B [--rtol 1e-3 --atol 1e-5]     tensors of two checkpoints (files or directories) side by side
    export-mtp  MODEL_DIR OUT_DIR              the multi-token-prediction layer(s) of a DeepSeek-V3 / MiMo style
                                               checkpoint as a draft-model checkpoint of their own
    dequant-fp8  MODEL_DIR OUT_DIR             block-scaled fp8 weights (+ weight_scale_inv) -> bf16 safetensors

Parity: the reference's tools/compare_tensor.py, tools/export_mtp.py and tools/dequant_minimax_fp8.py.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import shutil
from typing import Dict, Iterator, Tuple

import torch

from .loader import dequant_fp8_stream, iterate_file, iterate_weights, save_file


def _tensors(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    return iterate_weights(path) if os.path.isdir(path) else iterate_file(path)


def compare(a: str, b: str, rtol: float = 1e-3, atol: float = 1e-5) -> Dict[str, dict]:
    """Per-tensor report: max abs / relative difference and whether it is within tolerance; tensors
    present on one side only are listed with `missing`."""
    ta = dict(_tensors(a))
    report = {}
    seen = set()
    for name, y in _tensors(b):
        seen.add(name)
        x = ta.get(name)
        if x is None:
            report[name] = {"missing": "a"}
            continue
        if tuple(x.shape) != tuple(y.shape):
            report[name] = {"shape_a": list(x.shape), "shape_b": list(y.shape), "ok": False}
            continue
        xf, yf = x.float(), y.float()
        d = (xf - yf).abs()
        report[name] = {"max_abs": float(d.max()) if d.numel() else 0.0,
                        "max_rel": float((d / (yf.abs() + 1e-12)).max()) if d.numel() else 0.0,
                        "ok": bool(torch.allclose(xf, yf, rtol=rtol, atol=atol))}
    for name in ta:
        if name not in seen:
            report[name] = {"missing": "b"}
    return report


def export_mtp(model_dir: str, out_dir: str) -> int:
    """DeepSeek-V3 keeps MTP layer k as `model.layers.{num_hidden_layers + k}.*` (with enorm / hnorm /
    eh_proj / shared_head next to the decoder block); MiMo as `model.mtp_layers.{k}.*`.  The export
    renumbers them from 0 under `model.layers.*`, copies embeddings and head, and writes a config whose
    `num_hidden_layers` is the number of MTP layers.  Returns the number of tensors written."""
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    n_layers = int(cfg["num_hidden_layers"])
    n_mtp = int(cfg.get("num_nextn_predict_layers") or 0)
    out: Dict[str, torch.Tensor] = {}
    pat_ds = re.compile(r"^model\.layers\.(\d+)\.(.*)$")
    pat_mimo = re.compile(r"^model\.mtp_layers\.(\d+)\.(.*)$")
    weights = iterate_weights(model_dir)
    if (cfg.get("quantization_config") or {}).get("quant_method") == "fp8":
        weights = dequant_fp8_stream(weights)
    for name, t in weights:
        m = pat_ds.match(name)
        if m and int(m.group(1)) >= n_layers:
            out[f"model.layers.{int(m.group(1)) - n_layers}.{m.group(2)}"] = t
            continue
        m = pat_mimo.match(name)
        if m:
            out[f"model.layers.{m.group(1)}.{m.group(2)}"] = t
            n_mtp = max(n_mtp, int(m.group(1)) + 1)
            continue
        if name in ("model.embed_tokens.weight", "lm_head.weight", "model.norm.weight"):
            out[name] = t
    if not any(k.startswith("model.layers.") for k in out):
        raise ValueError(f"{model_dir} has no multi-token-prediction layers")
    os.makedirs(out_dir, exist_ok=True)
    save_file(out, os.path.join(out_dir, "model.safetensors"), {"format": "pt"})
    cfg = dict(cfg, num_hidden_layers=max(1, n_mtp), num_nextn_predict_layers=0)
    cfg.pop("quantization_config", None)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    for extra in ("tokenizer.json", "tokenizer_config.json", "generation_config.json"):
        if os.path.exists(os.path.join(model_dir, extra)):
            shutil.copy(os.path.join(model_dir, extra), os.path.join(out_dir, extra))
    return len(out)


def dequant_fp8(model_dir: str, out_dir: str, shard_bytes: int = 4 << 30) -> int:
    """Rewrites a block-scaled fp8 checkpoint as bf16 shards; the config loses its quantization_config."""
    os.makedirs(out_dir, exist_ok=True)
    shard, size, idx, n = {}, 0, 0, 0
    index = {}

    def flush():
        nonlocal shard, size, idx
        if shard:
            fn = f"model-{idx:05d}.safetensors"
            save_file(shard, os.path.join(out_dir, fn), {"format": "pt"})
            for k in shard:
                index[k] = fn
            shard, size, idx = {}, 0, idx + 1

    for name, t in dequant_fp8_stream(iterate_weights(model_dir)):
        shard[name] = t
        size += t.numel() * t.element_size()
        n += 1
        if size >= shard_bytes:
            flush()
    flush()
    with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": index}, f)
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    cfg.pop("quantization_config", None)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    return n


def main(argv=None):
    ap = argparse.ArgumentParser(description="checkpoint utilities")
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("compare")
    c.add_argument("a"), c.add_argument("b")
    c.add_argument("--rtol", type=float, default=1e-3), c.add_argument("--atol", type=float, default=1e-5)
    for name in ("export-mtp", "dequant-fp8"):
        p = sub.add_parser(name)
        p.add_argument("model_dir"), p.add_argument("out_dir")
    ns = ap.parse_args(argv)
    if ns.cmd == "compare":
        rep = compare(ns.a, ns.b, ns.rtol, ns.atol)
        bad = {k: v for k, v in rep.items() if not v.get("ok", False)}
        print(json.dumps({"tensors": len(rep), "different": bad}, indent=1))
        return 1 if bad else 0
    if ns.cmd == "export-mtp":
        print(export_mtp(ns.model_dir, ns.out_dir), "tensors written")
    else:
        print(dequant_fp8(ns.model_dir, ns.out_dir), "tensors written")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
