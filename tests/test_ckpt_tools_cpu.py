"""Checkpoint tools on small synthetic checkpoints."""
import json

import torch

from xllm_b200.ops import fp8
from xllm_b200.utils import ckpt_tools
from xllm_b200.utils.loader import iterate_weights, save_file


def test_compare_reports_differences(tmp_path):
    a = {"x.weight": torch.randn(4, 8), "y.weight": torch.randn(3)}
    b = {"x.weight": a["x.weight"].clone(), "y.weight": a["y.weight"] + 0.5, "z.weight": torch.zeros(2)}
    save_file(a, str(tmp_path / "a.safetensors"))
    save_file(b, str(tmp_path / "b.safetensors"))
    rep = ckpt_tools.compare(str(tmp_path / "a.safetensors"), str(tmp_path / "b.safetensors"))
    assert rep["x.weight"]["ok"] and not rep["y.weight"]["ok"] and abs(rep["y.weight"]["max_abs"] - 0.5) < 1e-6
    assert rep["z.weight"] == {"missing": "a"}
    assert ckpt_tools.main(["compare", str(tmp_path / "a.safetensors"), str(tmp_path / "a.safetensors")]) == 0


def test_export_mtp_renumbers_the_extra_layers(tmp_path):
    src = tmp_path / "src"
    src.mkdir()
    (src / "config.json").write_text(json.dumps({"model_type": "deepseek_v3", "num_hidden_layers": 2,
                                                 "num_nextn_predict_layers": 1, "hidden_size": 8}))
    t = {"model.embed_tokens.weight": torch.randn(10, 8), "lm_head.weight": torch.randn(10, 8),
         "model.layers.0.input_layernorm.weight": torch.ones(8), "model.layers.1.input_layernorm.weight": torch.ones(8),
         "model.layers.2.enorm.weight": torch.full((8,), 2.0), "model.layers.2.eh_proj.weight": torch.randn(8, 16),
         "model.layers.2.self_attn.o_proj.weight": torch.randn(8, 8)}
    save_file(t, str(src / "model.safetensors"))
    n = ckpt_tools.export_mtp(str(src), str(tmp_path / "out"))
    got = dict(iterate_weights(str(tmp_path / "out")))
    assert n == len(got) == 5
    assert torch.equal(got["model.layers.0.enorm.weight"], t["model.layers.2.enorm.weight"])
    assert "model.layers.0.input_layernorm.weight" not in got and "model.embed_tokens.weight" in got
    cfg = json.loads((tmp_path / "out" / "config.json").read_text())
    assert cfg["num_hidden_layers"] == 1 and cfg["num_nextn_predict_layers"] == 0


def test_dequant_fp8_writes_bf16_shards(tmp_path):
    src = tmp_path / "src"
    src.mkdir()
    (src / "config.json").write_text(json.dumps({"model_type": "deepseek_v3", "quantization_config": {
        "quant_method": "fp8", "weight_block_size": [128, 128]}}))
    w = torch.randn(256, 128) * 0.1
    q, s = fp8.quant_block128_ref(w)
    save_file({"a.weight": q, "a.weight_scale_inv": s, "norm.weight": torch.ones(4, dtype=torch.bfloat16)},
              str(src / "model.safetensors"))
    assert ckpt_tools.dequant_fp8(str(src), str(tmp_path / "out"), shard_bytes=1 << 12) == 2
    got = dict(iterate_weights(str(tmp_path / "out")))
    assert got["a.weight"].dtype == torch.bfloat16 and (got["a.weight"].float() - w).abs().max() < 0.03
    assert "quantization_config" not in json.loads((tmp_path / "out" / "config.json").read_text())
