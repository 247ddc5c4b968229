"""Launch-configuration policy against fake hardware."""
from xllm_b200.auto_config import Hardware, detect_hardware, kv_bytes_per_token, tune, weight_bytes
from xllm_b200.models import preset


def test_weight_and_kv_accounting():
    a = preset("qwen3-8b")
    wb = weight_bytes(a)
    assert 15.5e9 < wb < 17e9                              # 8.2 B parameters in bf16
    assert kv_bytes_per_token(a, 1, False) == 36 * 2 * 8 * 128 * 2
    assert kv_bytes_per_token(a, 8, False) == 36 * 2 * 1 * 128 * 2
    d = preset("deepseek-v3")
    assert kv_bytes_per_token(d, 8, True) == 61 * 576 * 2
    assert 1.2e12 < weight_bytes(d) < 1.45e12


def test_policy_on_fake_boxes():
    a = preset("qwen3-8b")
    one = tune(a, Hardware(n_gpus=1))
    assert one["nnodes"] == 1 and one["max_tokens_per_batch"] == 8192 and one["max_seqs_per_batch"] >= 64
    assert tune(a, Hardware(n_gpus=1), max_model_len=2048)["max_seqs_per_batch"] == 512
    eight = tune(a, Hardware(n_gpus=8))
    assert eight["nnodes"] == 1 and eight["dp_size"] == 8      # the model fits one GPU: replicas, not shards
    slo = tune(a, Hardware(n_gpus=1), tpot_slo_ms=40)
    assert slo["max_tokens_per_batch"] < 8192
    d = tune(preset("deepseek-v3"), Hardware(n_gpus=8))
    assert d["nnodes"] == 8 and d["ep_size"] == 8 and d["mla_latent_cache"] and d["speculative_method"] == "mtp"
    small = tune(a, Hardware(n_gpus=2, hbm_bytes=24 * 10 ** 9))
    assert small["nnodes"] == 2                                # 16 GB of weights do not leave KV room on a 24 GB part


def test_detect_hardware_with_a_probe():
    hw = detect_hardware(lambda: [{"name": "NVIDIA B200", "memory_bytes": 183 * 2 ** 30}] * 4)
    assert hw.n_gpus == 4 and hw.nvlink and hw.hbm_bytes == 183 * 2 ** 30
    assert detect_hardware(lambda: []).n_gpus == 1
