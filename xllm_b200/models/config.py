"""Model arguments parsed from a HuggingFace ``config.json``.

Counterpart of the reference's ``ModelArgs`` + per-model ``REGISTER_MODEL_ARGS`` loaders
(xllm/core/framework/model/model_args.h, xllm/models/llm/qwen3.h:259-286,
xllm/core/framework/hf_model_loader.cpp): one dataclass, filled by a per-``model_type`` hook.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional


@dataclass
class ModelArgs:
    model_type: str = "qwen3"
    architectures: List[str] = field(default_factory=list)
    vocab_size: int = 151936
    hidden_size: int = 4096
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 12288
    hidden_act: str = "silu"
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    rope_scaling: Optional[Dict[str, Any]] = None
    partial_rotary_factor: float = 1.0
    rope_interleaved: bool = False
    max_position_embeddings: int = 40960
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    qk_norm: bool = True
    sliding_window: int = 0
    bos_token_id: int = -1
    eos_token_id: int = -1
    stop_token_ids: List[int] = field(default_factory=list)
    dtype: str = "bfloat16"
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    n_shared_experts: int = 0
    shared_expert_intermediate_size: int = 0
    first_k_dense_replace: int = 0
    moe_layer_freq: int = 1
    mlp_only_layers: List[int] = field(default_factory=list)
    scoring_func: str = "softmax"
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    router_bias: bool = False  # e_score_correction_bias
    # MLA
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    mla_latent_cache: bool = False   # paged cache of [c_kv | k_pe] rows shared by all heads instead of per-head K/V
    mla_rope_split_half: bool = False  # checkpoint rotates (x[:d/2], x[d/2:]) pairs; the kernels rotate adjacent pairs
    # DSA (sparse attention through a lightweight indexer: DeepSeek-V3.2, GLM-5)
    index_n_heads: int = 0
    index_head_dim: int = 0
    index_topk: int = 0
    indexer_rope_interleave: bool = False
    # multi-token prediction
    num_nextn_predict_layers: int = 0
    # quantisation (from `quantization_config`)
    quant_method: str = ""
    quant_block: List[int] = field(default_factory=list)
    # run block-scaled fp8 checkpoints on the fp8 GEMM (weights stay e4m3) instead of dequantising at load
    fp8_execution: bool = False
    # VLM
    vision_config: Optional[Dict[str, Any]] = None
    image_token_id: int = -1
    video_token_id: int = -1
    vision_start_token_id: int = -1
    mrope_section: List[int] = field(default_factory=list)   # rotary pairs per (t, h, w) axis
    extra: Dict[str, Any] = field(default_factory=dict)

    @property
    def rotary_dim(self) -> int:
        d = self.qk_rope_head_dim if self.kv_lora_rank else self.head_dim
        return int(d * self.partial_rotary_factor)

    def is_moe_layer(self, i: int) -> bool:
        if self.num_experts <= 0:
            return False
        if i in self.mlp_only_layers or i < self.first_k_dense_replace:
            return False
        return (i + 1) % max(self.moe_layer_freq, 1) == 0 if self.moe_layer_freq > 1 else True


def _g(d, *names, default=None):
    for n in names:
        if n in d and d[n] is not None:
            return d[n]
    return default


def _eos_list(v):
    if v is None:
        return -1, []
    if isinstance(v, list):
        return (v[0] if v else -1), list(v)
    return int(v), [int(v)]


def model_args_from_dict(cfg: Dict[str, Any]) -> ModelArgs:
    text = cfg.get("text_config", cfg)  # VLM configs nest the language model
    mt = text.get("model_type", cfg.get("model_type", "qwen3"))
    a = ModelArgs(model_type=cfg.get("model_type", mt))
    a.architectures = list(cfg.get("architectures", []))
    a.vocab_size = _g(text, "vocab_size", default=a.vocab_size)
    a.hidden_size = _g(text, "hidden_size", default=a.hidden_size)
    a.num_hidden_layers = _g(text, "num_hidden_layers", default=a.num_hidden_layers)
    a.num_attention_heads = _g(text, "num_attention_heads", default=a.num_attention_heads)
    a.num_key_value_heads = _g(text, "num_key_value_heads", default=a.num_attention_heads)
    a.head_dim = _g(text, "head_dim", default=a.hidden_size // a.num_attention_heads)
    a.intermediate_size = _g(text, "intermediate_size", default=a.intermediate_size)
    a.hidden_act = _g(text, "hidden_act", default="silu")
    a.rms_norm_eps = _g(text, "rms_norm_eps", default=1e-6)
    a.rope_theta = float(_g(text, "rope_theta", default=10000.0))
    a.rope_scaling = _g(text, "rope_scaling")
    if isinstance(a.rope_scaling, dict) and "rope_theta" in a.rope_scaling:
        a.rope_theta = float(a.rope_scaling["rope_theta"])
    a.partial_rotary_factor = float(_g(text, "partial_rotary_factor", default=1.0))
    rp = _g(text, "rope_parameters")       # newer configs keep theta, the partial factor and the scaling here
    if isinstance(rp, dict):
        a.rope_theta = float(rp.get("rope_theta", a.rope_theta))
        a.partial_rotary_factor = float(rp.get("partial_rotary_factor", a.partial_rotary_factor))
        if rp.get("rope_type", "default") not in ("default", None) and a.rope_scaling is None:
            a.rope_scaling = dict(rp)
    if _g(text, "rotary_dim") and a.partial_rotary_factor == 1.0:
        a.partial_rotary_factor = float(text["rotary_dim"]) / a.head_dim
    a.max_position_embeddings = _g(text, "max_position_embeddings", default=32768)
    a.tie_word_embeddings = bool(_g(cfg, "tie_word_embeddings", default=_g(text, "tie_word_embeddings", default=False)))
    # Qwen-style configs carry a window plus a switch; Mistral-style configs carry only the window
    use_window = _g(text, "use_sliding_window", default=None)
    if use_window is None:
        use_window = mt in ("mistral", "mixtral")
    a.sliding_window = int(_g(text, "sliding_window", default=0) or 0) if use_window else 0
    a.bos_token_id = _g(text, "bos_token_id", default=-1)
    a.eos_token_id, a.stop_token_ids = _eos_list(_g(text, "eos_token_id", default=_g(cfg, "eos_token_id")))
    a.dtype = _g(text, "torch_dtype", "dtype", default=_g(cfg, "torch_dtype", "dtype", default="bfloat16"))
    base = mt.lower()
    a.qk_norm = bool(_g(text, "use_qk_norm", default=base.startswith("qwen3") or base in ("mimo_v2", "minimax_m2")))
    a.attention_bias = bool(_g(text, "attention_bias", default=base.startswith("qwen2") or base == "mimo"))
    a.rope_interleaved = base in ("glm4", "glm")    # GLM dense rotates adjacent pairs
    # MoE
    a.num_experts = _g(text, "num_experts", "n_routed_experts", "num_local_experts", default=0)
    a.num_experts_per_tok = _g(text, "num_experts_per_tok", default=0)
    a.moe_intermediate_size = _g(text, "moe_intermediate_size", default=0)
    a.norm_topk_prob = bool(_g(text, "norm_topk_prob", default=True))
    a.n_shared_experts = _g(text, "n_shared_experts", default=0) or 0
    a.shared_expert_intermediate_size = _g(text, "shared_expert_intermediate_size", default=0) or 0
    a.first_k_dense_replace = _g(text, "first_k_dense_replace", default=0)
    a.moe_layer_freq = _g(text, "moe_layer_freq", "decoder_sparse_step", default=1)
    a.mlp_only_layers = list(_g(text, "mlp_only_layers", default=[]))
    _v3_like = base in ("deepseek_v3", "deepseek_v32", "glm4_moe", "glm_moe_dsa", "minimax_m2", "kimi_k2")
    lt = _g(text, "mlp_layer_types", default=None)      # per-layer "dense" / "sparse" instead of first_k_dense_replace
    if isinstance(lt, list) and lt:
        a.mlp_only_layers = [i for i, t in enumerate(lt) if t == "dense"]
        a.first_k_dense_replace = 0
    a.scoring_func = _g(text, "scoring_func", default="sigmoid" if _v3_like else "softmax")
    a.n_group = _g(text, "n_group", default=1) or 1
    a.topk_group = _g(text, "topk_group", default=1) or 1
    a.routed_scaling_factor = float(_g(text, "routed_scaling_factor", default=1.0))
    # DeepSeek-V3 and its descendants always carry `e_score_correction_bias` (and rank expert groups
    # by the sum of their two best biased scores); older configs say so with topk_method
    a.router_bias = _g(text, "topk_method", default="") == "noaux_tc" or _v3_like
    # MLA
    a.q_lora_rank = _g(text, "q_lora_rank", default=0) or 0
    a.kv_lora_rank = _g(text, "kv_lora_rank", default=0) or 0
    a.qk_nope_head_dim = _g(text, "qk_nope_head_dim", default=0)
    a.qk_rope_head_dim = _g(text, "qk_rope_head_dim", default=0)
    a.v_head_dim = _g(text, "v_head_dim", default=0)
    a.num_nextn_predict_layers = _g(text, "num_nextn_predict_layers", default=0)
    if base == "rwkv7":
        # attention-free: heads of `head_size` channels, a 4x channel-mix unless the config says otherwise
        a.head_dim = int(_g(text, "head_size", "head_dim", default=64))
        a.num_attention_heads = int(_g(text, "num_attention_heads", "num_heads", default=a.hidden_size // a.head_dim))
        a.num_key_value_heads = a.num_attention_heads
        a.intermediate_size = int(_g(text, "intermediate_size", default=4 * a.hidden_size) or 4 * a.hidden_size)
        for key in ("layer_norm_eps", "decay_low_rank_dim", "a_low_rank_dim", "v_low_rank_dim", "gate_low_rank_dim",
                    "group_norm_eps"):
            if text.get(key) is not None:
                a.extra[key] = text[key]
    if base in ("deepseek_v32", "glm_moe_dsa"):
        a.index_n_heads = int(_g(text, "index_n_heads", default=64 if base == "deepseek_v32" else 32))
        a.index_head_dim = int(_g(text, "index_head_dim", default=128))
        a.index_topk = int(_g(text, "index_topk", default=2048))
        # DeepSeek-V3.2 rotates adjacent pairs in attention and halves in the indexer; the GLM
        # checkpoints (as HuggingFace runs them) rotate halves in both
        a.mla_rope_split_half = bool(_g(text, "rope_interleave", default=base == "deepseek_v32")) is False
        a.indexer_rope_interleave = bool(_g(text, "indexer_rope_interleave", default=False))
        a.mla_latent_cache = True            # sparse selection gathers rows of the latent cache
    q = cfg.get("quantization_config") or text.get("quantization_config")
    if q:
        a.quant_method = q.get("quant_method", "")
        a.quant_block = list(q.get("weight_block_size") or [])
    for key in ("layer_types", "full_attention_interval", "linear_num_value_heads", "linear_num_key_heads",
                "linear_key_head_dim", "linear_value_head_dim", "linear_conv_kernel_dim"):
        if text.get(key) is not None:
            a.extra[key] = text[key]
    a.vision_config = cfg.get("vision_config")
    a.image_token_id = _g(cfg, "image_token_id", default=-1)
    a.vision_start_token_id = _g(cfg, "vision_start_token_id", default=-1)
    rs = cfg.get("rope_scaling") or (cfg.get("text_config") or {}).get("rope_scaling") or \
        (rp if isinstance(rp, dict) else None) or {}
    a.mrope_section = list(rs.get("mrope_section") or [])
    a.video_token_id = _g(cfg, "video_token_id", default=-1)
    return a


def load_model_args(model_dir: str) -> ModelArgs:
    p = Path(model_dir) / "config.json"
    with open(p) as f:
        cfg = json.load(f)
    args = model_args_from_dict(cfg)
    gen = Path(model_dir) / "generation_config.json"
    if gen.exists():
        with open(gen) as f:
            g = json.load(f)
        eos, ids = _eos_list(g.get("eos_token_id"))
        if ids:
            args.stop_token_ids = sorted(set(args.stop_token_ids) | set(ids))
            if args.eos_token_id < 0:
                args.eos_token_id = eos
    return args


# ---- named synthetic configurations used by the benchmarks and tests -------------------------
def preset(name: str) -> ModelArgs:
    n = name.lower()
    if n in ("tiny", "tiny-qwen3"):
        return ModelArgs(model_type="qwen3", vocab_size=32000, hidden_size=256, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                         intermediate_size=768, rms_norm_eps=1e-6, rope_theta=1e6,
                         tie_word_embeddings=True, max_position_embeddings=4096, dtype="float32")
    if n == "tiny-hd128":                                   # head_dim of the tensor-core attention kernels
        return ModelArgs(model_type="qwen3", vocab_size=32000, hidden_size=512, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                         intermediate_size=1024, rms_norm_eps=1e-6, rope_theta=1e6,
                         tie_word_embeddings=True, max_position_embeddings=4096, dtype="float32")
    if n in ("qwen3-8b",):
        return ModelArgs(model_type="qwen3", vocab_size=151936, hidden_size=4096, num_hidden_layers=36,
                         num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                         intermediate_size=12288, rope_theta=1e6, max_position_embeddings=40960)
    if n in ("qwen3-32b",):
        return ModelArgs(model_type="qwen3", vocab_size=151936, hidden_size=5120, num_hidden_layers=64,
                         num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                         intermediate_size=25600, rope_theta=1e6, max_position_embeddings=40960)
    if n in ("qwen3-30b-a3b",):
        return ModelArgs(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048, num_hidden_layers=48,
                         num_attention_heads=32, num_key_value_heads=4, head_dim=128,
                         intermediate_size=6144, num_experts=128, num_experts_per_tok=8,
                         moe_intermediate_size=768, norm_topk_prob=True, rope_theta=1e6,
                         max_position_embeddings=40960)
    if n in ("deepseek-v3",):
        return ModelArgs(model_type="deepseek_v3", vocab_size=129280, hidden_size=7168, num_hidden_layers=61,
                         num_attention_heads=128, num_key_value_heads=128, head_dim=192,
                         intermediate_size=18432, num_experts=256, num_experts_per_tok=8,
                         moe_intermediate_size=2048, n_shared_experts=1, first_k_dense_replace=3,
                         scoring_func="sigmoid", n_group=8, topk_group=4, routed_scaling_factor=2.5,
                         router_bias=True, q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
                         qk_rope_head_dim=64, v_head_dim=128, qk_norm=False, rope_theta=10000.0,
                         num_nextn_predict_layers=1, quant_method="fp8", quant_block=[128, 128],
                         max_position_embeddings=163840)
    raise KeyError(f"unknown preset {name}")
