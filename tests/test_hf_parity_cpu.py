"""Every decoder family against its HuggingFace implementation: a tiny random model is built with
`transformers`, saved as a checkpoint directory (config.json + safetensors), loaded by this
framework's config parser and safetensors reader, and run through the engine on CPU in fp32.  Greedy
continuations must be identical and the logits of a whole sequence must agree to 1e-4.  This pins
the config mapping, the checkpoint name mapping and the layer arithmetic of each family."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from xllm_b200 import LLM, SamplingParams  # noqa: E402
from xllm_b200.api.embedding import hidden_states  # noqa: E402

COMMON = dict(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              intermediate_size=128, max_position_embeddings=512, rms_norm_eps=1e-6, tie_word_embeddings=False)


def _case(fam):
    t = transformers
    if fam == "llama":
        return t.LlamaConfig(**COMMON, head_dim=16), t.LlamaForCausalLM
    if fam == "mistral":
        return t.MistralConfig(**COMMON, head_dim=16, sliding_window=None), t.MistralForCausalLM
    if fam == "qwen2":
        return t.Qwen2Config(**COMMON), t.Qwen2ForCausalLM
    if fam == "qwen3":
        return t.Qwen3Config(**COMMON, head_dim=32), t.Qwen3ForCausalLM
    if fam == "qwen3_moe":
        return t.Qwen3MoeConfig(**COMMON, head_dim=16, moe_intermediate_size=32, num_experts=8, num_experts_per_tok=2,
                                norm_topk_prob=True), t.Qwen3MoeForCausalLM
    if fam in ("deepseek_v3", "deepseek_v3_latent"):
        return t.DeepseekV3Config(**COMMON, moe_intermediate_size=32, n_routed_experts=8, num_experts_per_tok=2,
                                  n_shared_experts=1, first_k_dense_replace=1, n_group=2, topk_group=1, q_lora_rank=32,
                                  kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                                  routed_scaling_factor=2.5), t.DeepseekV3ForCausalLM
    if fam == "glm_moe_dsa":
        # index_topk far below the prompt lengths: every step takes the sparse path
        return t.GlmMoeDsaConfig(**dict(COMMON, num_key_value_heads=4), moe_intermediate_size=32, n_routed_experts=8, num_experts_per_tok=2,
                                 n_shared_experts=1, mlp_layer_types=["dense", "sparse"], n_group=1, topk_group=1,
                                 q_lora_rank=32, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                                 routed_scaling_factor=2.5, index_topk=6, index_head_dim=16, index_n_heads=4,
                                 pad_token_id=0), t.GlmMoeDsaForCausalLM
    if fam == "glm4":
        return t.Glm4Config(**COMMON, head_dim=16, partial_rotary_factor=0.5, pad_token_id=0), t.Glm4ForCausalLM
    if fam == "glm4_moe":
        return t.Glm4MoeConfig(**COMMON, head_dim=16, partial_rotary_factor=0.5, moe_intermediate_size=32,
                               n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1, first_k_dense_replace=1,
                               n_group=1, topk_group=1, use_qk_norm=True, routed_scaling_factor=1.5), t.Glm4MoeForCausalLM
    if fam == "minimax_m2":
        return t.MiniMaxM2Config(**COMMON, head_dim=16, num_local_experts=8, num_experts_per_tok=2,
                                 rope_parameters={"rope_theta": 10000.0, "rope_type": "default",
                                                  "partial_rotary_factor": 0.5}), t.MiniMaxM2ForCausalLM
    raise KeyError(fam)


FAMILIES = ["llama", "mistral", "qwen2", "qwen3", "qwen3_moe", "deepseek_v3", "deepseek_v3_latent", "glm4", "glm4_moe",
            "minimax_m2", "glm_moe_dsa"]


@pytest.mark.parametrize("fam", FAMILIES)
def test_family_matches_huggingface(fam, tmp_path):
    try:
        cfg, cls = _case(fam)
    except (AttributeError, TypeError) as e:      # this transformers build lacks the family
        pytest.skip(str(e))
    torch.manual_seed(0)
    if fam == "glm_moe_dsa":
        # the oracle must build its causal mask explicitly: with the fused-attention back end this family's
        # indexer receives no mask at all and selects (and attends to) future tokens
        cfg._attn_implementation = "eager"
    hf = cls(cfg).float().eval()
    with torch.no_grad():                         # norms away from 1 and biases away from 0, so that both matter
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.copy_(1 + 0.1 * torch.randn_like(p))
            elif n.endswith("bias"):
                p.copy_(0.1 * torch.randn_like(p))
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (9, 21, 33)]
    llm = LLM(str(tmp_path), devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
              max_tokens_per_batch=256, enable_graph=False, mla_latent_cache=fam.endswith("_latent"))
    if fam.endswith("_latent"):                   # one shared row of kv_lora_rank + rope values per token
        k0, v0 = llm.engine.runner.kv_caches[0]
        assert k0.shape[1:] == (1, 16, 16 + 8) and v0.data_ptr() == k0.data_ptr()
    outs = llm.generate(prompts, SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True))
    for p, o in zip(prompts, outs):
        with torch.no_grad():
            ref = hf.generate(torch.tensor([p]), max_new_tokens=10, do_sample=False, eos_token_id=None,
                              pad_token_id=0)[0, len(p):].tolist()
        assert o.outputs[0].token_ids == ref
    seq = prompts[2] + outs[2].outputs[0].token_ids
    ours = llm.engine.model.logits(hidden_states(llm.engine, seq)).float()
    with torch.no_grad():
        ref = hf(torch.tensor([seq])).logits[0]
    assert float((ours - ref).abs().max()) < 1e-4


@pytest.mark.parametrize("fam", ["qwen2_vl", "qwen2_5_vl"])
def test_vision_language_model_matches_huggingface(fam, tmp_path):
    """Vision tower, merger, prompt expansion, 3-axis rotary positions and the decoder against
    HuggingFace, from a saved checkpoint directory and a random image."""
    import numpy as np
    from xllm_b200.api.vlm import VLM
    from xllm_b200.multimodal import Qwen2VLImageProcessor
    t = transformers
    IMG, VSTART, VEND = 500, 501, 502
    text = dict(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                intermediate_size=128, max_position_embeddings=512, rms_norm_eps=1e-6, tie_word_embeddings=False,
                rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]})
    torch.manual_seed(0)
    if fam == "qwen2_vl":
        vis = dict(depth=2, embed_dim=32, hidden_size=64, num_heads=2, mlp_ratio=2, patch_size=14, spatial_merge_size=2,
                   temporal_patch_size=2, in_channels=3)
        cfg = t.Qwen2VLConfig(text_config=text, vision_config=vis, image_token_id=IMG, vision_start_token_id=VSTART,
                              vision_end_token_id=VEND, video_token_id=503)
        hf = t.Qwen2VLForConditionalGeneration(cfg)
    else:
        vis = dict(depth=2, hidden_size=32, out_hidden_size=64, intermediate_size=48, num_heads=2, patch_size=14,
                   spatial_merge_size=2, temporal_patch_size=2, in_channels=3, window_size=56, fullatt_block_indexes=[1])
        cfg = t.Qwen2_5_VLConfig(text_config=text, vision_config=vis, image_token_id=IMG, vision_start_token_id=VSTART,
                                 vision_end_token_id=VEND, video_token_id=503)
        hf = t.Qwen2_5_VLForConditionalGeneration(cfg)
    hf = hf.float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n and p.dim() == 1 and not n.endswith("bias"):
                p.copy_(1 + 0.1 * torch.randn_like(p))
            elif n.endswith("bias"):
                p.copy_(0.1 * torch.randn_like(p))
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    vlm = VLM(str(tmp_path), devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
              max_tokens_per_batch=64, enable_graph=False)
    vlm.processor = Qwen2VLImageProcessor(14, 2, 2, min_pixels=56 * 56, max_pixels=140 * 140)
    img = (np.random.default_rng(1).random((120, 150, 3)) * 255).astype(np.uint8)
    prompt = [11, 12, VSTART, IMG, VEND, 13, 14, 15]
    ids, mm = vlm.prepare(prompt, [img])
    pv, grid = vlm.processor([img])
    with torch.no_grad():
        ref = hf.generate(input_ids=torch.tensor([ids]), pixel_values=pv, image_grid_thw=grid, max_new_tokens=8,
                          do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(ids):].tolist()
        hv = hf.model.visual(pv, grid_thw=grid)
        hv = hv.pooler_output if hasattr(hv, "pooler_output") else hv
    assert float((hv - mm.embeds).abs().max()) < 1e-4
    got = vlm.generate_mm([dict(prompt_token_ids=prompt, images=[img])],
                          SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))[0]
    assert got == ref


def test_qwen3_next_hybrid_matches_huggingface(tmp_path):
    """Gated-delta-net layers (convolution tail + recurrent state per request), gated full attention,
    zero-centred norms and the gated shared expert against HuggingFace; prompts are prefilled in
    chunks so that the states carry over between steps, and several requests decode together."""
    t = transformers
    if not hasattr(t, "Qwen3NextForCausalLM"):
        pytest.skip("no Qwen3-Next in this transformers build")
    cfg = t.Qwen3NextConfig(vocab_size=512, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                            head_dim=32, intermediate_size=128, max_position_embeddings=512, rms_norm_eps=1e-6,
                            tie_word_embeddings=False, linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16,
                            linear_value_head_dim=16, linear_conv_kernel_dim=4, num_experts=8, num_experts_per_tok=2,
                            moe_intermediate_size=32, shared_expert_intermediate_size=48, norm_topk_prob=True,
                            decoder_sparse_step=1, mlp_only_layers=[], full_attention_interval=4)
    torch.manual_seed(0)
    hf = t.Qwen3NextForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("layernorm.weight") or n.endswith("model.norm.weight") or n.endswith("_norm.weight"):
                p.copy_(0.1 * torch.randn_like(p))
            elif n.endswith("linear_attn.norm.weight"):
                p.copy_(1 + 0.1 * torch.randn_like(p))
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (9, 40, 23)]
    llm = LLM(str(tmp_path), devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
              max_tokens_per_batch=24, enable_graph=False)
    assert llm.engine.model.needs_state
    outs = llm.generate(prompts, SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True))
    for p, o in zip(prompts, outs):
        with torch.no_grad():
            ref = hf.generate(torch.tensor([p]), max_new_tokens=10, do_sample=False, eos_token_id=None,
                              pad_token_id=0)[0, len(p):].tolist()
        assert o.outputs[0].token_ids == ref
    assert not llm.engine.model.state.owner               # every slot was given back


@pytest.mark.parametrize("moe", [False, True])
def test_qwen3_vl_matches_huggingface(moe, tmp_path):
    """Qwen3-VL: interpolated position table, deepstack features added after the first decoder
    layers, interleaved 3-axis rotary embedding, q/k norms; with the dense or the MoE decoder (whose
    checkpoints keep a layer's experts in two fused tensors)."""
    import numpy as np
    from xllm_b200.api.vlm import VLM
    from xllm_b200.multimodal import Qwen2VLImageProcessor
    t = transformers
    if not hasattr(t, "Qwen3VLForConditionalGeneration"):
        pytest.skip("no Qwen3-VL in this transformers build")
    IMG, VSTART, VEND = 500, 501, 502
    text = dict(vocab_size=512, hidden_size=64, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                intermediate_size=128, max_position_embeddings=512, rms_norm_eps=1e-6, tie_word_embeddings=False,
                rope_scaling={"rope_type": "default", "mrope_section": [2, 3, 3], "mrope_interleaved": True})
    vis = dict(depth=3, hidden_size=32, out_hidden_size=64, intermediate_size=48, num_heads=2, patch_size=16, spatial_merge_size=2,
               temporal_patch_size=2, in_channels=3, num_position_embeddings=36, deepstack_visual_indexes=[0, 2])
    torch.manual_seed(0)
    if moe:
        if not hasattr(t, "Qwen3VLMoeForConditionalGeneration"):
            pytest.skip("no Qwen3-VL-MoE in this transformers build")
        text.update(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32, decoder_sparse_step=1, mlp_only_layers=[])
        cfg = t.Qwen3VLMoeConfig(text_config=text, vision_config=vis, image_token_id=IMG, vision_start_token_id=VSTART,
                                 vision_end_token_id=VEND, video_token_id=503)
        hf = t.Qwen3VLMoeForConditionalGeneration(cfg).float().eval()
    else:
        cfg = t.Qwen3VLConfig(text_config=text, vision_config=vis, image_token_id=IMG, vision_start_token_id=VSTART,
                              vision_end_token_id=VEND, video_token_id=503)
        hf = t.Qwen3VLForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n and p.dim() == 1 and not n.endswith("bias"):
                p.copy_(1 + 0.1 * torch.randn_like(p))
            elif n.endswith("bias"):
                p.copy_(0.1 * torch.randn_like(p))
            elif "pos_embed" in n:
                p.copy_(0.2 * torch.randn_like(p))
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    vlm = VLM(str(tmp_path), devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
              max_tokens_per_batch=32, enable_graph=False)
    vlm.processor = Qwen2VLImageProcessor(16, 2, 2, min_pixels=64 * 64, max_pixels=160 * 160)
    img = (np.random.default_rng(1).random((120, 150, 3)) * 255).astype(np.uint8)
    prompt = [11, 12, VSTART, IMG, VEND, 13, 14, 15]
    ids, mm = vlm.prepare(prompt, [img])
    pv, grid = vlm.processor([img])
    with torch.no_grad():
        kinds = torch.tensor([[1 if i == IMG else 0 for i in ids]])      # which prompt tokens are image placeholders
        ref = hf.generate(input_ids=torch.tensor([ids]), pixel_values=pv, image_grid_thw=grid, mm_token_type_ids=kinds,
                          max_new_tokens=8, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(ids):].tolist()
        hv = hf.model.visual(pv, grid_thw=grid)
    assert float((hv.pooler_output - mm.embeds[:, :64]).abs().max()) < 1e-4
    assert float((hv.deepstack_features[1] - mm.embeds[:, 128:192]).abs().max()) < 1e-4
    got = vlm.generate_mm([dict(prompt_token_ids=prompt, images=[img])],
                          SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))[0]
    assert got == ref


@pytest.mark.parametrize("moe", [False, True])
def test_qwen3_5_text_matches_huggingface(moe, tmp_path):
    """Qwen3.5 text decoder: the gated-delta-net layers with four separate input projections, a dense
    MLP or the MoE with a gated shared expert, every fourth layer gated full attention."""
    t = transformers
    if not hasattr(t, "Qwen3_5ForCausalLM") or not hasattr(t, "Qwen3_5MoeForCausalLM"):
        pytest.skip("no Qwen3.5 in this transformers build")
    common = dict(vocab_size=512, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                  head_dim=32, max_position_embeddings=512, rms_norm_eps=1e-6, tie_word_embeddings=False,
                  linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=16,
                  linear_conv_kernel_dim=4)
    torch.manual_seed(0)
    if moe:
        cfg = t.Qwen3_5MoeTextConfig(**common, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                                     shared_expert_intermediate_size=48)
        hf = t.Qwen3_5MoeForCausalLM(cfg).float().eval()
    else:
        cfg = t.Qwen3_5TextConfig(**common, intermediate_size=128)
        hf = t.Qwen3_5ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("layernorm.weight") or n.endswith("model.norm.weight") or n.endswith("_norm.weight"):
                p.copy_(0.1 * torch.randn_like(p))
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (9, 40, 23)]
    llm = LLM(str(tmp_path), devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
              max_tokens_per_batch=24, enable_graph=False)
    outs = llm.generate(prompts, SamplingParams(max_tokens=10, temperature=0.0, ignore_eos=True))
    for p, o in zip(prompts, outs):
        with torch.no_grad():
            ref = hf.generate(torch.tensor([p]), max_new_tokens=10, do_sample=False, eos_token_id=None,
                              pad_token_id=0)[0, len(p):].tolist()
        assert o.outputs[0].token_ids == ref


def test_qwen3_5_vision_language_matches_huggingface(tmp_path):
    """Qwen3.5 with images: hybrid decoder (state slots) + vision tower + interleaved M-RoPE on the
    full-attention layers, prompt prefilled in two chunks."""
    import numpy as np
    from xllm_b200.api.vlm import VLM
    from xllm_b200.multimodal import Qwen2VLImageProcessor
    t = transformers
    if not hasattr(t, "Qwen3_5ForConditionalGeneration"):
        pytest.skip("no Qwen3.5 in this transformers build")
    IMG, VSTART, VEND = 500, 501, 502
    text = dict(vocab_size=512, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                intermediate_size=128, max_position_embeddings=512, rms_norm_eps=1e-6, tie_word_embeddings=False,
                linear_num_value_heads=4, linear_num_key_heads=2, linear_key_head_dim=16, linear_value_head_dim=16,
                linear_conv_kernel_dim=4,
                rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.25,
                                 "mrope_section": [2, 3, 3], "mrope_interleaved": True})
    vis = dict(depth=2, hidden_size=32, out_hidden_size=64, intermediate_size=48, num_heads=2, patch_size=16, spatial_merge_size=2,
               temporal_patch_size=2, in_channels=3, num_position_embeddings=36)
    cfg = t.Qwen3_5Config(text_config=text, vision_config=vis, image_token_id=IMG, vision_start_token_id=VSTART,
                          vision_end_token_id=VEND, video_token_id=503)
    torch.manual_seed(0)
    hf = t.Qwen3_5ForConditionalGeneration(cfg).float().eval()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    vlm = VLM(str(tmp_path), devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
              max_tokens_per_batch=16, enable_graph=False)
    vlm.processor = Qwen2VLImageProcessor(16, 2, 2, min_pixels=64 * 64, max_pixels=160 * 160)
    img = (np.random.default_rng(1).random((120, 150, 3)) * 255).astype(np.uint8)
    prompt = [11, 12, VSTART, IMG, VEND, 13, 14, 15]
    ids, mm = vlm.prepare(prompt, [img])
    pv, grid = vlm.processor([img])
    with torch.no_grad():
        kinds = torch.tensor([[1 if i == IMG else 0 for i in ids]])
        ref = hf.generate(input_ids=torch.tensor([ids]), pixel_values=pv, image_grid_thw=grid, mm_token_type_ids=kinds,
                          max_new_tokens=8, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(ids):].tolist()
    got = vlm.generate_mm([dict(prompt_token_ids=prompt, images=[img])],
                          SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))[0]
    assert got == ref


def test_glm4v_matches_huggingface(tmp_path):
    """GLM-4V: learned position embeddings resampled bicubically per image, RMSNorm / SwiGLU vision blocks,
    strided-convolution downsample and gated merger, in front of the GLM-4 decoder with contiguous M-RoPE
    sections over the rotated half of each head; the prompt is prefilled in chunks."""
    import numpy as np
    from xllm_b200.api.vlm import VLM
    from xllm_b200.multimodal import Glm4vImageProcessor
    t = transformers
    if not hasattr(t, "Glm4vForConditionalGeneration"):
        pytest.skip("no GLM-4V in this transformers build")
    IMG, ISTART, IEND = 500, 501, 502
    text = dict(vocab_size=512, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                intermediate_size=128, max_position_embeddings=512, rms_norm_eps=1e-5, tie_word_embeddings=False,
                attention_bias=True,
                rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5,
                                 "mrope_section": [2, 3, 3]})
    vis = dict(depth=2, hidden_size=32, out_hidden_size=128, intermediate_size=48, num_heads=2, patch_size=14, spatial_merge_size=2,
               temporal_patch_size=2, in_channels=3, image_size=84, rms_norm_eps=1e-5)
    cfg = t.Glm4vConfig(text_config=text, vision_config=vis, image_token_id=IMG, video_token_id=503, image_start_token_id=ISTART,
                        image_end_token_id=IEND, video_start_token_id=504, video_end_token_id=505)
    torch.manual_seed(0)
    hf = t.Glm4vForConditionalGeneration(cfg).float().eval()
    hf.save_pretrained(str(tmp_path), safe_serialization=True)
    vlm = VLM(str(tmp_path), devices="cpu", dtype="float32", block_size=16, num_blocks=64, max_seqs_per_batch=8,
              max_tokens_per_batch=16, enable_graph=False, processor=Glm4vImageProcessor(14, 2, 2))
    img = (np.random.default_rng(3).random((100, 130, 3)) * 255).astype(np.uint8)
    prompt = [11, 12, ISTART, IMG, IEND, 13, 14, 15]
    ids, mm = vlm.prepare(prompt, [img])
    pv, grid = vlm.processor([img])
    with torch.no_grad():
        feats = hf.get_image_features(pv, grid)
        feats = feats.pooler_output if hasattr(feats, "pooler_output") else feats
        feats = torch.cat(list(feats)) if isinstance(feats, (list, tuple)) else feats
        assert (mm.embeds - feats).abs().max() < 1e-4                      # the tower alone
        kinds = torch.tensor([[1 if i == IMG else 0 for i in ids]])
        ref = hf.generate(input_ids=torch.tensor([ids]), pixel_values=pv, image_grid_thw=grid, mm_token_type_ids=kinds,
                          max_new_tokens=7, do_sample=False, eos_token_id=None, pad_token_id=0)[0, len(ids):].tolist()
    got = vlm.generate_mm([dict(prompt_token_ids=prompt, images=[img])],
                          SamplingParams(max_tokens=7, temperature=0.0, ignore_eos=True))[0]
    assert got == ref            # (the eighth token is a tie to 8e-4 in this random model)
