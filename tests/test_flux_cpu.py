"""Flux-family pipeline parts: rotary embedding against complex multiplication, AdaLN-Zero identity, packing,
the flow-matching scheduler against its closed form, CLIP and T5 text encoders against HuggingFace, the VAE
decoder's geometry and checkpoint names, and a tiny end-to-end run with a step cache."""
import math

import pytest
import torch

from xllm_b200.dit.flux import (FlowMatchEulerScheduler, FluxArgs, FluxPipeline, FluxTransformer, apply_rope, image_ids,
                                pack_latents, rope_cos_sin, timestep_embedding, unpack_latents)
from xllm_b200.dit.text_encoders import ClipTextEncoder, T5TextEncoder
from xllm_b200.dit.vae import VaeDecoder


def _tiny(guidance=True):
    return FluxArgs(in_channels=16, num_layers=2, num_single_layers=2, attention_head_dim=16, num_attention_heads=2,
                    joint_attention_dim=24, pooled_projection_dim=12, guidance_embeds=guidance, axes_dims_rope=(4, 6, 6))


def test_rope_is_a_complex_rotation_and_relative():
    ids = torch.tensor([[0, 0, 0], [0, 3, 5], [0, 7, 2]], dtype=torch.float32)
    cos, sin = rope_cos_sin(ids, (4, 6, 6))
    assert cos.shape == (3, 16)
    x = torch.randn(1, 2, 3, 16)
    got = apply_rope(x, cos[None, None], sin[None, None])
    z = torch.view_as_complex(x.reshape(1, 2, 3, 8, 2).contiguous())
    rot = torch.polar(torch.ones(3, 8), torch.atan2(sin[:, 0::2], cos[:, 0::2]))
    assert torch.allclose(got, torch.view_as_real(z * rot[None, None]).flatten(-2), atol=1e-5)
    # scores depend on position differences only
    q, k = torch.randn(1, 1, 1, 16), torch.randn(1, 1, 1, 16)
    def score(pq, pk):
        cq, sq = rope_cos_sin(torch.tensor([pq], dtype=torch.float32), (4, 6, 6))
        ck, sk = rope_cos_sin(torch.tensor([pk], dtype=torch.float32), (4, 6, 6))
        return float((apply_rope(q, cq, sq) * apply_rope(k, ck, sk)).sum())
    assert abs(score([0, 5, 9], [0, 2, 4]) - score([0, 13, 6], [0, 10, 1])) < 1e-4


def test_zero_modulation_makes_every_block_the_identity():
    m = FluxTransformer(_tiny())
    m.init_random(std=0.2, seed=1)
    for k in m.p:
        if ".norm1.linear" in k or ".norm1_context.linear" in k or ".norm.linear" in k:
            m.p[k].zero_()                                     # gates are zero: AdaLN-Zero at initialisation
    img, txt, temb = torch.randn(1, 6, 32), torch.randn(1, 3, 32), torch.randn(1, 32)
    cos, sin = rope_cos_sin(torch.cat([torch.zeros(3, 3), image_ids(4, 6)], 0), (4, 6, 6))
    i2, t2 = m.double_block(0, img, txt, temb, cos[None, None], sin[None, None])
    assert torch.equal(i2, img) and torch.equal(t2, txt)
    x = torch.randn(1, 9, 32)
    assert torch.equal(m.single_block(0, x, temb, cos[None, None], sin[None, None]), x)


def test_transformer_shapes_text_order_and_guidance():
    m = FluxTransformer(_tiny())
    m.init_random(std=0.1, seed=2)
    lat = pack_latents(torch.randn(2, 4, 4, 6))
    text, pooled, t = torch.randn(2, 5, 24), torch.randn(2, 12), torch.tensor([0.7, 0.2])
    ids_i, ids_t = image_ids(4, 6), torch.zeros(5, 3)
    g = torch.tensor([3.5, 3.5])
    out = m.forward(lat, text, pooled, t, ids_i, ids_t, g)
    assert out.shape == lat.shape and torch.isfinite(out).all()
    # text tokens all sit at position 0: the image output does not depend on their order
    perm = torch.tensor([3, 0, 4, 1, 2])
    assert torch.allclose(m.forward(lat, text[:, perm], pooled, t, ids_i, ids_t, g), out, atol=1e-4)
    # batch rows are independent, the guidance scale and the timestep matter
    assert torch.allclose(m.forward(lat[:1], text[:1], pooled[:1], t[:1], ids_i, ids_t, g[:1]), out[:1], atol=1e-4)
    assert not torch.allclose(m.forward(lat, text, pooled, t, ids_i, ids_t, g * 2), out, atol=1e-4)
    assert not torch.allclose(m.forward(lat, text, pooled, t * 0.5, ids_i, ids_t, g), out, atol=1e-4)
    e = timestep_embedding(torch.tensor([0.0, 500.0]))
    assert e.shape == (2, 256) and torch.allclose(e[0, :128], torch.ones(128)) and torch.allclose(e[0, 128:], torch.zeros(128))


def test_packing_scheduler_and_names():
    x = torch.randn(2, 16, 8, 12)
    p = pack_latents(x)
    assert p.shape == (2, 24, 64) and torch.equal(unpack_latents(p, 8, 12), x)
    assert torch.equal(p[0, 7], x[0, :, 2:4, 2:4].reshape(-1))                # token 7 = patch (row 1, column 1)
    assert image_ids(8, 12)[7].tolist() == [0.0, 1.0, 1.0]
    s = FlowMatchEulerScheduler()
    sig = s.set_timesteps(4, image_seq_len=4096)
    e = math.exp(1.15)
    assert abs(sig[0] - 1.0) < 1e-9 and abs(sig[-1] - e / (e + 3.0)) < 1e-9 and s.sigmas[-1] == 0.0
    assert abs(s.mu(256) - 0.5) < 1e-9 and abs(s.mu(4096) - 1.15) < 1e-9
    # with the exact velocity of a straight path, Euler steps land on the clean sample whatever the step count
    x0, noise = torch.randn(3, 5), torch.randn(3, 5)
    x = noise.clone()
    for i in range(4):
        x = s.step(noise - x0, i, x)
    assert torch.allclose(x, x0, atol=1e-5)
    names = set(FluxTransformer(FluxArgs(num_layers=1, num_single_layers=1, attention_head_dim=8, num_attention_heads=2,
                                         joint_attention_dim=8, pooled_projection_dim=8, axes_dims_rope=(2, 2, 4))).p)
    for n in ("x_embedder.weight", "context_embedder.bias", "time_text_embed.guidance_embedder.linear_2.weight",
              "time_text_embed.text_embedder.linear_1.weight", "transformer_blocks.0.norm1_context.linear.weight",
              "transformer_blocks.0.attn.add_k_proj.weight", "transformer_blocks.0.attn.norm_added_q.weight",
              "transformer_blocks.0.attn.to_add_out.bias", "transformer_blocks.0.ff_context.net.0.proj.weight",
              "single_transformer_blocks.0.proj_mlp.weight", "single_transformer_blocks.0.attn.norm_k.weight",
              "norm_out.linear.weight", "proj_out.bias"):
        assert n in names, n


def test_text_encoders_match_huggingface(tmp_path):
    t = pytest.importorskip("transformers")
    cfg = t.CLIPTextConfig(vocab_size=120, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                           max_position_embeddings=16, eos_token_id=2, bos_token_id=0, pad_token_id=1)
    torch.manual_seed(0)
    hf = t.CLIPTextModel(cfg).float().eval()
    (tmp_path / "clip").mkdir()
    hf.save_pretrained(str(tmp_path / "clip"), safe_serialization=True)
    mine = ClipTextEncoder.from_pretrained(str(tmp_path / "clip"))
    ids = torch.tensor([[0, 5, 9, 33, 119, 7, 7, 7], [0, 44, 119, 3, 3, 3, 3, 3]])     # 119: the largest id ends a prompt
    with torch.no_grad():
        want = hf(input_ids=ids)
    last, pooled = mine(ids)
    assert (last - want.last_hidden_state).abs().max() < 1e-4
    assert (pooled - want.pooler_output).abs().max() < 1e-4
    cfg5 = t.T5Config(vocab_size=100, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_heads=4, relative_attention_num_buckets=8,
                      relative_attention_max_distance=16, feed_forward_proj="gated-gelu", dropout_rate=0.0)
    hf5 = t.T5EncoderModel(cfg5).float().eval()
    (tmp_path / "t5").mkdir()
    hf5.save_pretrained(str(tmp_path / "t5"), safe_serialization=True)
    enc = T5TextEncoder.from_pretrained(str(tmp_path / "t5"))
    ids5 = torch.randint(2, 100, (2, 11))
    with torch.no_grad():
        want5 = hf5(input_ids=ids5).last_hidden_state
    assert (enc(ids5) - want5).abs().max() < 1e-4


def test_vae_decoder_geometry_and_pipeline_end_to_end():
    vae = VaeDecoder(latent_channels=4, block_out_channels=(8, 16, 16), layers_per_block=1, norm_groups=4)
    vae.init_random(seed=3)
    for n in ("decoder.conv_in.weight", "decoder.mid_block.attentions.0.to_q.weight", "decoder.mid_block.resnets.1.conv2.bias",
              "decoder.up_blocks.0.upsamplers.0.conv.weight", "decoder.up_blocks.2.resnets.0.conv_shortcut.weight",
              "decoder.conv_norm_out.weight", "decoder.conv_out.bias"):
        assert n in vae.p, n
    assert "decoder.up_blocks.2.upsamplers.0.conv.weight" not in vae.p          # the last block does not upsample
    img = vae.decode(torch.randn(1, 4, 6, 10))
    assert img.shape == (1, 3, 24, 40) and torch.isfinite(img).all()
    # pipeline: tiny stand-ins for the two text encoders
    tr = FluxTransformer(_tiny())
    tr.init_random(std=0.1, seed=4)
    clip = lambda ids: (None, torch.nn.functional.one_hot(ids[:, 0] % 12, 12).float())
    t5 = lambda ids: torch.nn.functional.one_hot(ids % 24, 24).float()
    pipe = FluxPipeline(tr, VaeDecoder(latent_channels=4, block_out_channels=(8, 8, 16, 16), layers_per_block=1, norm_groups=4), clip, t5,
                        latent_channels=4)
    pipe.vae.init_random(seed=5)
    ids = torch.tensor([[3, 4, 5, 6]])
    a = pipe(ids, ids, height=32, width=48, steps=4, seed=1)
    b = pipe(ids, ids, height=32, width=48, steps=4, seed=1)
    c = pipe(ids, ids, height=32, width=48, steps=4, seed=2)
    assert a.shape == (1, 3, 32, 48) and torch.equal(a, b) and not torch.equal(a, c) and a.abs().max() <= 1.0
    with pytest.raises(ValueError):
        pipe(ids, ids, height=30, width=48)
    # a step cache skips the blocks after the first on some steps and stays close to the exact result
    from xllm_b200.dit.cache import make_cache
    calls = {"n": 0}
    orig = tr.single_block
    tr.single_block = lambda *a_, **k_: (calls.__setitem__("n", calls["n"] + 1), orig(*a_, **k_))[1]
    exact = pipe(ids, ids, height=32, width=48, steps=8, seed=1)
    n_exact = calls["n"]
    calls["n"] = 0
    cached = pipe(ids, ids, height=32, width=48, steps=8, seed=1, cache=make_cache("residual", skip_interval=2, warmup=1))
    assert calls["n"] < n_exact and (cached - exact).abs().mean() < 0.2


def _write_flux_checkpoint(root):
    """A tiny checkpoint directory in the layout of the public releases."""
    import json

    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    import transformers as t
    from xllm_b200.utils.loader import save_file
    args = FluxArgs(in_channels=16, num_layers=1, num_single_layers=1, attention_head_dim=16, num_attention_heads=2,
                    joint_attention_dim=32, pooled_projection_dim=32, guidance_embeds=True, axes_dims_rope=(4, 6, 6))
    tr = FluxTransformer(args)
    tr.init_random(std=0.1, seed=7)
    (root / "transformer").mkdir(parents=True)
    (root / "transformer" / "config.json").write_text(json.dumps({**{k: getattr(args, k) for k in args.__dataclass_fields__},
                                                                   "axes_dims_rope": list(args.axes_dims_rope)}))
    save_file({k: v.contiguous() for k, v in tr.p.items()}, str(root / "transformer" / "diffusion_pytorch_model.safetensors"))
    vae = VaeDecoder(latent_channels=4, block_out_channels=(8, 8, 16, 16), layers_per_block=1, norm_groups=4)
    vae.init_random(seed=8)
    (root / "vae").mkdir()
    (root / "vae" / "config.json").write_text(json.dumps({"latent_channels": 4, "block_out_channels": [8, 8, 16, 16], "layers_per_block": 1,
                                                          "norm_num_groups": 4, "scaling_factor": 0.3611, "shift_factor": 0.1159}))
    save_file({k: v.contiguous() for k, v in vae.p.items()}, str(root / "vae" / "diffusion_pytorch_model.safetensors"))
    torch.manual_seed(0)
    t.CLIPTextModel(t.CLIPTextConfig(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                                     max_position_embeddings=16, eos_token_id=2, bos_token_id=0, pad_token_id=1)
                    ).save_pretrained(str(root / "text_encoder"), safe_serialization=True)
    t.T5EncoderModel(t.T5Config(vocab_size=300, d_model=32, d_kv=8, d_ff=64, num_layers=1, num_heads=4, relative_attention_num_buckets=8,
                                relative_attention_max_distance=16, feed_forward_proj="gated-gelu", dropout_rate=0.0)
                     ).save_pretrained(str(root / "text_encoder_2"), safe_serialization=True)
    for sub in ("tokenizer", "tokenizer_2"):
        tok = Tokenizer(models.BPE())
        tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
        tok.decoder = decoders.ByteLevel()
        tok.train_from_iterator(["a photo of a small red house by the sea at dusk " * 4],
                                trainers.BpeTrainer(vocab_size=290, special_tokens=["<s>", "<pad>", "</s>"],
                                                    initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
        (root / sub).mkdir()
        tok.save(str(root / sub / "tokenizer.json"))
    (root / "model_index.json").write_text(json.dumps({"_class_name": "FluxPipeline"}))


def test_flux_checkpoint_directory_and_image_route(tmp_path):
    import base64
    import http.client
    import json
    import threading
    import zlib

    from xllm_b200.api.server import ApiServer
    from xllm_b200.dit.pipeline import FluxImagePipeline
    from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
    _write_flux_checkpoint(tmp_path / "flux")
    pipe = FluxImagePipeline.from_pretrained(str(tmp_path / "flux"), steps=3)
    assert pipe.pipe.transformer.args.num_layers == 1 and pipe.clip_len == 16
    a = pipe.generate("a red house", size="32x48", seed=5)
    b = pipe.generate("a red house", size="32x48", seed=5)
    c = pipe.generate("the sea at dusk", size="32x48", seed=5)
    assert a[0].shape == (48, 32, 3) and (a[0] == b[0]).all() and (a[0] != c[0]).any()       # the prompt matters
    eng = LLMEngine(EngineConfig(model="tiny", device="cpu", dtype="float32", num_blocks=16, enable_graph=False))
    srv = ApiServer(eng, None, model_name="flux-tiny", host="127.0.0.1", port=0, backend="dit")
    srv.image_pipeline = pipe
    t = threading.Thread(target=srv.serve_forever, args=(10,), daemon=True)
    t.start()
    try:
        conn = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=120)
        conn.request("POST", "/v1/images/generations", json.dumps({"prompt": "a red house", "size": "32x32", "n": 2, "seed": 1,
                                                                    "num_inference_steps": 2}), {"Content-Type": "application/json"})
        r = conn.getresponse()
        out = json.loads(r.read().decode())
        assert r.status == 200 and len(out["data"]) == 2
        png = base64.b64decode(out["data"][0]["b64_json"])
        assert png[:8] == b"\x89PNG\r\n\x1a\n" and int.from_bytes(png[16:20], "big") == 32 and int.from_bytes(png[20:24], "big") == 32
        conn.request("POST", "/v1/images/generations", json.dumps({"prompt": "x", "size": "30x32"}), {"Content-Type": "application/json"})
        r = conn.getresponse()
        r.read()
        assert r.status == 400
        conn.close()
    finally:
        srv.shutdown()
        t.join(timeout=5)
