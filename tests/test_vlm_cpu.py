"""Qwen2-VL-style model on CPU: image processor, prompt expansion, M-RoPE positions, and the engine
path (image embeddings merged at prefill, 3-axis rotary table, chunked prefill, paged decode)
against a dense textbook forward."""
import math

import numpy as np
import torch

from xllm_b200.api.vlm import VLM
from xllm_b200.api.llm import SamplingParams
from xllm_b200.engine.llm_engine import EngineConfig, LLMEngine
from xllm_b200.models import ModelArgs
from xllm_b200.multimodal import Qwen2VLImageProcessor, expand_image_tokens, mrope_positions, smart_resize

IMG, VSTART, VEND = 900, 901, 902


def _args(head_dim=16, hidden=64, sections=(2, 3, 3)):
    return ModelArgs(model_type="qwen2_vl", vocab_size=1000, hidden_size=hidden, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=head_dim, intermediate_size=128, qk_norm=False, attention_bias=True,
                     rope_theta=10000.0, max_position_embeddings=512, tie_word_embeddings=False, image_token_id=IMG,
                     vision_start_token_id=VSTART, mrope_section=list(sections),
                     vision_config=dict(embed_dim=32, num_heads=2, depth=2, mlp_ratio=2, patch_size=14,
                                        spatial_merge_size=2, temporal_patch_size=2, in_chans=3))


def test_processor_and_positions():
    assert smart_resize(100, 200, 28, 56 * 56, 10 ** 6) == (112, 196)
    proc = Qwen2VLImageProcessor()
    img = (np.random.default_rng(0).random((60, 90, 3)) * 255).astype(np.uint8)
    pv, grid = proc([img])
    h, w = smart_resize(60, 90, 28, 56 * 56, proc.max_pixels)
    assert grid.tolist() == [[1, h // 14, w // 14]] and pv.shape == ((h // 14) * (w // 14), 3 * 2 * 14 * 14)
    n = proc.tokens_per_image(grid)[0]
    ids = expand_image_tokens([5, VSTART, IMG, VEND, 6, 7], IMG, [n])
    assert ids.count(IMG) == n and len(ids) == 5 + n
    pos, delta = mrope_positions(ids, IMG, grid, 2)
    gh, gw = grid[0, 1].item() // 2, grid[0, 2].item() // 2
    assert pos[:, 0].tolist() == [0, 0, 0] and pos[:, 1].tolist() == [1, 1, 1]
    assert pos[0, 2:2 + n].unique().tolist() == [2]                       # one temporal position for a still image
    assert pos[1, 2:2 + n].max().item() == 2 + gh - 1 and pos[2, 2:2 + n].max().item() == 2 + gw - 1
    nxt = 2 + max(gh, gw)
    assert pos[:, 2 + n].tolist() == [nxt] * 3 and delta == (nxt + 3) - len(ids)


def _dense_reference(model, ids, embeds_rows, embeds_vals, pos3):
    """Textbook forward over the whole sequence: merged embeddings, M-RoPE, causal attention."""
    a = model.args
    sd = dict(model.named_params())
    x = sd["model.embed_tokens.weight"][ids].clone()
    x[embeds_rows] = embeds_vals
    T = ids.shape[0]
    d, nq, nkv = a.head_dim, a.num_attention_heads, a.num_key_value_heads
    half = d // 2
    inv = 1.0 / (a.rope_theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / d))
    axis = torch.repeat_interleave(torch.arange(3), torch.tensor(model.mrope_section))
    ang = (pos3.double()[axis] * inv[:, None]).T
    cos, sin = ang.cos().float()[:, None, :], ang.sin().float()[:, None, :]

    def norm(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + a.rms_norm_eps) * w

    def rope(v):
        v1, v2 = v[..., :half], v[..., half:]
        return torch.cat([v1 * cos - v2 * sin, v2 * cos + v1 * sin], -1)

    for i in range(a.num_hidden_layers):
        p = f"model.layers.{i}."
        h = norm(x, sd[p + "input_layernorm.weight"])
        qkv = h @ sd[p + "self_attn.qkv_proj.weight"].T + sd[p + "self_attn.qkv_proj.bias"]
        q, k, v = qkv.split([nq * d, nkv * d, nkv * d], -1)
        q, k, v = rope(q.view(T, nq, d)), rope(k.view(T, nkv, d)), v.view(T, nkv, d)
        k, v = k.repeat_interleave(nq // nkv, 1), v.repeat_interleave(nq // nkv, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(d)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(T, nq * d)
        x = x + o @ sd[p + "self_attn.o_proj.weight"].T
        h = norm(x, sd[p + "post_attention_layernorm.weight"])
        g, u = (h @ sd[p + "mlp.gate_up_proj.weight"].T).chunk(2, -1)
        x = x + (torch.nn.functional.silu(g) * u) @ sd[p + "mlp.down_proj.weight"].T
    return norm(x, sd["model.norm.weight"]) @ sd["lm_head.weight"].T


def test_vlm_engine_matches_dense_reference():
    vlm = VLM.__new__(VLM)
    vlm.engine = LLMEngine(EngineConfig(model="v", device="cpu", dtype="float32", num_blocks=64, enable_graph=False,
                                        max_tokens_per_batch=16, enable_schedule_overlap=False), model_args=_args())   # prompts span chunks
    vlm.tokenizer = None
    model = vlm.engine.model
    model.init_random(std=0.05, seed=3)
    vlm.processor = Qwen2VLImageProcessor(14, 2, 2, min_pixels=56 * 56, max_pixels=112 * 112)
    vlm.image_token_id = IMG
    rng = np.random.default_rng(1)
    img_a = (rng.random((80, 100, 3)) * 255).astype(np.uint8)
    img_b = (rng.random((56, 56, 3)) * 255).astype(np.uint8)
    reqs = [dict(prompt_token_ids=[11, 12, VSTART, IMG, VEND, 13, 14, 15], images=[img_a]),
            dict(prompt_token_ids=[21, 22, 23, 24], images=[]),
            dict(prompt_token_ids=[31, VSTART, IMG, VEND, 32, VSTART, IMG, VEND, 33], images=[img_b, img_a])]
    got = vlm.generate_mm(reqs, SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True))
    for r, g in zip(reqs, got):
        ids, mm = vlm.prepare(r["prompt_token_ids"], r["images"])
        seq = list(ids)
        for _ in range(5):
            L = len(seq)
            pos3 = torch.cat([mm.mrope, (torch.arange(mm.mrope.shape[1], L) + mm.delta).repeat(3, 1)], dim=1)
            rows = torch.tensor(mm.positions, dtype=torch.long)
            logits = _dense_reference(model, torch.tensor(seq), rows, mm.embeds, pos3)
            seq.append(int(logits[-1].argmax()))
        assert g == seq[len(ids):], (g, seq[len(ids):])
    assert not vlm.engine.mm


def test_vlm_engine_with_a_video_and_an_image_matches_dense_reference():
    VID = 903
    args = _args()
    args.video_token_id = VID
    vlm = VLM.__new__(VLM)
    vlm.engine = LLMEngine(EngineConfig(model="v", device="cpu", dtype="float32", num_blocks=64, enable_graph=False,
                                        max_tokens_per_batch=32, enable_schedule_overlap=False), model_args=args)
    vlm.tokenizer = None
    model = vlm.engine.model
    model.init_random(std=0.05, seed=5)
    vlm.processor = Qwen2VLImageProcessor(14, 2, 2, min_pixels=56 * 56, max_pixels=112 * 112)
    from xllm_b200.multimodal import Qwen2VLVideoProcessor
    vlm.video_processor = Qwen2VLVideoProcessor(14, 2, 2, min_pixels=56 * 56, max_pixels=84 * 84)
    vlm.image_token_id = IMG
    rng = np.random.default_rng(2)
    img = (rng.random((56, 84, 3)) * 255).astype(np.uint8)
    video = torch.from_numpy((rng.random((3, 3, 60, 60)) * 255).astype(np.uint8))     # 3 frames -> padded to 4
    req = dict(prompt_token_ids=[11, VSTART, VID, VEND, 12, VSTART, IMG, VEND, 13], images=[img], videos=[video])
    got = vlm.generate_mm([req], SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))[0]
    ids, mm = vlm.prepare(req["prompt_token_ids"], [img], [video])
    n_vid = sum(1 for t in ids if t == VID)
    n_img = sum(1 for t in ids if t == IMG)
    assert n_vid == 2 * 2 * 2 and n_img == 2 * 3 and mm.embeds.shape[0] == n_vid + n_img
    assert ids.index(VID) < ids.index(IMG) and mm.positions == [i for i, t in enumerate(ids) if t in (VID, IMG)]
    # the video's two frame groups sit at consecutive temporal positions, rows / columns restart per group
    v0 = ids.index(VID)
    assert mm.mrope[0, v0:v0 + 8].tolist() == [2] * 4 + [3] * 4 and mm.mrope[1, v0:v0 + 4].tolist() == [2, 2, 3, 3]
    seq = list(ids)
    for _ in range(4):
        L = len(seq)
        pos3 = torch.cat([mm.mrope, (torch.arange(mm.mrope.shape[1], L) + mm.delta).repeat(3, 1)], dim=1)
        logits = _dense_reference(model, torch.tensor(seq), torch.tensor(mm.positions), mm.embeds, pos3)
        seq.append(int(logits[-1].argmax()))
    assert got == seq[len(ids):]


def test_chat_route_takes_image_parts(tmp_path):
    """`/v1/chat/completions` with an image_url part (a data: URL): the server decodes the image, renders
    the placeholder through the chat template, runs the vision tower and generates; the same request
    without the image generates something else, and a text-only model refuses image parts."""
    import base64
    import http.client
    import io
    import json
    import threading

    from PIL import Image
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers

    from xllm_b200 import _rt
    from xllm_b200.api.server import ApiServer
    from xllm_b200.utils.tokenizer import TokenizerWrapper
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    tok.decoder = decoders.ByteLevel()
    specials = ["<|im_start|>", "<|im_end|>", "<|endoftext|>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>",
                "<|video_pad|>"]
    trainer = trainers.BpeTrainer(vocab_size=400, special_tokens=specials, initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(["describe this picture please user assistant system\n" * 5], trainer)
    path = tmp_path / "tokenizer.json"
    tok.save(str(path))
    impl = _rt.BpeTokenizer()
    impl.load_hf_file(str(path))
    wrapper = TokenizerWrapper(impl, "", {}, "qwen3")
    ids = {s: wrapper.encode(s)[0] for s in specials}
    args = _args()
    args.image_token_id, args.video_token_id = ids["<|image_pad|>"], ids["<|video_pad|>"]
    args.vision_start_token_id = ids["<|vision_start|>"]
    eng = LLMEngine(EngineConfig(model="v", device="cpu", dtype="float32", num_blocks=64, enable_graph=False,
                                 max_tokens_per_batch=64), model_args=args)
    eng.model.init_random(std=0.05, seed=3)
    srv = ApiServer(eng, wrapper, model_name="tiny-vl", host="127.0.0.1", port=0)
    t = threading.Thread(target=srv.serve_forever, args=(10,), daemon=True)
    t.start()

    def chat(content):
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=60)
        c.request("POST", "/v1/chat/completions", json.dumps({"messages": [{"role": "user", "content": content}],
                                                              "max_tokens": 6, "temperature": 0, "ignore_eos": True}),
                  {"Content-Type": "application/json"})
        r = c.getresponse()
        out = json.loads(r.read().decode())
        c.close()
        return r.status, out

    try:
        rng = np.random.default_rng(0)
        buf = io.BytesIO()
        Image.fromarray((rng.random((56, 84, 3)) * 255).astype(np.uint8)).save(buf, format="PNG")
        url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
        st, with_img = chat([{"type": "text", "text": "describe this picture"}, {"type": "image_url", "image_url": {"url": url}}])
        assert st == 200 and with_img["usage"]["completion_tokens"] == 6
        n_img_tokens = (56 // 14) * (84 // 14) // 4
        st, text_only = chat("describe this picture")
        assert st == 200
        assert with_img["usage"]["prompt_tokens"] == text_only["usage"]["prompt_tokens"] + n_img_tokens + 2
        st, again = chat([{"type": "text", "text": "describe this picture"}, {"type": "image_url", "image_url": {"url": url}}])
        assert again["choices"][0]["message"]["content"] == with_img["choices"][0]["message"]["content"]
        st, bad = chat([{"type": "image_url", "image_url": {"url": "https://example.com/x.png"}}])
        assert st == 400 and "data:" in bad["error"]["message"]
        st, bad = chat([{"type": "image_url", "image_url": {"url": "data:image/png;base64,AAAA"}}])
        assert st == 400
        assert not eng.mm
    finally:
        srv.shutdown()
        t.join(timeout=5)


def test_oxygenvlm_runs_the_glm4v_tower_in_front_of_a_qwen3_decoder():
    """`oxygenvlm`: image request through the engine equals the dense reference; `oxygenvlm_text` is the
    decoder alone under the same registry."""
    from xllm_b200.models.registry import create_model
    from xllm_b200.multimodal import Glm4vImageProcessor
    args = ModelArgs(model_type="oxygenvlm", vocab_size=1000, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=16, intermediate_size=128, qk_norm=False, attention_bias=True, rope_theta=10000.0,
                     max_position_embeddings=512, tie_word_embeddings=False, image_token_id=IMG, vision_start_token_id=VSTART,
                     mrope_section=[2, 3, 3],
                     vision_config=dict(hidden_size=32, out_hidden_size=64, intermediate_size=48, num_heads=2, depth=2,
                                        patch_size=14, spatial_merge_size=2, temporal_patch_size=2, in_channels=3,
                                        image_size=84))
    vlm = VLM.__new__(VLM)
    vlm.engine = LLMEngine(EngineConfig(model="o", device="cpu", dtype="float32", num_blocks=64, enable_graph=False,
                                        max_tokens_per_batch=16), model_args=args)
    vlm.tokenizer = None
    model = vlm.engine.model
    assert type(model).__name__ == "OxygenVLForConditionalGeneration" and type(model.visual).__name__ == "Glm4vVisionTower"
    model.init_random(std=0.05, seed=4)
    vlm.processor = Glm4vImageProcessor(14, 2, 2)
    vlm.image_token_id = IMG
    img = (np.random.default_rng(5).random((70, 98, 3)) * 255).astype(np.uint8)
    req = dict(prompt_token_ids=[11, VSTART, IMG, VEND, 12, 13], images=[img])
    got = vlm.generate_mm([req], SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))[0]
    ids, mm = vlm.prepare(req["prompt_token_ids"], [img])
    assert mm.embeds.shape == (sum(1 for t in ids if t == IMG), 64) and torch.isfinite(mm.embeds).all()
    seq = list(ids)
    for _ in range(4):
        L = len(seq)
        pos3 = torch.cat([mm.mrope, (torch.arange(mm.mrope.shape[1], L) + mm.delta).repeat(3, 1)], dim=1)
        logits = _dense_reference(model, torch.tensor(seq), torch.tensor(mm.positions), mm.embeds, pos3)
        seq.append(int(logits[-1].argmax()))
    assert got == seq[len(ids):]
    text_args = ModelArgs(**{**args.__dict__, "model_type": "oxygenvlm_text", "vision_config": None})
    text = create_model(text_args, torch.float32, "cpu")
    assert not hasattr(text, "visual") and text.mrope_section == [2, 3, 3]
