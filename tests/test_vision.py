"""Images in prompts: preprocessing, the vision tower, image tokens in the engine (rows, rotary positions, prefix
keys, row cache), mmproj round trip. CPU (fp32)."""
import io

import pytest
import torch

from legion_b200.config import ModelConfig
from legion_b200.engine.lm import EngineConfig, build_engine
from legion_b200.engine.types import ChatMessage, GenerateRequest, SamplingParams
from legion_b200.models.weights import random_weights
from legion_b200.vision import (VisionConfig, VisionHparams, VisionRuntime, VisionTower, decode_image, expand_image_tokens,
                                mrope_positions, preprocess, random_vision_weights)
from legion_b200.vision.media import mrope_axis_of_freq
from legion_b200.vision.preprocess import VisionError, smart_size


def png(w, h, color=(200, 30, 40), fmt="PNG"):
    from PIL import Image
    im = Image.new("RGB", (w, h), color)
    for x in range(0, w, 7):                      # some structure, so that rows differ between patches
        for y in range(0, h, 5):
            im.putpixel((x, y), ((x * 3) % 256, (y * 5) % 256, (x + y) % 256))
    buf = io.BytesIO()
    im.save(buf, fmt)
    return buf.getvalue()


def test_smart_size_and_patches_in_merge_order():
    hp = VisionHparams(patch_size=4, spatial_merge_size=2, temporal_patch_size=2, min_tokens=2, max_tokens=64)
    h, w = smart_size(60, 100, 8, hp.image_min_pixels, hp.image_max_pixels)
    assert h % 8 == 0 and w % 8 == 0 and hp.image_min_pixels <= h * w <= hp.image_max_pixels
    with pytest.raises(VisionError):
        smart_size(1, 1000, 8, 64, 4096)
    img = decode_image(png(100, 60))
    assert img.shape == (60, 100, 3) and img.dtype == torch.uint8
    pre = preprocess(img, hp)
    t, gh, gw = pre.grid
    assert pre.patches.shape == (gh * gw, 3 * 2 * 4 * 4) and (gh * 4, gw * 4) == pre.size
    # merge order: the first four patches are the 2 x 2 block in the top left corner; both frames of the temporal
    # patch hold the same still image
    hp2 = VisionHparams(patch_size=4, spatial_merge_size=2, temporal_patch_size=2, min_tokens=2, max_tokens=64,
                        resize="stretch")
    pre2 = preprocess(img, hp2)
    p = pre2.patches.view(-1, 3, 2, 4, 4)
    assert torch.equal(p[:, :, 0], p[:, :, 1])
    full = torch.zeros(3, pre2.size[0], pre2.size[1])
    from legion_b200.vision.tower import merge_order_coords
    rr, cc = merge_order_coords(pre2.grid[1], pre2.grid[2], 2, "cpu")
    assert (rr[:4].tolist(), cc[:4].tolist()) == ([0, 0, 1, 1], [0, 1, 0, 1])
    for i in range(p.shape[0]):
        full[:, rr[i] * 4:rr[i] * 4 + 4, cc[i] * 4:cc[i] * 4 + 4] = p[i, :, 0]
    x = torch.nn.functional.interpolate(img.permute(2, 0, 1)[None].float() / 255, size=pre2.size, mode="bicubic",
                                        align_corners=False, antialias=True)[0].clamp(0, 1)
    assert torch.allclose(full, (x - 0.5) / 0.5, atol=1e-5)
    with pytest.raises(VisionError):
        decode_image(b"not an image")


def test_tower_is_invariant_to_how_patches_are_grouped_and_respects_the_grid():
    cfg = VisionConfig(depth=2, hidden=32, n_head=2, intermediate=48, out_hidden=24, patch_size=4, num_pos=16,
                       deepstack_layers=(0,))
    tower = VisionTower(cfg, random_vision_weights(cfg, seed=2))
    hp = VisionHparams(patch_size=4, spatial_merge_size=2, min_tokens=2, max_tokens=64)
    pre = preprocess(decode_image(png(48, 32)), hp)
    e = tower.encode(pre.patches, pre.grid)
    gh, gw = pre.grid[1] // 2, pre.grid[2] // 2
    assert e.rows.shape == (gh * gw, 24) and e.grid == (1, gh, gw) and e.deepstack[0].shape == e.rows.shape
    assert torch.isfinite(e.rows).all()
    # attention is unmasked over the whole image and positions come from the grid: a different image changes every
    # row; the same image gives the same rows
    e2 = tower.encode(pre.patches, pre.grid)
    assert torch.equal(e.rows, e2.rows)
    other = preprocess(decode_image(png(48, 32, color=(10, 200, 90))), hp)
    assert (tower.encode(other.patches, other.grid).rows - e.rows).abs().max() > 1e-4
    with pytest.raises(ValueError):
        tower.encode(pre.patches[:-1], pre.grid)
    pool = VisionConfig(depth=1, hidden=32, n_head=2, intermediate=48, out_hidden=24, patch_size=4, num_pos=16,
                        projector="pool", spatial_merge_size=2)
    pt = VisionTower(pool, random_vision_weights(pool, seed=3))
    assert pt.encode(pre.patches, pre.grid).rows.shape == (gh * gw, 24)


def test_image_token_expansion_and_rotary_positions():
    toks, spans = expand_image_tokens([1, 5, 9, 5, 9, 7], 9, [4, 2])
    assert toks == [1, 5, 9, 9, 9, 9, 5, 9, 9, 7] and spans == [(2, 4), (7, 2)]
    with pytest.raises(ValueError):
        expand_image_tokens([1, 9, 2], 9, [4, 2])
    toks2, spans2 = expand_image_tokens([1, 2, 3], 9, [2], start_token=20, end_token=21)
    assert toks2 == [1, 20, 9, 9, 21, 2, 3] and spans2 == [(2, 2)]
    pos, delta = mrope_positions(len(toks), spans, [(1, 2, 2), (1, 1, 2)])
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:6].tolist() == [2, 2, 2, 2] and pos[1, 2:6].tolist() == [2, 2, 3, 3] and pos[2, 2:6].tolist() == [2, 3, 2, 3]
    assert pos[:, 6].tolist() == [4, 4, 4]                      # text continues from start + max(rows, columns)
    assert pos[:, 7:9].tolist() == [[5, 5], [5, 5], [5, 6]] and pos[:, 9].tolist() == [7, 7, 7]
    assert delta == 8 - len(toks)
    ax = mrope_axis_of_freq(32, (11, 11, 10), True)
    assert ax[:6].tolist() == [0, 1, 2, 0, 1, 2] and int((ax == 1).sum()) == 11 and int((ax == 2).sum()) == 10
    ax2 = mrope_axis_of_freq(32, (16, 8, 8), False)
    assert ax2.tolist() == [0] * 16 + [1] * 8 + [2] * 8


def _engine(mrope, deepstack=()):
    cfg = ModelConfig(arch="qwen3", n_layer=3, hidden=64, vocab=512, n_head=4, n_kv_head=2, head_dim=64, dense_ff=128,
                      mrope_sections=(11, 11, 10) if mrope else None)
    w = random_weights(cfg, "cpu", torch.float32, seed=4, std=0.05)
    eng = build_engine(cfg, weights=w, engine_cfg=EngineConfig(ctx_size=512, max_seqs=4, block_size=16, prefill_chunk=24,
                                                               max_batch_tokens=64), start=True)
    vc = VisionConfig(depth=2, hidden=32, n_head=2, intermediate=48, out_hidden=64, patch_size=4, num_pos=16,
                      deepstack_layers=deepstack)
    rt = VisionRuntime(VisionTower(vc, random_vision_weights(vc, seed=5)),
                       VisionHparams(patch_size=4, spatial_merge_size=2, min_tokens=2, max_tokens=64))
    eng.attach_vision(rt)
    return eng, rt


@pytest.mark.parametrize("mrope,deep", [(False, ()), (True, (0,))])
def test_engine_consumes_images(mrope, deep):
    """A chat request with an image: the placeholder expands to the tower's rows, the reply depends on the image,
    chunked prefill (chunks cut through the image) equals one pass, the same request again hits the prefix cache and
    the row cache, and another image behind the same placeholder ids does not."""
    eng, rt = _engine(mrope, deep)
    a, b = png(48, 32), png(48, 32, color=(10, 200, 90))

    def ask(img, text="what is this?", **kw):
        msg = ChatMessage("user", [{"type": "image"}, {"type": "text", "text": text}])
        req = GenerateRequest(messages=[msg], images=[img], sampling=SamplingParams(max_tokens=8, ignore_eos=True, **kw))
        return eng.generate(req).collect()

    r1 = ask(a)
    assert r1.error is None and len(r1.token_ids) == 8
    n_img = (48 // 8) * (32 // 8)
    assert r1.usage.prompt_tokens > n_img
    assert rt.encoded == 1
    r2 = ask(a)
    assert r2.token_ids == r1.token_ids and rt.encoded == 1 and rt.cache.hits >= 1
    assert r2.usage.cached_tokens >= 16                        # the image's blocks came from the prefix cache
    r3 = ask(b)
    assert rt.encoded == 2 and r3.usage.cached_tokens < r2.usage.cached_tokens + 16
    # logits of the image prompt: chunked prefill == one pass, and the image matters
    seq = eng.prepare(GenerateRequest(messages=[ChatMessage("user", [{"type": "image"}, {"type": "text", "text": "hi"}])],
                                      images=[a], sampling=SamplingParams(max_tokens=1)))
    seq_b = eng.prepare(GenerateRequest(messages=[ChatMessage("user", [{"type": "image"}, {"type": "text", "text": "hi"}])],
                                        images=[b], sampling=SamplingParams(max_tokens=1)))
    assert seq.tokens == seq_b.tokens and seq.key_tokens() != seq_b.key_tokens()
    assert seq.media.spans[0][1] == n_img
    if mrope:
        assert seq.media.rope_delta == max(48 // 8, 32 // 8) - n_img
    eng.shutdown()
    outs = []
    for s_, chunks in ((seq, None), (seq_b, None), (seq, 10)):
        e2, rt2 = _engine(mrope, deep)
        e2.shutdown()
        s2 = e2.prepare(s_.req)
        e2.waiting.push(s2)
        e2._admit()
        n = len(s2.tokens)
        step = chunks or n
        last = None
        for p0 in range(0, n, step):
            m = min(step, n - p0)
            bt = e2.build_batch([(s2, p0, m)])
            last = e2.model.forward(bt, e2.kv, e2.states).logits
            s2.n_computed = p0 + m
        outs.append(last[-1].float())
    assert (outs[0] - outs[1]).abs().max() > 1e-4
    assert torch.allclose(outs[0], outs[2], atol=2e-4, rtol=1e-4)


def test_requests_with_images_need_a_tower_and_matching_placeholders():
    cfg = ModelConfig(arch="qwen3", n_layer=1, hidden=64, vocab=512, n_head=4, n_kv_head=2, head_dim=64, dense_ff=128)
    eng = build_engine(cfg, weights=random_weights(cfg, "cpu", torch.float32, seed=4),
                       engine_cfg=EngineConfig(ctx_size=256, max_seqs=2, block_size=16), start=False)
    with pytest.raises(ValueError):
        eng.prepare(GenerateRequest(prompt="x", images=[png(16, 16)], sampling=SamplingParams(max_tokens=1)))


def test_mmproj_round_trip(tmp_path):
    from legion_b200.loaders.vision import load_mmproj, write_tiny_mmproj
    cfg = VisionConfig(depth=2, hidden=32, n_head=2, intermediate=48, out_hidden=24, patch_size=4, num_pos=16,
                       deepstack_layers=(1,))
    path = str(tmp_path / "mmproj.gguf")
    write_tiny_mmproj(path, cfg, seed=7)
    tower, hp = load_mmproj(path)
    want = random_vision_weights(cfg, seed=7)
    assert tower.cfg.depth == 2 and tower.cfg.deepstack_layers == (1,) and tower.cfg.out_hidden == 24
    assert all(torch.allclose(tower.w[k], want[k]) for k in want)
    pre = preprocess(decode_image(png(32, 32)), hp)
    a = tower.encode(pre.patches, pre.grid)
    b = VisionTower(cfg, want).encode(pre.patches, pre.grid)
    assert torch.allclose(a.rows, b.rows) and torch.allclose(a.deepstack[0], b.deepstack[0])


def test_images_over_http_openai_and_anthropic_shapes():
    """An image part in a chat request reaches the tower through the HTTP surface (data: URL for the OpenAI shape,
    base64 source for the Anthropic shape); a server whose model has no tower answers 400."""
    import base64
    from fastapi.testclient import TestClient
    from legion_b200.server.app import ServerConfig, create_app
    eng, rt = _engine(True, (0,))
    c = TestClient(create_app(eng, ServerConfig()))
    b64 = base64.b64encode(png(48, 32)).decode()
    r = c.post("/v1/chat/completions", json={"max_tokens": 5, "messages": [{"role": "user", "content": [
        {"type": "text", "text": "what is this?"}, {"type": "image_url", "image_url": {"url": "data:image/png;base64," + b64}}]}]})
    assert r.status_code == 200, r.text
    j = r.json()
    assert j["usage"]["prompt_tokens"] > 24 and j["usage"]["completion_tokens"] == 5 and rt.encoded == 1
    r = c.post("/v1/messages", json={"model": "m", "max_tokens": 4, "messages": [{"role": "user", "content": [
        {"type": "image", "source": {"type": "base64", "media_type": "image/png", "data": b64}},
        {"type": "text", "text": "and this?"}]}]})
    assert r.status_code == 200, r.text
    assert rt.encoded == 1 and rt.cache.hits >= 1               # the same image: rows from the cache
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [
        {"type": "image_url", "image_url": {"url": "data:image/png;base64,AAAA"}}]}]})
    assert r.status_code == 400
    eng.shutdown()
    from legion_b200.config import ModelConfig
    plain = build_engine(ModelConfig(arch="qwen3", n_layer=1, hidden=64, vocab=512, n_head=4, n_kv_head=2, head_dim=64,
                                     dense_ff=128), engine_cfg=EngineConfig(ctx_size=256, max_seqs=2, block_size=16))
    c2 = TestClient(create_app(plain, ServerConfig()))
    r = c2.post("/v1/chat/completions", json={"max_tokens": 2, "messages": [{"role": "user", "content": [
        {"type": "image_url", "image_url": {"url": "data:image/png;base64," + b64}}]}]})
    plain.shutdown()
    assert r.status_code == 400 and "vision" in r.text


def test_tower_from_a_hugging_face_checkpoint_directory(tmp_path):
    """``model.visual.*`` tensors and ``vision_config`` of a checkpoint directory -> the same tower."""
    import json as _json
    from legion_b200.loaders.safetensors_io import save_file
    from legion_b200.loaders.vision import hf_names, load_vision_hf
    cfg = VisionConfig(depth=2, hidden=32, n_head=2, intermediate=48, out_hidden=24, patch_size=4, num_pos=16,
                       deepstack_layers=(0,))
    w = random_vision_weights(cfg, seed=9)
    tensors = {}
    for flat, name in hf_names(cfg).items():
        t = w[flat]
        if flat == "patch.w":
            t = t.reshape(cfg.hidden, 3, cfg.temporal_patch_size, cfg.patch_size, cfg.patch_size)
        tensors[name] = t.contiguous()
    tensors["model.language_model.embed_tokens.weight"] = torch.zeros(4, 24)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(_json.dumps({
        "text_config": {"hidden_size": 24},
        "vision_config": {"depth": 2, "hidden_size": 32, "num_heads": 2, "intermediate_size": 48, "out_hidden_size": 24,
                          "patch_size": 4, "temporal_patch_size": 2, "spatial_merge_size": 2,
                          "num_position_embeddings": 16, "deepstack_visual_indexes": [0], "hidden_act": "gelu_pytorch_tanh"}}))
    (tmp_path / "preprocessor_config.json").write_text(_json.dumps({
        "image_mean": [0.4, 0.5, 0.6], "image_std": [0.2, 0.3, 0.4], "size": {"shortest_edge": 256, "longest_edge": 4096}}))
    tower, hp = load_vision_hf(str(tmp_path))
    assert tower.cfg.deepstack_layers == (0,) and tower.cfg.out_hidden == 24 and hp.image_mean == (0.4, 0.5, 0.6)
    assert hp.image_min_pixels == 256 and hp.image_max_pixels == 4096
    assert all(torch.allclose(tower.w[k], w[k]) for k in w)
    pre = preprocess(decode_image(png(40, 24)), hp)
    assert torch.allclose(tower.encode(pre.patches, pre.grid).rows, VisionTower(cfg, w).encode(pre.patches, pre.grid).rows)
    (tmp_path / "config.json").write_text(_json.dumps({"hidden_size": 24}))
    assert load_vision_hf(str(tmp_path)) is None


def test_tower_matches_the_transformers_qwen3_vl_vision_model(tmp_path):
    """A tiny random ``Qwen3VLVisionModel`` of the ``transformers`` package, saved under the names a checkpoint
    directory uses and read through ``load_vision_hf``: merged rows and every deepstack tap equal what that
    implementation computes for the same patches (patch embedding, resampled positions, 2-D rotary embedding in
    merge order, blocks, mergers)."""
    import json
    import os
    pytest.importorskip("transformers.models.qwen3_vl.modeling_qwen3_vl")
    from safetensors.torch import save_file
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLVisionConfig
    from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLVisionModel
    from legion_b200.loaders.vision import load_vision_hf
    torch.manual_seed(0)
    vc = Qwen3VLVisionConfig(depth=3, hidden_size=32, num_heads=4, intermediate_size=48, out_hidden_size=40,
                             patch_size=4, temporal_patch_size=2, spatial_merge_size=2, num_position_embeddings=36,
                             deepstack_visual_indexes=[0, 2], hidden_act="gelu_pytorch_tanh", in_channels=3)
    vc._attn_implementation = "eager"
    m = Qwen3VLVisionModel(vc).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            p.copy_(torch.randn_like(p) * (0.1 if p.dim() >= 2 else 0.3)
                    + (1.0 if ("norm" in n and n.endswith("weight")) else 0.0))
    save_file({"model.visual." + k: v.contiguous() for k, v in m.state_dict().items()},
              os.path.join(tmp_path, "model.safetensors"))
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump({"model_type": "qwen3_vl", "vision_config": vc.to_dict(), "text_config": {"hidden_size": 40}}, f)
    tower, _ = load_vision_hf(str(tmp_path))
    for gh, gw in ((6, 10), (4, 4)):
        patches = torch.randn(gh * gw, 3 * 2 * 4 * 4)
        with torch.no_grad():
            want = m(patches, torch.tensor([[1, gh, gw]]))
            got = tower.encode(patches, (1, gh, gw))
        assert (got.rows - want.pooler_output).abs().max().item() < 1e-4
        assert len(got.deepstack) == 2
        for a, b in zip(got.deepstack, want.deepstack_features):
            assert (a - b).abs().max().item() < 1e-4


def test_image_prompt_matches_the_transformers_qwen3_vl_model(tmp_path):
    """The whole image path against ``transformers``' ``Qwen3VLForConditionalGeneration`` on a tiny random checkpoint
    it saved: text weights through the HF loader, the tower through ``load_vision_hf``; a prompt with two images
    (placeholder expansion, tower rows in place of the placeholders, deepstack rows added after the first layers,
    interleaved multi-section rotary positions and the position offset behind an image) gives the same logits at every
    position, and the greedy continuation through the engine (chunked prefill that cuts through an image) is the
    same."""
    import io
    pytest.importorskip("transformers.models.qwen3_vl.modeling_qwen3_vl")
    from PIL import Image
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLConfig
    from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLForConditionalGeneration
    from legion_b200.loaders.hf_map import load_hf
    from legion_b200.loaders.vision import load_vision_hf
    from legion_b200.vision.preprocess import decode_image, preprocess
    torch.manual_seed(0)
    IMG, VS, VE = 300, 301, 302
    conf = Qwen3VLConfig(
        text_config=dict(vocab_size=320, hidden_size=64, intermediate_size=96, num_hidden_layers=3,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=32, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [6, 5, 5],
                                          "mrope_interleaved": True},
                         tie_word_embeddings=False, pad_token_id=0, eos_token_id=1, bos_token_id=2),
        vision_config=dict(depth=3, hidden_size=32, num_heads=4, intermediate_size=48, out_hidden_size=64, patch_size=4,
                           temporal_patch_size=2, spatial_merge_size=2, num_position_embeddings=36,
                           deepstack_visual_indexes=[0, 1], hidden_act="gelu_pytorch_tanh", in_channels=3),
        image_token_id=IMG, video_token_id=303, vision_start_token_id=VS, vision_end_token_id=VE,
        tie_word_embeddings=False)
    for c in (conf, conf.text_config, conf.vision_config):
        c._attn_implementation = "eager"
    m = Qwen3VLForConditionalGeneration(conf).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn_like(p) * 0.08)
            elif "norm" in n and n.endswith("weight"):
                p.copy_(1.0 + 0.2 * torch.randn_like(p))
            else:
                p.copy_(0.2 * torch.randn_like(p))
    m.save_pretrained(str(tmp_path), safe_serialization=True)
    cfg, w, _ = load_hf(str(tmp_path), "cpu", torch.float32)
    assert cfg.arch == "qwen3" and cfg.mrope_sections == (6, 5, 5) and cfg.mrope_interleaved
    tower, _ = load_vision_hf(str(tmp_path))
    hp = VisionHparams(patch_size=4, spatial_merge_size=2, min_tokens=2, max_tokens=64)

    def picture(wd, ht, k):
        im = Image.new("RGB", (wd, ht))
        px = im.load()
        for y in range(ht):
            for x in range(wd):
                px[x, y] = ((x * 7 + k) % 256, (y * 11 + 3 * k) % 256, (x * y + k) % 256)
        buf = io.BytesIO()
        im.save(buf, format="PNG")
        return buf.getvalue()

    images = [picture(40, 24, 1), picture(16, 32, 9)]
    toks = [5, 17, 33, VS, IMG, VE, 44, 91, VS, IMG, VE, 12, 7, 250]

    def make(**kw):
        e = build_engine(cfg, weights=dict(w), start=kw.pop("start", False),
                         engine_cfg=EngineConfig(ctx_size=256, max_seqs=2, block_size=16, max_batch_tokens=256, **kw))
        e.attach_vision(VisionRuntime(tower, hp, image_token=IMG, start_token=VS, end_token=VE))
        return e

    eng = make()
    seq = eng.prepare(GenerateRequest(prompt_tokens=toks, images=images, sampling=SamplingParams(max_tokens=1)))
    eng.waiting.push(seq)
    eng._admit()
    n = len(seq.tokens)
    b = eng.build_batch([(seq, 0, n)])
    b.logit_rows = None
    with torch.no_grad():
        mine = eng.model.forward(b, eng.kv, eng.states).logits.float()
    pre = [preprocess(decode_image(i), hp) for i in images]
    ids = torch.tensor([seq.tokens])
    feed = dict(pixel_values=torch.cat([p.patches for p in pre]), image_grid_thw=torch.tensor([list(p.grid) for p in pre]))
    with torch.no_grad():
        ref = m(input_ids=ids, mm_token_type_ids=(ids == IMG).long(), **feed).logits[0].float()
        cont = m.generate(input_ids=ids, mm_token_type_ids=(ids == IMG).long(), max_new_tokens=6, do_sample=False,
                          **feed)[0, n:].tolist()
    assert n == len(toks) - 2 + sum(p.grid[1] * p.grid[2] // 4 for p in pre)
    assert (mine - ref).abs().max().item() < 2e-4
    eng2 = make(start=True, prefill_chunk=16)
    out = eng2.generate(GenerateRequest(prompt_tokens=toks, images=images,
                                        sampling=SamplingParams(max_tokens=6, ignore_eos=True))).collect()
    eng2.shutdown()
    assert out.token_ids == cont


def test_gemma4_tower_matches_the_transformers_vision_model_and_round_trips_as_mmproj(tmp_path):
    """The Gemma 4 tower (two position tables, rotary embedding in two halves of a head, normed q / k / v, sandwich
    norms, k x k average pool, standardisation, un-weighted norm and projection) read from a checkpoint written with
    ``transformers``' ``Gemma4VisionModel`` and ``Gemma4MultimodalEmbedder``: the rows for a random image equal that
    implementation's soft tokens after its embedder; the preprocessor's channel-major, merge-order patches against
    the package's raster (row, column, channel) patches are part of what is compared. Then the ``gemma4v`` mmproj
    form: written, read back, same rows."""
    import json
    import os
    pytest.importorskip("transformers.models.gemma4.modeling_gemma4")
    from safetensors.torch import save_file
    from transformers.models.gemma4.configuration_gemma4 import Gemma4TextConfig, Gemma4VisionConfig as HC
    from transformers.models.gemma4.modeling_gemma4 import Gemma4MultimodalEmbedder, Gemma4VisionModel
    from legion_b200.loaders.vision import load_mmproj, load_vision_hf, write_tiny_gemma4v_mmproj
    from legion_b200.vision.gemma4v import Gemma4VisionTower
    from legion_b200.vision.preprocess import preprocess
    torch.manual_seed(0)
    vc = HC(hidden_size=32, intermediate_size=48, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4,
            head_dim=8, pooling_kernel_size=3, patch_size=4, position_embedding_size=32, standardize=True,
            use_clipped_linears=False, rope_parameters={"rope_type": "default", "rope_theta": 100.0})
    vc._attn_implementation = "eager"
    tc = Gemma4TextConfig(hidden_size=40, num_hidden_layers=2, layer_types=["sliding_attention", "full_attention"],
                          vocab_size=64, intermediate_size=32, num_attention_heads=2, num_key_value_heads=1, head_dim=8)
    vm, em = Gemma4VisionModel(vc).eval().float(), Gemma4MultimodalEmbedder(vc, tc).eval().float()
    with torch.no_grad():
        for mod in (vm, em):
            for n, p in mod.named_parameters():
                p.copy_(torch.randn_like(p) * (0.15 if p.dim() >= 2 else 0.2) + (1.0 if "norm" in n else 0.0))
        vm.std_bias.copy_(torch.randn(32) * 0.2)
        vm.std_scale.copy_(1 + 0.2 * torch.randn(32))
    sd = {"model.vision_tower." + k: v.contiguous() for k, v in vm.state_dict().items()}
    sd.update({"model.embed_vision." + k: v.contiguous() for k, v in em.state_dict().items()})
    save_file(sd, os.path.join(tmp_path, "model.safetensors"))
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump({"model_type": "gemma4", "vision_config": vc.to_dict(), "text_config": {"hidden_size": 40}}, f)
    tower, hp = load_vision_hf(str(tmp_path))
    assert isinstance(tower, Gemma4VisionTower) and hp.temporal_patch_size == 1 and hp.spatial_merge_size == 3
    gh, gw = 6, 9
    img = torch.randint(0, 256, (gh * 4, gw * 4, 3), dtype=torch.uint8)
    hp.image_min_pixels = hp.image_max_pixels = gh * gw * 16
    pre = preprocess(img, hp)
    assert pre.grid == (1, gh, gw)
    got = tower.encode(pre.patches, pre.grid)
    x = (img.float() / 255).permute(2, 0, 1)
    pv = x.reshape(3, gh, 4, gw, 4).permute(1, 3, 2, 4, 0).reshape(gh * gw, -1)[None]
    pos = torch.stack(torch.meshgrid(torch.arange(gw), torch.arange(gh), indexing="xy"), -1).reshape(-1, 2)[None]
    with torch.no_grad():
        want = em(vm(pixel_values=pv, pixel_position_ids=pos).last_hidden_state)
    assert got.rows.shape == want.shape == (6, 40) and got.grid == (1, 2, 3)
    assert (got.rows - want).abs().max().item() < 1e-4
    # the mmproj form of the same kind of tower
    path = str(tmp_path / "g4v.gguf")
    cfg, w = write_tiny_gemma4v_mmproj(path, seed=3)
    t2, hp2 = load_mmproj(path)
    assert isinstance(t2, Gemma4VisionTower) and t2.cfg.standardize and hp2.max_tokens == 1120
    P, k = cfg.patch_size, cfg.spatial_merge_size
    patches = torch.rand(2 * k * k, 3 * P * P)
    a = Gemma4VisionTower(cfg, w).encode(patches, (1, k, 2 * k)).rows
    b = t2.encode(patches, (1, k, 2 * k)).rows
    assert a.shape == (2, cfg.out_hidden) and torch.allclose(a, b, atol=1e-5)
