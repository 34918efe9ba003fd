"""Multimodal end to end on CPU: a tiny random Qwen2-VL checkpoint (transformers) is saved to disk and served through
the engine with the bundled vision plugin; an image in the request becomes spliced embeddings + three-axis positions.
Greedy tokens must equal ``generate`` of the transformers model given the same pixels."""
import asyncio
import base64
import io
import json
import os

import pytest
import torch

transformers = pytest.importorskip("transformers")

from ksanallm_b200.config.schema import parse_serving_config  # noqa: E402
from ksanallm_b200.serving.ksana_engine import EngineArgs, KsanaLLMEngine  # noqa: E402
from ksanallm_b200.serving.plugins.qwen2_vl import mrope_positions  # noqa: E402

IMG, VSTART, VEND = 290, 291, 292


def _tiny_model(tmp):
    cfg = transformers.Qwen2VLConfig(
        text_config=dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         intermediate_size=128, vocab_size=300, max_position_embeddings=512,
                         rope_scaling=dict(type="mrope", mrope_section=[2, 3, 3]), tie_word_embeddings=False),
        vision_config=dict(depth=2, embed_dim=32, hidden_size=64, num_heads=4, mlp_ratio=2, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2, in_channels=3),
        image_token_id=IMG, video_token_id=293, vision_start_token_id=VSTART, vision_end_token_id=VEND,
        tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = transformers.Qwen2VLForConditionalGeneration(cfg).eval().float()
    hf.generation_config.eos_token_id = None
    hf.save_pretrained(tmp, safe_serialization=True)
    with open(os.path.join(tmp, "ksana_plugin.py"), "w") as f:
        f.write("from ksanallm_b200.serving.plugins.qwen2_vl import KsanaPlugin  # noqa: F401\n")
    return hf


def test_mrope_positions_rule():
    # text, a 1 x 4 x 6-patch image (2 x 3 merged tokens), text
    toks = [5, 6, IMG, IMG, IMG, IMG, IMG, IMG, 7, 8]
    pos = mrope_positions(toks, [(1, 4, 6)], IMG, 2)
    assert pos[0].tolist() == [0, 1, 2, 2, 2, 2, 2, 2, 5, 6]
    assert pos[1].tolist() == [0, 1, 2, 2, 2, 3, 3, 3, 5, 6]
    assert pos[2].tolist() == [0, 1, 2, 3, 4, 2, 3, 4, 5, 6]


def _png_url(img):
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    return "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()


def test_image_requests_match_transformers_generate(tmp_path):
    """Two requests with the SAME token ids and different images run concurrently (their KV must not be shared through
    the prefix tree); the second image spans several prefill chunks."""
    from PIL import Image
    tmp = str(tmp_path)
    hf = _tiny_model(tmp)
    g = torch.Generator().manual_seed(1)
    imgs = [Image.fromarray((torch.rand(h, w, 3, generator=g) * 255).byte().numpy()) for h, w in ((56, 84), (112, 140))]
    args = EngineArgs(config_file="", model_dir=tmp, device="cpu",
                      serving=parse_serving_config({"setting": {"batch_scheduler": {
                          "max_batch_size": 4, "max_step_tokens": 128, "max_token_len": 256,
                          "split_fuse_token_num": 16, "enable_auto_prefix_cache": True},
                          "block_manager": {"block_token_num": 16}}}))
    eng = KsanaLLMEngine(args)
    eng.initialize()
    try:
        assert eng.plugin is not None and eng.model_config.rope_scaling.mrope_section == [2, 3, 3]
        prompt = [5, 9, VSTART, IMG, VEND, 33, 4, 8]

        def body(img):
            return {"input_tokens": prompt, "stream": False,
                    "messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": _png_url(img)}},
                                                              {"type": "text", "text": "x"}]}],
                    "sampling_config": {"max_new_tokens": 6, "topk": 1, "ignore_eos": True}}

        async def both():
            return await asyncio.gather(*[eng.generate(json.loads(json.dumps(body(i))), streamer=False) for i in imgs])

        results = asyncio.run(both())
        # once more, one after the other: nothing of the first round may have been cached under these token ids
        results += [asyncio.run(eng.generate(json.loads(json.dumps(body(i))), streamer=False)) for i in imgs]
        for k, (st, out) in enumerate(results):
            img = imgs[k % 2]
            assert st.OK()
            wide = out.input_tokens
            n_img = wide.count(IMG)
            assert n_img == (6, 20)[k % 2] and len(wide) == len(prompt) - 1 + n_img
            feats = eng.plugin.impl.image_processor(images=[img.convert("RGB")], return_tensors="pt")
            with torch.no_grad():
                want = hf.generate(input_ids=torch.tensor([wide]), pixel_values=feats["pixel_values"],
                                   image_grid_thw=feats["image_grid_thw"],
                                   attention_mask=torch.ones(1, len(wide), dtype=torch.long),
                                   max_new_tokens=6, do_sample=False)[0, len(wide):].tolist()
            assert out.output_tokens[0] == want
        assert eng.llm.cache.stats.prefix_hit_tokens == 0
    finally:
        eng.shutdown()


def test_openai_chat_route_hands_image_parts_to_the_plugin(tmp_path):
    """/v1/chat/completions with an image_url part: the raw messages reach the plugin (the stand-in chat template
    renders no image placeholder, so the test inserts the one a vision-language template would) and the request
    runs to completion."""
    from fastapi.testclient import TestClient
    from PIL import Image
    from ksanallm_b200.serving.server import LLMServer
    tmp = str(tmp_path)
    _tiny_model(tmp)
    img = Image.fromarray((torch.rand(56, 84, 3) * 255).byte().numpy())
    args = EngineArgs(config_file="", model_dir=tmp, device="cpu",
                      serving=parse_serving_config({"setting": {"batch_scheduler": {
                          "max_batch_size": 2, "max_step_tokens": 128, "max_token_len": 256}}}))
    os.environ["KSANA_SKIP_WARMUP"] = "1"
    server = LLMServer(args)
    server.initialize()
    try:
        seen = {}
        impl = server.model.plugin.impl
        orig = impl.preprocess

        def spy(**kw):
            seen["messages"] = kw.get("messages")
            toks = list(kw["input_tokens"])
            kw["input_tokens"] = toks[:2] + [VSTART, IMG, VEND] + toks[2:]  # what a VL chat template would render
            return orig(**kw)

        impl.preprocess = spy
        with TestClient(server.app) as c:
            r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [
                {"type": "image_url", "image_url": {"url": _png_url(img)}}, {"type": "text", "text": "hi"}]}],
                "max_tokens": 4, "temperature": 0, "ignore_eos": True})
        assert r.status_code == 200, r.text
        assert seen["messages"][0]["content"][0]["type"] == "image_url"
        assert r.json()["usage"]["completion_tokens"] == 4
    finally:
        server.model.shutdown()


def test_image_request_across_a_prefill_decode_hand_over(tmp_path):
    """Prefill and decode instances both run the plugin on the forwarded request; the decode side continues from the
    handed-over first token with positions extended past the prompt's three-axis layout, and answers like a single
    instance."""
    from PIL import Image
    tmp = str(tmp_path)
    _tiny_model(tmp)
    os.environ["KSANA_SKIP_WARMUP"] = "1"
    img = Image.fromarray((torch.rand(56, 84, 3, generator=torch.Generator().manual_seed(4)) * 255).byte().numpy())

    def make(role, **extra):
        serving = parse_serving_config({"setting": {"batch_scheduler": {
            "max_batch_size": 2, "max_step_tokens": 128, "max_token_len": 256, "enable_auto_prefix_cache": True},
            "block_manager": {"block_token_num": 16}}})
        cs = serving.setting.connector
        cs.group_role, cs.connector_waiting_sec = role, 30
        cs.extra.update(extra)
        e = KsanaLLMEngine(EngineArgs(config_file="", model_dir=tmp, device="cpu", serving=serving))
        e.initialize()
        return e

    body = {"input_tokens": [5, 9, VSTART, IMG, VEND, 33, 4, 8], "stream": False,
            "messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": _png_url(img)}}]}],
            "sampling_config": {"max_new_tokens": 6, "topk": 1, "ignore_eos": True}}
    single = make("none")
    decode = make("decode")
    prefill = make("prefill", peer_transfer_addr="%s:%d" % decode.connector.transfer_addr)
    try:
        st, want = asyncio.run(single.generate(json.loads(json.dumps(body)), streamer=False))
        assert st.OK()
        ctx = {"kv-comm-request-id": "img-1"}

        async def both():
            d = asyncio.create_task(decode.generate(json.loads(json.dumps(body)), streamer=False, req_ctx=ctx))
            p = asyncio.create_task(prefill.generate(json.loads(json.dumps(body)), streamer=False, req_ctx=ctx))
            return await asyncio.gather(p, d)

        (pst, pout), (dst, dout) = asyncio.run(both())
        assert pst.OK() and dst.OK()
        assert dout.output_tokens == want.output_tokens and dout.input_tokens == want.input_tokens
    finally:
        for e in (single, decode, prefill):
            e.shutdown()
