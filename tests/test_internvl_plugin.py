"""InternVL end to end on CPU: tiny random checkpoint (transformers layout) served with the bundled plugin; greedy
tokens must equal ``generate`` of the transformers model given the same pixels. Tiling rule checked separately."""
import asyncio
import json
import os

import pytest
import torch

transformers = pytest.importorskip("transformers")
if not hasattr(transformers, "InternVLForConditionalGeneration"):
    pytest.skip("this transformers has no InternVL", allow_module_level=True)

from ksanallm_b200.config.schema import parse_serving_config  # noqa: E402
from ksanallm_b200.serving.ksana_engine import EngineArgs, KsanaLLMEngine  # noqa: E402
from ksanallm_b200.serving.plugins.internvl import tile_grid  # noqa: E402

IMG = 290


def test_tile_grid_prefers_the_closest_aspect_ratio():
    assert tile_grid(448, 448, 448, 1) == (1, 1)
    assert tile_grid(1000, 500, 448, 6) == (2, 1)
    assert tile_grid(500, 1500, 448, 6) == (1, 3)
    assert tile_grid(1200, 800, 448, 6) == (3, 2)


def test_image_request_matches_transformers_generate(tmp_path):
    from PIL import Image
    tmp = str(tmp_path)
    cfg = transformers.InternVLConfig(
        text_config=dict(model_type="qwen2", hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, intermediate_size=128, vocab_size=300, max_position_embeddings=512,
                         tie_word_embeddings=False),
        vision_config=dict(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                           image_size=[56, 56], patch_size=[14, 14]),
        image_token_id=IMG, downsample_ratio=0.5, tie_word_embeddings=False)
    torch.manual_seed(0)
    hf = transformers.InternVLForConditionalGeneration(cfg).eval().float()
    hf.generation_config.eos_token_id = None
    hf.save_pretrained(tmp, safe_serialization=True)
    with open(os.path.join(tmp, "ksana_plugin.py"), "w") as f:
        f.write("from ksanallm_b200.serving.plugins.internvl import KsanaPlugin  # noqa: F401\n")
    os.environ["KSANA_SKIP_WARMUP"] = "1"
    args = EngineArgs(config_file="", model_dir=tmp, device="cpu",
                      serving=parse_serving_config({"setting": {"batch_scheduler": {
                          "max_batch_size": 2, "max_step_tokens": 128, "max_token_len": 256}}}))
    eng = KsanaLLMEngine(args)
    eng.initialize()
    try:
        assert eng.model_config.model_type == "qwen2" and eng.model_config.qkv_bias
        g = torch.Generator().manual_seed(1)
        img = Image.fromarray((torch.rand(70, 90, 3, generator=g) * 255).byte().numpy())
        prompt = [5, 9, IMG, 33, 4, 8]
        body = {"input_tokens": prompt, "stream": False, "images": [img],
                "sampling_config": {"max_new_tokens": 6, "topk": 1, "ignore_eos": True}}
        st, out = asyncio.run(eng.generate(body, streamer=False))
        assert st.OK()
        wide = out.input_tokens
        assert wide.count(IMG) == 4  # (56 / 14)^2 patches * 0.5^2
        px = eng.plugin.impl.tiles_of(img)
        with torch.no_grad():
            want = hf.generate(input_ids=torch.tensor([wide]), pixel_values=px,
                               attention_mask=torch.ones(1, len(wide), dtype=torch.long),
                               max_new_tokens=6, do_sample=False)[0, len(wide):].tolist()
        assert out.output_tokens[0] == want
    finally:
        eng.shutdown()
