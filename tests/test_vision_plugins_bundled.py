"""Bundled plugins whose vision side is the checkpoint's own remote code (Qwen-VL, InternLM-XComposer2): prompt
handling, placeholder positions and the spliced rows, with stand-in towers; and one request through a tiny engine."""
import asyncio
import types

import pytest
import torch

from ksanallm_b200.serving import plugin as plugin_host
from ksanallm_b200.serving.plugins import internlmxcomposer2, qwen_vl

H = 256
START = 1000


class _Tower:
    def __init__(self):
        self.seen = []

    def encode(self, urls):
        self.seen.append(list(urls))
        return torch.stack([torch.full((256, H), float(len(u))) for u in urls])


def _qwen_tokens(urls, text=(5, 6, 7)):
    toks = [3, 4]
    for u in urls:
        b = list(u.encode())
        toks += [START] + b + [START + 2] * (256 - len(b)) + [START + 1]
        toks += list(text)
    return toks


def _host(impl):
    engine = types.SimpleNamespace(model_config=types.SimpleNamespace(hidden_size=H),
                                   tokenizer=types.SimpleNamespace(tokenizer=None))
    return plugin_host.PluginHost(impl, engine)


def test_qwen_vl_reads_urls_back_and_splices_256_rows_per_image():
    impl = qwen_vl.KsanaPlugin()
    tower = _Tower()
    impl.init_plugin(model_path="", visual={"image_start_id": START}, tower=tower, device="cpu")
    urls = ["file:///tmp/a.png", "data:image/png;base64,QUJD"]
    toks = _qwen_tokens(urls)
    out = _host(impl).preprocess({"input_tokens": toks}, toks)
    assert tower.seen == [urls]
    assert "input_tokens" not in out  # the 256 slots are already in the prompt
    (p0, e0), (p1, e1) = out["refit"]
    assert toks[p0 - 1] == START and toks[p0 + 256] == START + 1 and toks[p1 - 1] == START
    assert e0.shape == (256, H) and float(e0[0, 0]) == len(urls[0]) and float(e1[0, 0]) == len(urls[1])
    assert _host(impl).preprocess({}, [1, 2, 3]) is None
    with pytest.raises(ValueError):
        qwen_vl.image_urls([START, 65, 66], START)
    assert plugin_host.search_plugin_path("", {"plugin_name": "qwen_vl"}).endswith("qwen_vl.py")


class _Tok:
    def __call__(self, text, add_special_tokens=True, **kw):
        ids = ([1] if add_special_tokens else []) + [10 + (ord(c) % 50) for c in text]
        return types.SimpleNamespace(input_ids=ids)


class _IXC:
    def encode_img(self, image):
        n = 4 if "small" in image else 6
        return torch.full((1, n, H), float(n))


def test_internlm_xcomposer2_builds_the_chat_prompt_around_image_rows():
    impl = internlmxcomposer2.KsanaPlugin()
    impl.init_plugin(model_path="", tokenizer=_Tok(), model=_IXC(), max_length=4096, device="cpu")
    msgs = [{"role": "user", "content": [{"type": "text", "text": f"compare {internlmxcomposer2.MARK} with {internlmxcomposer2.MARK}"},
                                         {"type": "image_url", "image_url": {"url": "small.png"}},
                                         {"type": "image_url", "image_url": {"url": "big.png"}}]}]
    out = _host(impl).preprocess({"messages": msgs}, [1, 2])
    toks = out["input_tokens"]
    (p0, e0), (p1, e1) = out["refit"]
    assert toks[0] == 1 and toks.count(1) == 1                      # one BOS, on the first piece
    assert toks[p0:p0 + 4] == [0] * 4 and toks[p1:p1 + 6] == [0] * 6  # placeholders where the rows go
    assert e0.shape == (4, H) and e1.shape == (6, H) and p1 > p0 + 4
    # a single image without a marker goes in front of the prompt
    one = [{"role": "user", "content": [{"type": "text", "text": "what is this"},
                                        {"type": "image_url", "image_url": {"url": "small.png"}}]}]
    out1 = _host(impl).preprocess({"messages": one}, [1, 2])
    assert out1["refit"][0][0] == 0 and out1["input_tokens"][:4] == [0] * 4 and out1["input_tokens"][4] == 1
    # the cut never splits an image
    impl.max_length = out["refit"][1][0] + 3
    cut = _host(impl).preprocess({"messages": msgs}, [1, 2])
    assert len(cut["refit"]) == 1 and len(cut["input_tokens"]) == out["refit"][1][0]
    assert _host(impl).preprocess({"messages": [{"role": "user", "content": "text only"}]}, [1, 2]) is None


def test_spliced_rows_reach_the_model(tmp_path):
    """Through a tiny engine: the request with spliced rows generates something else than the same tokens without."""
    from ksanallm_b200.config.schema import parse_serving_config
    from ksanallm_b200.serving.ksana_engine import EngineArgs, KsanaLLMEngine
    cfg = parse_serving_config({"setting": {"global": {}, "batch_scheduler": {
        "max_batch_size": 4, "max_step_tokens": 512, "max_token_len": 1024}, "block_manager": {"block_token_num": 16}}})
    eng = KsanaLLMEngine(EngineArgs(config_file="", synthetic_model="tiny-llama", device="cpu", serving=cfg))
    eng.initialize()
    try:
        impl = qwen_vl.KsanaPlugin()
        impl.init_plugin(model_path="", visual={"image_start_id": START}, tower=_Tower(), device="cpu")
        toks = _qwen_tokens(["file:///x.png"])
        body = {"input_tokens": toks, "sampling_config": {"max_new_tokens": 4, "topk": 1, "ignore_eos": True}}
        st0, plain = asyncio.run(eng.generate(dict(body), streamer=False))
        eng.plugin = plugin_host.PluginHost(impl, eng)
        st1, spliced = asyncio.run(eng.generate(dict(body), streamer=False))
        assert st0.OK() and st1.OK()
        assert spliced.output_tokens != plain.output_tokens
    finally:
        eng.shutdown()
