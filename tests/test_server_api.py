"""HTTP API on CPU with a tiny random-weight model: /generate (stream + non-stream), /forward (msgpack probes),
/health, /metrics and the OpenAI routes (chat, completions, embeddings, models)."""
import base64
import json
import os
import struct

import msgpack
import pytest
from fastapi.testclient import TestClient

from ksanallm_b200.serving.ksana_engine import EngineArgs
from ksanallm_b200.serving.server import LLMServer

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def client():
    args = EngineArgs.from_config_file(os.path.join(ROOT, "examples", "tiny_cpu.yaml"), synthetic_model="tiny-llama",
                                       device="cpu")
    server = LLMServer(args)
    server.initialize()
    with TestClient(server.app) as c:
        yield c
    server.model.shutdown()


def test_health_and_models(client):
    assert client.get("/health").json() == {"status": "healthy"}
    ms = client.get("/v1/models").json()
    assert ms["object"] == "list" and ms["data"][0]["id"] == "tiny-llama"
    assert client.get("/v1/models/nope").status_code == 404


def test_generate_non_stream_and_stream_agree(client):
    body = {"prompt": "hello world", "stream": False,
            "sampling_config": {"max_new_tokens": 8, "topk": 1, "ignore_eos": True}}
    r = client.post("/generate", content=json.dumps(body))
    assert r.status_code == 200
    j = r.json()
    assert len(j["output_token_ids"][0]) == 8 and isinstance(j["texts"][0], str)
    assert j["input_token_ids"][0] == 1  # BOS of the stand-in tokenizer
    body["stream"] = True
    r = client.post("/generate", content=json.dumps(body))
    chunks = [json.loads(c) for c in r.content.split(b"\0") if c]
    assert chunks[-1]["output_token_ids"] == j["output_token_ids"]
    lens = [len(c["output_token_ids"][0]) for c in chunks]
    assert lens == sorted(lens)  # every chunk carries the full output so far


def test_generate_parallel_sampling_logprobs_and_errors(client):
    body = {"input_tokens": [5, 6, 7, 8], "stream": False,
            "sampling_config": {"max_new_tokens": 4, "topk": 20, "temperature": 0.8, "num_return_sequences": 3,
                                "logprobs": 2, "ignore_eos": True}}
    j = client.post("/generate", content=json.dumps(body)).json()
    assert len(j["output_token_ids"]) == 3 and all(len(o) == 4 for o in j["output_token_ids"])
    assert len(j["logprobs"][0]) == 4 and len(j["logprobs"][0][0]["top"]) == 2
    bad = client.post("/generate", content=json.dumps({"prompt": "x", "stream": False,
                                                        "sampling_config": {"topk": 5000}}))
    assert bad.status_code == 500
    too_long = client.post("/generate", content=json.dumps({"input_tokens": list(range(3, 400)), "stream": False}))
    assert too_long.status_code == 500 and "max_token_len" in too_long.text


def test_beam_search(client):
    body = {"input_tokens": [9, 10, 11], "stream": False,
            "sampling_config": {"max_new_tokens": 5, "num_beams": 3, "num_return_sequences": 2, "ignore_eos": True}}
    j = client.post("/generate", content=json.dumps(body)).json()
    assert len(j["output_token_ids"]) == 2
    assert all(len(o) == 5 for o in j["output_token_ids"])
    assert j["output_token_ids"][0] != j["output_token_ids"][1]


def test_forward_probes(client):
    req = {"requests": [{"input_tokens": [3, 4, 5, 6, 7], "request_target": [
        {"target_name": "logits", "slice_pos": [[0, -2]], "token_reduce_mode": "GATHER_TOKEN_ID"},
        {"target_name": "layernorm", "token_id": [4], "token_reduce_mode": "GATHER_ALL"},
        {"target_name": "transformer", "slice_pos": [[1, 2]], "token_reduce_mode": "GATHER_ALL"}]}]}
    r = client.post("/forward", content=msgpack.packb(req), headers={"Content-Type": "application/x-msgpack"})
    assert r.status_code == 200
    resp = msgpack.unpackb(r.content, raw=False)["responses"][0]
    assert resp["input_token_ids"] == [3, 4, 5, 6, 7]
    t0, t1, t2 = [x["tensor"] for x in resp["response"]]
    assert t0["shape"] == [4] and t1["shape"] == [1, 256] and t2["shape"] == [2, 256]
    probs = struct.unpack("<4f", base64.b64decode(t0["data"]))
    assert all(0.0 <= p <= 1.0 for p in probs)
    bad = client.post("/forward", content=msgpack.packb({"requests": [{"input_tokens": [1, 2], "request_target": [
        {"target_name": "nope"}]}]}))
    assert bad.status_code == 500


def test_openai_chat_and_completions(client):
    r = client.post("/v1/chat/completions", json={"model": "tiny-llama", "messages": [
        {"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0, "ignore_eos": True})
    assert r.status_code == 200
    j = r.json()
    assert j["object"] == "chat.completion" and j["choices"][0]["message"]["role"] == "assistant"
    assert j["usage"]["completion_tokens"] == 6
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6,
                                                  "temperature": 0, "stream": True, "ignore_eos": True,
                                                  "stream_options": {"include_usage": True}})
    lines = [l for l in r.text.split("\n\n") if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    events = [json.loads(l[6:]) for l in lines[:-1]]
    assert events[0]["choices"][0]["delta"]["role"] == "assistant"
    assert any(e["choices"] and e["choices"][0]["finish_reason"] for e in events)
    assert events[-1]["usage"]["completion_tokens"] == 6
    r = client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 5, "temperature": 0, "logprobs": 2,
                                             "ignore_eos": True})
    c = r.json()["choices"][0]
    assert len(c["logprobs"]["tokens"]) == 5
    e = client.post("/v1/embeddings", json={"input": ["abc", "defg"]}).json()
    assert len(e["data"]) == 2 and len(e["data"][0]["embedding"]) == 256


def test_metrics_endpoint(client):
    t = client.get("/metrics").text
    assert "ksana_time_to_first_token_us_count" in t and "ksana_generated_token_num" in t


def test_structured_output_json_schema_and_regex(client):
    """Grammar-constrained decoding: whatever the random model prefers, the output must satisfy the schema / the
    regular expression (token bitmask applied in the sampler), for greedy and for sampled requests."""
    pytest.importorskip("xgrammar")
    import re
    schema = {"type": "object", "properties": {"a": {"type": "integer"}, "ok": {"type": "boolean"}},
              "required": ["a", "ok"], "additionalProperties": False}
    for seed in (7, 8):
        body = {"prompt": "give json", "stream": False,
                "sampling_config": dict(topk=40, temperature=1.0, seed=seed, max_new_tokens=96, json_schema=schema)}
        r = client.post("/generate", content=json.dumps(body))
        assert r.status_code == 200, r.text
        obj = json.loads(r.json()["texts"][0])
        assert set(obj) == {"a", "ok"} and isinstance(obj["a"], int) and isinstance(obj["ok"], bool)
    # greedy: this random model keeps choosing white space, which JSON allows anywhere between tokens; what it emits
    # is still a prefix the grammar accepts
    body = {"prompt": "give json", "stream": False, "sampling_config": dict(topk=1, max_new_tokens=16, json_schema=schema)}
    assert re.fullmatch(r'\{\s*("a"\s*:?\s*-?\d*)?[\s\S]*', client.post("/generate", content=json.dumps(body)).json()["texts"][0])
    body = {"prompt": "phone", "stream": False,
            "sampling_config": {"topk": 1, "max_new_tokens": 32, "structured_output_regex": r"\d{3}-\d{4}"}}
    text = client.post("/generate", content=json.dumps(body)).json()["texts"][0]
    assert re.fullmatch(r"\d{3}-\d{4}", text)
    # the OpenAI route: response_format json_schema
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "json please"}],
                                                  "max_tokens": 96, "temperature": 1.0, "top_k": 40, "seed": 7,
                                                  "response_format": {"type": "json_schema", "json_schema": {
                                                      "name": "t", "schema": schema}}})
    assert r.status_code == 200, r.text
    obj = json.loads(r.json()["choices"][0]["message"]["content"])
    assert set(obj) == {"a", "ok"}


def test_openai_logit_bias_and_penalties_reach_the_sampler(client):
    r = client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 6, "temperature": 0, "ignore_eos": True,
                                             "logit_bias": {"100": 50}})
    assert r.json()["choices"][0]["text"] == "aaaaaa"  # id 100 is the byte 'a' of the stand-in tokenizer
    r = client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 6, "temperature": 0, "ignore_eos": True,
                                             "logit_bias": {"100": 50, "101": 49.5}, "frequency_penalty": 1.0})
    text = r.json()["choices"][0]["text"]
    assert set(text) == {"a", "b"} and text.startswith("ab")  # every use of a token costs it one logit
    assert client.post("/v1/completions", json={"prompt": "x", "max_tokens": 4, "presence_penalty": 3.0}).status_code != 200
