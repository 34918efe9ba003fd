"""/v1/chat/completions with tools and a reasoning parser, end to end through the adapter: the engine is replaced by
one that "generates" a scripted text token by token, so the route's parsing, finish reasons and SSE deltas can be
checked exactly (non-streaming and streaming must describe the same message)."""
import asyncio
import json
import types

from fastapi import FastAPI
from fastapi.testclient import TestClient

from ksanallm_b200.config.schema import parse_serving_config
from ksanallm_b200.serving.ksana_engine import EngineArgs, KsanaPythonOutput, Status
from ksanallm_b200.serving.openai.adapter import add_openai_routes
from ksanallm_b200.serving.tokenizer import TokenizerProcessor

SCRIPT = ('<think>the user wants the weather</think>Let me check.\n'
          '<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris", "unit": "C"}}\n</tool_call>')
TOOLS = [{"type": "function", "function": {"name": "get_weather", "description": "weather",
                                           "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}}]


class ScriptedEngine:
    def __init__(self):
        self.tokenizer = TokenizerProcessor(None, 32000)
        self.serving = parse_serving_config({})
        self.model_config = types.SimpleNamespace(vocab_size=32000, max_position_embeddings=2048)
        self.args = types.SimpleNamespace(model_dir="scripted")
        self.tokens = self.tokenizer.encode(SCRIPT, add_special_tokens=False)

    async def generate(self, request_dict, streamer=None, req_ctx=None):
        ids = list(request_dict["input_tokens"])
        if not streamer:
            return Status(), KsanaPythonOutput(input_tokens=ids, output_tokens=[list(self.tokens)],
                                               finish_reasons=["stop"], finished=True)

        async def it():
            for n in range(3, len(self.tokens) + 3, 3):  # three tokens per step, full output so far each time
                await asyncio.sleep(0)
                yield KsanaPythonOutput(input_tokens=ids, output_tokens=[list(self.tokens[:n])],
                                        finish_reasons=["stop" if n >= len(self.tokens) else None],
                                        finished=n >= len(self.tokens))
        return Status(), it()


def _client():
    args = EngineArgs(config_file="", tool_call_parser="hermes", reasoning_parser="deepseek_r1",
                      enable_auto_tool_choice=True)
    app = FastAPI()
    add_openai_routes(app, ScriptedEngine(), args)
    return TestClient(app)


def test_tool_call_and_reasoning_non_streaming():
    c = _client()
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "weather in Paris?"}],
                                             "tools": TOOLS, "tool_choice": "auto", "max_tokens": 128})
    assert r.status_code == 200, r.text
    ch = r.json()["choices"][0]
    msg = ch["message"]
    assert ch["finish_reason"] == "tool_calls"
    assert msg["reasoning_content"] == "the user wants the weather"
    assert msg["content"].strip() == "Let me check."
    call = msg["tool_calls"][0]["function"]
    assert call["name"] == "get_weather" and json.loads(call["arguments"]) == {"city": "Paris", "unit": "C"}


def test_streaming_deltas_rebuild_the_same_message():
    c = _client()
    r = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "weather in Paris?"}],
                                             "tools": TOOLS, "tool_choice": "auto", "max_tokens": 128, "stream": True})
    assert r.status_code == 200
    events = [json.loads(l[6:]) for l in r.text.split("\n\n") if l.startswith("data: ") and l != "data: [DONE]"]
    reasoning = content = args = ""
    name, finish = None, None
    for e in events:
        for ch in e.get("choices", []):
            d = ch.get("delta", {})
            reasoning += d.get("reasoning_content") or ""
            content += d.get("content") or ""
            for tc in d.get("tool_calls") or []:
                fn = tc.get("function", {})
                name = fn.get("name") or name
                args += fn.get("arguments") or ""
            finish = ch.get("finish_reason") or finish
    assert reasoning == "the user wants the weather"
    assert content.strip() == "Let me check."
    assert name == "get_weather" and json.loads(args) == {"city": "Paris", "unit": "C"}
    assert finish == "tool_calls"
