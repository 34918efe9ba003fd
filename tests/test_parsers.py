"""Tool-call and reasoning parsers: whole-text extraction and streaming deltas that reassemble to the same calls."""
import json

import pytest

from ksanallm_b200.serving.reasoning import get_reasoning_parser
from ksanallm_b200.serving.tool_parsers import get_tool_parser

ARGS = {"city": "Paris", "days": 3}
CASES = {
    "hermes": 'Sure.<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris", "days": 3}}\n</tool_call>',
    "llama": '<|python_tag|>{"name": "get_weather", "parameters": {"city": "Paris", "days": 3}}',
    "mistral": '[TOOL_CALLS] [{"name": "get_weather", "arguments": {"city": "Paris", "days": 3}}]',
    "internlm2": 'ok<|action_start|><|plugin|>{"name": "get_weather", "parameters": {"city": "Paris", "days": 3}}<|action_end|>',
    "pythonic": '[get_weather(city="Paris", days=3)]',
    "llama4_pythonic": '<|python_start|>[get_weather(city="Paris", days=3)]<|python_end|>',
    "deepseekv3": 'x<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>get_weather\n```json\n{"city": "Paris", "days": 3}\n```<｜tool▁call▁end｜><｜tool▁calls▁end｜>',
    "deepseekv31": '<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>get_weather<｜tool▁sep｜>{"city": "Paris", "days": 3}<｜tool▁call▁end｜><｜tool▁calls▁end｜>',
    "deepseekv32": '<｜DSML｜function_calls>\n<｜DSML｜invoke name="get_weather">\n<｜DSML｜parameter name="city" string="true">Paris</｜DSML｜parameter>\n<｜DSML｜parameter name="days" string="false">3</｜DSML｜parameter>\n</｜DSML｜invoke>\n</｜DSML｜function_calls>',
    "kimi_k2": '<|tool_calls_section_begin|><|tool_call_begin|>functions.get_weather:0<|tool_call_argument_begin|>{"city": "Paris", "days": 3}<|tool_call_end|><|tool_calls_section_end|>',
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_extract_tool_calls(name):
    p = get_tool_parser(name)()
    ext = p.extract_tool_calls(CASES[name])
    assert ext.tools_called and len(ext.tool_calls) == 1
    fn = ext.tool_calls[0]["function"]
    assert fn["name"] == "get_weather"
    assert json.loads(fn["arguments"]) == ARGS


@pytest.mark.parametrize("name", ["hermes", "llama", "mistral", "deepseekv3", "deepseekv31", "kimi_k2", "internlm2"])
def test_streaming_reassembles(name):
    p = get_tool_parser(name)()
    text = CASES[name]
    names, args, content = {}, {}, ""
    prev = ""
    for i in range(0, len(text), 3):
        cur = text[: i + 3]
        d = p.extract_tool_calls_streaming(prev, cur, cur[len(prev):])
        prev = cur
        if not d:
            continue
        content += d.get("content", "")
        for tc in d.get("tool_calls", []):
            f = tc.get("function", {})
            if f.get("name"):
                names[tc["index"]] = f["name"]
            args[tc["index"]] = args.get(tc["index"], "") + f.get("arguments", "")
    assert names == {0: "get_weather"}
    assert json.loads(args[0]) == ARGS
    assert "tool" not in content.lower() or name in ("hermes",) and "<tool_call>" not in content


def test_plain_text_is_not_a_tool_call():
    for name in CASES:
        ext = get_tool_parser(name)().extract_tool_calls("just some text, no tools [1, 2]")
        assert not ext.tools_called and ext.content == "just some text, no tools [1, 2]"


def test_reasoning_parsers():
    r1 = get_reasoning_parser("deepseek_r1")()
    assert r1.extract("step one</think>answer") == ("step one", "answer")
    assert r1.extract("<think>a</think>b") == ("a", "b")
    q = get_reasoning_parser("qwen3")()
    assert q.extract("no thinking here") == (None, "no thinking here")
    assert q.extract("<think>hmm</think>\n\nyes") == ("hmm", "\n\nyes")
    st = q.new_stream_state()
    rs, cs = "", ""
    for piece in ["<th", "ink>rea", "soning</th", "ink>ans", "wer"]:
        r, c = q.extract_streaming(st, piece)
        rs += r or ""
        cs += c or ""
    assert rs == "reasoning" and cs == "answer"
    st = r1.new_stream_state()
    rs, cs = "", ""
    for piece in ["thinking...", "</think>", "done"]:
        r, c = r1.extract_streaming(st, piece)
        rs += r or ""
        cs += c or ""
    assert rs == "thinking..." and cs == "done"
