"""Tool-call parsers: turn model text into OpenAI ``tool_calls`` (whole text and streaming).

Parser names match the reference (src/ksana_llm/python/openaiapi/tool_parsers/: deepseekv3, deepseekv31,
deepseekv32, hermes, internlm2, kimi_k2, llama, llama4_pythonic, mistral, pythonic). Each parser only implements
``parse_partial(text)`` - a tolerant parse of a possibly incomplete generation into leading content plus a list of
(name, argument-text-so-far, complete) - and the base class derives both the final extraction and the streaming
deltas (a tool call's name is emitted once, its arguments as string increments) by diffing successive parses.
"""
from __future__ import annotations

import ast
import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple, Type


@dataclass
class ParsedCall:
    name: str
    arguments: str  # JSON text (possibly a prefix while streaming)
    complete: bool = True


@dataclass
class ExtractedToolCalls:
    tools_called: bool
    tool_calls: List[Dict[str, Any]] = field(default_factory=list)
    content: Optional[str] = None


def _call_id() -> str:
    return "call_" + uuid.uuid4().hex[:24]


def _json_args(obj: Any) -> str:
    return json.dumps(obj, ensure_ascii=False)


def _balanced_json_prefix(s: str) -> Tuple[Optional[str], bool]:
    """Longest prefix of ``s`` that is one JSON value: (text, complete)."""
    s = s.lstrip()
    if not s or s[0] not in "{[":
        return (None, False)
    depth, in_str, esc = 0, False, False
    for i, ch in enumerate(s):
        if in_str:
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
            continue
        if ch == '"':
            in_str = True
        elif ch in "{[":
            depth += 1
        elif ch in "}]":
            depth -= 1
            if depth == 0:
                return s[:i + 1], True
    return s, False


def _partial_name_args(blob: str, args_keys=("arguments", "parameters")) -> Optional[ParsedCall]:
    """``{"name": "f", "arguments": {...`` possibly cut anywhere -> ParsedCall with the argument text so far."""
    text, complete = _balanced_json_prefix(blob)
    if text is None:
        return None
    if complete:
        try:
            obj = json.loads(text)
            if isinstance(obj, dict) and "name" in obj:
                args = next((obj[k] for k in args_keys if k in obj), {})
                return ParsedCall(str(obj["name"]), args if isinstance(args, str) else _json_args(args), True)
        except Exception:
            return None
    m = re.search(r'"name"\s*:\s*"([^"]*)"', text)
    if not m:
        return None
    name = m.group(1)
    am = re.search(r'"(?:%s)"\s*:\s*' % "|".join(args_keys), text)
    if not am:
        return ParsedCall(name, "", False)
    rest = text[am.end():]
    atext, adone = _balanced_json_prefix(rest)
    return ParsedCall(name, atext or "", False if not adone else False)


class ToolParser:
    """Base class. Subclasses implement ``parse_partial``."""

    def __init__(self, tokenizer=None):
        self.tokenizer = tokenizer
        self._sent_content = 0
        self._sent: List[Dict[str, Any]] = []  # per call: {"id", "name_sent", "args_sent"}

    def parse_partial(self, text: str) -> Tuple[str, List[ParsedCall]]:
        raise NotImplementedError

    def adjust_request(self, request):
        return request

    # ---- whole text ---------------------------------------------------------------------------------------------
    def extract_tool_calls(self, model_output: str, request=None) -> ExtractedToolCalls:
        try:
            content, calls = self.parse_partial(model_output)
        except Exception:
            return ExtractedToolCalls(False, [], model_output)
        calls = [c for c in calls if c.name]
        if not calls:
            return ExtractedToolCalls(False, [], model_output)
        out = []
        for c in calls:
            args = c.arguments
            try:
                json.loads(args)
            except Exception:
                args = args if args else "{}"
            out.append({"id": _call_id(), "type": "function", "function": {"name": c.name, "arguments": args}})
        content = content.strip() if content else None
        return ExtractedToolCalls(True, out, content or None)

    # ---- streaming ---------------------------------------------------------------------------------------------------
    def extract_tool_calls_streaming(self, previous_text: str, current_text: str, delta_text: str,
                                     request=None) -> Optional[Dict[str, Any]]:
        """Returns an OpenAI delta ({"content": ...} and/or {"tool_calls": [...]}) or None when nothing new."""
        try:
            content, calls = self.parse_partial(current_text)
        except Exception:
            return None
        delta: Dict[str, Any] = {}
        safe = self._safe_content_len(content, current_text, bool(calls))
        if safe > self._sent_content:
            delta["content"] = content[self._sent_content:safe]
            self._sent_content = safe
        tcs = []
        for i, c in enumerate(calls):
            if i >= len(self._sent):
                self._sent.append({"id": _call_id(), "name_sent": False, "args_sent": 0})
            st = self._sent[i]
            item: Dict[str, Any] = {"index": i}
            if not st["name_sent"] and c.name and (c.complete or c.arguments or i + 1 < len(calls)):
                item.update({"id": st["id"], "type": "function", "function": {"name": c.name, "arguments": ""}})
                st["name_sent"] = True
            if st["name_sent"] and len(c.arguments) > st["args_sent"]:
                inc = c.arguments[st["args_sent"]:]
                item.setdefault("function", {})["arguments"] = inc
                st["args_sent"] = len(c.arguments)
            if len(item) > 1:
                tcs.append(item)
        if tcs:
            delta["tool_calls"] = tcs
        return delta or None

    # text that might still turn into a tool-call marker is held back
    markers: Tuple[str, ...] = ()

    def _safe_content_len(self, content: str, full: str, has_calls: bool) -> int:
        if has_calls:
            return len(content)
        n = len(content)
        for mk in self.markers:
            for k in range(min(len(mk) - 1, n), 0, -1):
                if mk.startswith(content[n - k:]):
                    return n - k
        return n


# ---- concrete parsers ---------------------------------------------------------------------------------------------

class HermesToolParser(ToolParser):
    """``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` (Hermes, Qwen2.5 / Qwen3)."""
    markers = ("<tool_call>",)

    def parse_partial(self, text):
        parts = text.split("<tool_call>")
        content = parts[0]
        calls = []
        for p in parts[1:]:
            body = p.split("</tool_call>")[0]
            c = _partial_name_args(body)
            if c is not None:
                c.complete = "</tool_call>" in p and c.complete
                calls.append(c)
        return content, calls


class LlamaToolParser(ToolParser):
    """Llama 3.x JSON tool calls: ``{"name": ..., "parameters": {...}}`` objects separated by ``;``, optionally
    after ``<|python_tag|>``."""
    markers = ("<|python_tag|>", "{")

    def parse_partial(self, text):
        t = text
        content = ""
        if "<|python_tag|>" in t:
            content, t = t.split("<|python_tag|>", 1)
        stripped = t.lstrip()
        if not stripped.startswith("{"):
            return text, []
        calls = []
        rest = stripped
        while rest:
            blob, done = _balanced_json_prefix(rest)
            if blob is None:
                break
            c = _partial_name_args(blob)
            if c is None:
                return text, []
            calls.append(c)
            if not done:
                break
            rest = rest[len(blob):].lstrip().lstrip(";").lstrip()
        return content, calls


class MistralToolParser(ToolParser):
    """``[TOOL_CALLS] [{"name": ..., "arguments": {...}}, ...]``."""
    markers = ("[TOOL_CALLS]",)

    def parse_partial(self, text):
        if "[TOOL_CALLS]" not in text:
            return text, []
        content, rest = text.split("[TOOL_CALLS]", 1)
        rest = rest.lstrip()
        calls = []
        if rest.startswith("["):
            rest = rest[1:]
        while rest.lstrip().startswith("{"):
            rest = rest.lstrip()
            blob, done = _balanced_json_prefix(rest)
            c = _partial_name_args(blob)
            if c is None:
                break
            calls.append(c)
            if not done:
                break
            rest = rest[len(blob):].lstrip().lstrip(",")
        return content, calls


class InternLM2ToolParser(ToolParser):
    """``<|action_start|><|plugin|>{"name": ..., "parameters": {...}}<|action_end|>``."""
    markers = ("<|action_start|>",)

    def parse_partial(self, text):
        if "<|action_start|>" not in text:
            return text, []
        content, rest = text.split("<|action_start|>", 1)
        rest = rest.replace("<|plugin|>", "", 1).split("<|action_end|>")[0]
        c = _partial_name_args(rest, ("parameters", "arguments"))
        return content, [c] if c else []


def _pythonic_calls(src: str) -> List[ParsedCall]:
    tree = ast.parse(src.strip(), mode="eval")
    body = tree.body
    elts = body.elts if isinstance(body, (ast.List, ast.Tuple)) else [body]
    out = []
    for e in elts:
        if not isinstance(e, ast.Call):
            raise ValueError("not a call")
        name = ast.unparse(e.func)
        args = {kw.arg: ast.literal_eval(kw.value) for kw in e.keywords}
        out.append(ParsedCall(name, _json_args(args), True))
    return out


class PythonicToolParser(ToolParser):
    """``[get_weather(city="Paris"), other(x=1)]`` (Llama 3.2 / ToolACE pythonic style)."""
    markers = ("[",)
    prefix = ""
    suffix = ""

    def parse_partial(self, text):
        t = text.strip()
        if self.prefix and self.prefix in t:
            t = t.split(self.prefix, 1)[1]
        if self.suffix and self.suffix in t:
            t = t.split(self.suffix, 1)[0]
        t = t.strip()
        if not (t.startswith("[") and re.match(r"\[\s*[A-Za-z_][\w\.]*\s*\(", t)):
            return text, []
        for candidate in (t, t + ")]", t + "]", t + '")]', t + "')]"):
            try:
                calls = _pythonic_calls(candidate)
                if candidate is not t:
                    for c in calls[-1:]:
                        c.complete = False
                        c.arguments = c.arguments.rstrip("}")  # still growing
                return "", calls
            except Exception:
                continue
        return "", []


class Llama4PythonicToolParser(PythonicToolParser):
    prefix = "<|python_start|>"
    suffix = "<|python_end|>"
    markers = ("<|python_start|>", "[")


class DeepSeekV3ToolParser(ToolParser):
    """``<｜tool▁calls▁begin｜><｜tool▁call▁begin｜>function<｜tool▁sep｜>NAME\\n```json\\n{...}\\n```<｜tool▁call▁end｜>...``."""
    CALLS_BEGIN = "<｜tool▁calls▁begin｜>"
    CALL_BEGIN = "<｜tool▁call▁begin｜>"
    SEP = "<｜tool▁sep｜>"
    CALL_END = "<｜tool▁call▁end｜>"
    markers = (CALLS_BEGIN,)

    def parse_partial(self, text):
        if self.CALLS_BEGIN not in text:
            return text, []
        content, rest = text.split(self.CALLS_BEGIN, 1)
        calls = []
        for seg in rest.split(self.CALL_BEGIN)[1:]:
            done = self.CALL_END in seg
            seg = seg.split(self.CALL_END)[0]
            if self.SEP not in seg:
                continue
            _typ, after = seg.split(self.SEP, 1)
            name, _, body = after.partition("\n")
            body = body.strip()
            if body.startswith("```json"):
                body = body[len("```json"):]
            body = body.strip()
            if body.endswith("```"):
                body = body[:-3].rstrip()
            atext, adone = _balanced_json_prefix(body) if body else ("", False)
            calls.append(ParsedCall(name.strip(), atext or "", done and adone))
        return content, calls


class DeepSeekV31ToolParser(DeepSeekV3ToolParser):
    """V3.1: ``<｜tool▁call▁begin｜>NAME<｜tool▁sep｜>{json}<｜tool▁call▁end｜>`` (no type tag, no code fence)."""

    def parse_partial(self, text):
        if self.CALLS_BEGIN not in text:
            return text, []
        content, rest = text.split(self.CALLS_BEGIN, 1)
        calls = []
        for seg in rest.split(self.CALL_BEGIN)[1:]:
            done = self.CALL_END in seg
            seg = seg.split(self.CALL_END)[0]
            if self.SEP not in seg:
                if seg.strip():
                    calls.append(ParsedCall(seg.strip(), "", False))
                continue
            name, body = seg.split(self.SEP, 1)
            atext, adone = _balanced_json_prefix(body) if body.strip() else ("", False)
            calls.append(ParsedCall(name.strip(), atext or "", done and adone))
        return content, calls


class DeepSeekV32ToolParser(ToolParser):
    """V3.2 "DSML" blocks: ``<｜DSML｜function_calls>`` containing ``<｜DSML｜invoke name="f">`` elements whose
    ``<｜DSML｜parameter name="p" string="true|false">value</｜DSML｜parameter>`` children carry the arguments."""
    BEGIN = "<｜DSML｜function_calls>"
    markers = (BEGIN,)

    def parse_partial(self, text):
        if self.BEGIN not in text:
            return text, []
        content, rest = text.split(self.BEGIN, 1)
        calls = []
        for m in re.finditer(r'<｜DSML｜invoke name="([^"]+)">(.*?)(</｜DSML｜invoke>|$)', rest, re.S):
            name, body, end = m.group(1), m.group(2), m.group(3)
            args = {}
            for pm in re.finditer(r'<｜DSML｜parameter name="([^"]+)"(?: string="(true|false)")?>(.*?)</｜DSML｜parameter>',
                                  body, re.S):
                key, is_str, val = pm.group(1), pm.group(2), pm.group(3)
                if is_str == "false":
                    try:
                        args[key] = json.loads(val)
                        continue
                    except Exception:
                        pass
                args[key] = val
            calls.append(ParsedCall(name, _json_args(args), bool(end)))
        return content, calls


class KimiK2ToolParser(ToolParser):
    """``<|tool_calls_section_begin|><|tool_call_begin|>functions.NAME:IDX<|tool_call_argument_begin|>{json}
    <|tool_call_end|>...<|tool_calls_section_end|>``."""
    SECTION = "<|tool_calls_section_begin|>"
    markers = (SECTION,)

    def parse_partial(self, text):
        if self.SECTION not in text:
            return text, []
        content, rest = text.split(self.SECTION, 1)
        calls = []
        for seg in rest.split("<|tool_call_begin|>")[1:]:
            done = "<|tool_call_end|>" in seg
            seg = seg.split("<|tool_call_end|>")[0]
            if "<|tool_call_argument_begin|>" not in seg:
                continue
            fid, body = seg.split("<|tool_call_argument_begin|>", 1)
            name = fid.strip()
            if name.startswith("functions."):
                name = name[len("functions."):]
            name = name.rsplit(":", 1)[0]
            atext, adone = _balanced_json_prefix(body) if body.strip() else ("", False)
            calls.append(ParsedCall(name, atext or "", done and adone))
        return content, calls


_PARSERS: Dict[str, Type[ToolParser]] = {
    "hermes": HermesToolParser,
    "llama": LlamaToolParser,
    "llama3_json": LlamaToolParser,
    "mistral": MistralToolParser,
    "internlm2": InternLM2ToolParser,
    "pythonic": PythonicToolParser,
    "llama4_pythonic": Llama4PythonicToolParser,
    "deepseekv3": DeepSeekV3ToolParser,
    "deepseekv31": DeepSeekV31ToolParser,
    "deepseekv32": DeepSeekV32ToolParser,
    "kimi_k2": KimiK2ToolParser,
}


def get_tool_parser(name: str) -> Type[ToolParser]:
    if name not in _PARSERS:
        raise KeyError(f"unknown tool parser {name!r}; available: {sorted(_PARSERS)}")
    return _PARSERS[name]


def register_tool_parser(name: str, cls: Type[ToolParser]) -> None:
    _PARSERS[name] = cls


def import_tool_parser_plugin(path: str) -> None:
    """``--tool-parser-plugin``: a Python file that calls ``register_tool_parser``."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("ksana_tool_parser_plugin", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
