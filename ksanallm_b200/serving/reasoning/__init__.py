"""Reasoning ("thinking") parsers: split model output into ``reasoning_content`` and ``content``.

Same parser names as the reference (src/ksana_llm/python/openaiapi/reasoning/: deepseek_r1, deepseek_v3, qwen3).
All three families delimit the reasoning with ``<think>`` ... ``</think>``; they differ in whether the opening tag
is part of the prompt template (DeepSeek-R1: the model starts inside the thinking section) and in whether
thinking can be switched off per request (Qwen3 / DeepSeek-V3.1 ``enable_thinking``).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple, Type


class ReasoningParser:
    start_token = "<think>"
    end_token = "</think>"
    starts_in_reasoning = False

    def __init__(self, tokenizer=None):
        self.tokenizer = tokenizer
        self.think_start_token_id = self._tid(self.start_token)
        self.think_end_token_id = self._tid(self.end_token)

    def _tid(self, tok: str) -> Optional[int]:
        t = self.tokenizer
        if t is None:
            return None
        try:
            vocab = t.get_vocab()
            if tok in vocab:
                return int(vocab[tok])
            ids = t.encode(tok, add_special_tokens=False)
            return int(ids[0]) if len(ids) == 1 else None
        except Exception:
            return None

    def in_reasoning_at_start(self, enable_thinking: Optional[bool]) -> bool:
        return self.starts_in_reasoning and enable_thinking is not False

    # ---- whole-text split ------------------------------------------------------------------------------------
    def extract(self, text: str, enable_thinking: Optional[bool] = None) -> Tuple[Optional[str], Optional[str]]:
        """Returns (reasoning_content, content)."""
        s, e = self.start_token, self.end_token
        if s in text:
            text = text.split(s, 1)[1]
            inside = True
        else:
            inside = self.in_reasoning_at_start(enable_thinking) or e in text
        if not inside:
            return None, text
        if e in text:
            r, c = text.split(e, 1)
            return (r or None), (c or None)
        return (text or None), None

    # ---- streaming split ---------------------------------------------------------------------------------------
    def new_stream_state(self, enable_thinking: Optional[bool] = None) -> Dict:
        # "head": nothing emitted yet - a model that starts in reasoning mode may still write the opening tag itself
        return {"mode": "reasoning" if self.in_reasoning_at_start(enable_thinking) else "unknown", "buf": "",
                "head": True}

    def extract_streaming(self, state: Dict, delta: str) -> Tuple[Optional[str], Optional[str]]:
        """Feeds one text delta, returns (reasoning_delta, content_delta). Tags split across deltas are handled by
        holding back a possible tag prefix."""
        state["buf"] += delta
        r_out, c_out = "", ""
        while True:
            buf = state["buf"]
            if state["mode"] == "content":
                c_out += buf
                state["buf"] = ""
                break
            if state["mode"] == "unknown":
                stripped = buf.lstrip()
                if stripped.startswith(self.start_token):
                    state["buf"] = stripped[len(self.start_token):]
                    state["mode"] = "reasoning"
                    continue
                if self.start_token.startswith(stripped) and len(stripped) < len(self.start_token):
                    break  # might still become the tag
                state["mode"] = "content" if self.end_token not in buf else "reasoning"
                continue
            # reasoning
            if state.get("head"):
                stripped = buf.lstrip()
                if stripped.startswith(self.start_token):
                    buf = state["buf"] = stripped[len(self.start_token):]
                    state["head"] = False
                elif stripped and self.start_token.startswith(stripped):
                    break  # might still become the opening tag
                elif stripped:
                    state["head"] = False
            i = buf.find(self.end_token)
            if i >= 0:
                r_out += buf[:i]
                state["buf"] = buf[i + len(self.end_token):]
                state["mode"] = "content"
                continue
            hold = 0
            for k in range(min(len(self.end_token) - 1, len(buf)), 0, -1):
                if self.end_token.startswith(buf[-k:]):
                    hold = k
                    break
            r_out += buf[:len(buf) - hold]
            state["buf"] = buf[len(buf) - hold:]
            break
        return (r_out or None), (c_out or None)


class DeepSeekR1ReasoningParser(ReasoningParser):
    starts_in_reasoning = True


class DeepSeekV3ReasoningParser(ReasoningParser):
    """DeepSeek-V3.1 style: thinking only when the request enables it."""

    def in_reasoning_at_start(self, enable_thinking):
        return bool(enable_thinking)


class Qwen3ReasoningParser(ReasoningParser):
    """Qwen3: the template emits <think> itself unless thinking is disabled."""

    def in_reasoning_at_start(self, enable_thinking):
        return False


_PARSERS: Dict[str, Type[ReasoningParser]] = {
    "deepseek_r1": DeepSeekR1ReasoningParser,
    "deepseek_v3": DeepSeekV3ReasoningParser,
    "qwen3": Qwen3ReasoningParser,
}


def get_reasoning_parser(name: str) -> Type[ReasoningParser]:
    if name not in _PARSERS:
        raise KeyError(f"unknown reasoning parser {name!r}; available: {sorted(_PARSERS)}")
    return _PARSERS[name]


def register_reasoning_parser(name: str, cls: Type[ReasoningParser]) -> None:
    _PARSERS[name] = cls
