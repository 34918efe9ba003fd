"""Tokenizer processor: HF tokenizer load, chat templates, incremental decode for streaming.

Reference: src/ksana_llm/python/ksana_llm/processor_op_base.py:73-163. A byte-level stand-in tokenizer is used
when a model directory ships no tokenizer files (synthetic-weight runs, tests).
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional, Sequence


class ByteTokenizer:
    """UTF-8 bytes + 3 (ids 0..2 are pad / bos / eos). Deterministic, no files needed."""

    bos_token_id, eos_token_id, pad_token_id = 1, 2, 0
    chat_template = None

    def __init__(self, vocab_size: int = 32000):
        self.vocab_size = vocab_size

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        ids = [b + 3 for b in text.encode("utf-8")]
        return ([self.bos_token_id] if add_special_tokens else []) + ids

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        bs = bytes((i - 3) & 0xFF for i in ids if i >= 3 and i < 259)
        return bs.decode("utf-8", errors="replace")

    def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True, **kw):
        text = "".join(f"<|{m['role']}|>\n{_content_text(m.get('content'))}\n" for m in messages)
        if add_generation_prompt:
            text += "<|assistant|>\n"
        return self.encode(text) if tokenize else text

    def convert_ids_to_tokens(self, ids):
        return [self.decode([i]) for i in ids]

    def get_vocab(self) -> Dict[str, int]:
        return {chr(i): i + 3 for i in range(256)}


def _content_text(content) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    parts = []
    for c in content:
        if isinstance(c, dict) and c.get("type") == "text":
            parts.append(c.get("text", ""))
    return "".join(parts)


class TokenizerProcessor:
    def __init__(self, tokenizer_path: Optional[str], vocab_size: int = 32000, add_special_tokens: bool = True,
                 skip_special_tokens: bool = True, chat_template: Optional[str] = None):
        self.add_special_tokens = add_special_tokens
        self.skip_special_tokens = skip_special_tokens
        self.tokenizer = None
        if tokenizer_path and os.path.isdir(tokenizer_path) and any(
                os.path.exists(os.path.join(tokenizer_path, f)) for f in
                ("tokenizer.json", "tokenizer.model", "vocab.json", "tokenizer_config.json")):
            from transformers import AutoTokenizer
            self.tokenizer = AutoTokenizer.from_pretrained(tokenizer_path, trust_remote_code=True)
        if self.tokenizer is None:
            self.tokenizer = ByteTokenizer(vocab_size)
        if chat_template:
            if os.path.isfile(chat_template):
                with open(chat_template, "r", encoding="utf-8") as f:
                    chat_template = f.read()
            self.tokenizer.chat_template = chat_template

    @property
    def eos_token_id(self):
        return getattr(self.tokenizer, "eos_token_id", None)

    def encode(self, prompt: str, add_special_tokens: Optional[bool] = None) -> List[int]:
        ast = self.add_special_tokens if add_special_tokens is None else add_special_tokens
        return list(self.tokenizer.encode(prompt, add_special_tokens=ast))

    def decode(self, ids: Sequence[int], skip_special_tokens: Optional[bool] = None) -> str:
        sst = self.skip_special_tokens if skip_special_tokens is None else skip_special_tokens
        return self.tokenizer.decode(list(ids), skip_special_tokens=sst)

    def apply_chat_template(self, messages: List[Dict[str, Any]], add_generation_prompt: bool = True,
                            tools: Optional[List[Dict[str, Any]]] = None, **kwargs) -> str:
        kw = dict(kwargs)
        if tools:
            kw["tools"] = tools
        return self.tokenizer.apply_chat_template(messages, tokenize=False,
                                                  add_generation_prompt=add_generation_prompt, **kw)


class IncrementalDetokenizer:
    """Streams text deltas without re-decoding the whole output and without emitting broken UTF-8:
    decodes a sliding window [prefix_offset, end) and only releases text once it no longer ends in U+FFFD."""

    def __init__(self, proc: TokenizerProcessor):
        self.proc = proc
        self.tokens: List[int] = []
        self.prefix_offset = 0
        self.read_offset = 0
        self.text = ""

    def push(self, new_tokens: Sequence[int]) -> str:
        self.tokens.extend(new_tokens)
        prefix_text = self.proc.decode(self.tokens[self.prefix_offset:self.read_offset])
        new_text = self.proc.decode(self.tokens[self.prefix_offset:])
        if len(new_text) > len(prefix_text) and not new_text.endswith("�"):
            delta = new_text[len(prefix_text):]
            self.prefix_offset = self.read_offset
            self.read_offset = len(self.tokens)
            self.text += delta
            return delta
        return ""
