"""Structured (grammar-constrained) generation.

Per request a grammar (JSON schema, free JSON, or a regular expression) is compiled once with xgrammar and one
matcher per output sequence produces the token bitmask that the batched sampler applies on the device. While a
reasoning model is still inside its thinking section (before ``think_end_token_id``) no mask is applied.
Reference: src/ksana_llm/runtime/structured_generation/* and generation_controller.cpp:11-38.
"""
from __future__ import annotations

import json
from typing import Dict, List, Optional

import numpy as np


class _TokenizerInfoCache:
    cache: Dict[int, object] = {}

    @classmethod
    def get(cls, tokenizer, vocab_size: int):
        import xgrammar as xgr
        key = id(tokenizer)
        if key not in cls.cache:
            tok = getattr(tokenizer, "tokenizer", tokenizer)
            info = None
            try:
                if hasattr(tok, "backend_tokenizer") or hasattr(tok, "vocab_file"):
                    info = xgr.TokenizerInfo.from_huggingface(tok, vocab_size=vocab_size)
            except Exception:
                info = None
            if info is None:
                vocab = [""] * vocab_size
                for s, i in tok.get_vocab().items():
                    if 0 <= i < vocab_size:
                        vocab[i] = s
                stop = [t for t in [getattr(tok, "eos_token_id", None)] if t is not None]
                info = xgr.TokenizerInfo(vocab, vocab_type=xgr.VocabType.RAW, vocab_size=vocab_size,
                                         stop_token_ids=stop)
            cls.cache[key] = (info, xgr.GrammarCompiler(info))
        return cls.cache[key]


class GrammarState:
    """Grammar shared by all output sequences of one request; one matcher per sequence."""

    def __init__(self, compiled, vocab_size: int, think_end_token_id: Optional[int] = None):
        self.compiled = compiled
        self.vocab_size = vocab_size
        self.think_end = think_end_token_id
        self.matchers: Dict[int, object] = {}
        self.thinking: Dict[int, bool] = {}
        self.words = (vocab_size + 31) // 32

    def _matcher(self, seq_id: int):
        import xgrammar as xgr
        m = self.matchers.get(seq_id)
        if m is None:
            m = self.matchers[seq_id] = xgr.GrammarMatcher(self.compiled)
            self.thinking[seq_id] = self.think_end is not None
        return m

    def next_bitmask(self, seq_id: int) -> Optional[np.ndarray]:
        import xgrammar as xgr
        m = self._matcher(seq_id)
        if self.thinking.get(seq_id):
            return None
        if m.is_terminated():
            return None
        bm = xgr.allocate_token_bitmask(1, self.vocab_size)
        m.fill_next_token_bitmask(bm, 0)
        return bm[0].numpy().astype(np.int32)

    def accept(self, seq_id: int, token: int) -> bool:
        m = self._matcher(seq_id)
        if self.thinking.get(seq_id):
            if token == self.think_end:
                self.thinking[seq_id] = False
            return True
        if m.is_terminated():
            return True
        return bool(m.accept_token(int(token)))

    def is_terminated(self, seq_id: int) -> bool:
        m = self.matchers.get(seq_id)
        return bool(m is not None and not self.thinking.get(seq_id) and m.is_terminated())


def build_grammar(params, tokenizer, vocab_size: int, think_end_token_id: Optional[int] = None) -> GrammarState:
    _, compiler = _TokenizerInfoCache.get(tokenizer, vocab_size)
    if params.json_schema:
        schema = params.json_schema if isinstance(params.json_schema, str) else json.dumps(params.json_schema)
        compiled = compiler.compile_json_schema(schema)
    elif params.structured_output_regex:
        compiled = compiler.compile_regex(params.structured_output_regex)
    else:
        compiled = compiler.compile_builtin_json_grammar()
    return GrammarState(compiled, vocab_size, think_end_token_id)
