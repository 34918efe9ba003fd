"""Per-request sampling configuration.

Field names follow the reference's ``sampling_config`` JSON object
(src/ksana_llm/python/ksana_llm/ksana_engine.py:179-241) and its C++ ``SamplingConfig`` validation
(src/ksana_llm/utils/request.cpp:11-35: 1 <= topk <= 1024; ``do_sample=False`` or ``topk == 1`` means
greedy).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class SamplingParams:
    topk: int = 1
    topp: float = 1.0
    temperature: float = 1.0
    max_new_tokens: int = 1024
    logprobs: int = 0
    repetition_penalty: float = 1.0
    no_repeat_ngram_size: int = 0
    encoder_no_repeat_ngram_size: int = 0
    decoder_no_repeat_ngram_size: int = 0
    num_beams: int = 1
    num_return_sequences: int = 1
    length_penalty: float = 1.0
    stop_token_ids: List[int] = field(default_factory=list)
    stop_strings: List[str] = field(default_factory=list)
    ignore_eos: bool = False
    do_sample: Optional[bool] = None
    enable_structured_output: bool = False
    json_schema: Optional[str] = None
    structured_output_regex: Optional[str] = None
    enable_thinking: Optional[bool] = None
    seed: Optional[int] = None
    # OpenAI-style controls (the reference's request converter forwards them: openaiapi/request_converter.py:175-211,
    # 394): additive penalties on tokens already generated, per-token bias, and a floor on the output length
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    logit_bias: Optional[dict] = None   # {token id (int or str): bias added to that logit}
    min_tokens: int = 0                 # EOS / stop tokens are not allowed before this many output tokens

    def verify(self) -> None:
        if not (1 <= self.topk <= 1024):
            raise ValueError("topk must be in [1, 1024]")
        if not (0.0 < self.topp <= 1.0):
            raise ValueError("topp must be in (0, 1]")
        if self.temperature < 0.0:
            raise ValueError("temperature must be >= 0")
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be >= 0")
        if self.repetition_penalty <= 0.0:
            raise ValueError("repetition_penalty must be > 0")
        if self.num_beams < 1 or self.num_return_sequences < 1:
            raise ValueError("num_beams and num_return_sequences must be >= 1")
        if self.num_beams > 1 and self.num_return_sequences > self.num_beams:
            raise ValueError("num_return_sequences must be <= num_beams")
        if self.logprobs < 0 or self.logprobs > 64:
            raise ValueError("logprobs must be in [0, 64]")
        if not (-2.0 <= self.presence_penalty <= 2.0) or not (-2.0 <= self.frequency_penalty <= 2.0):
            raise ValueError("presence_penalty and frequency_penalty must be in [-2, 2]")
        if self.min_tokens < 0 or self.min_tokens > self.max_new_tokens:
            raise ValueError("min_tokens must be in [0, max_new_tokens]")

    @property
    def use_greedy(self) -> bool:
        if self.num_beams > 1:
            return False
        if self.do_sample is False:
            return True
        return self.topk == 1 or self.temperature == 0.0

    @property
    def needs_logits_processing(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.no_repeat_ngram_size > 0 or
                self.presence_penalty != 0.0 or self.frequency_penalty != 0.0 or bool(self.logit_bias) or
                self.min_tokens > 0 or
                self.encoder_no_repeat_ngram_size > 0 or self.decoder_no_repeat_ngram_size > 0 or
                self.enable_structured_output or self.json_schema is not None or
                self.structured_output_regex is not None)

    @classmethod
    def from_dict(cls, d: Optional[Dict[str, Any]]) -> "SamplingParams":
        d = dict(d or {})
        names = set(cls.__dataclass_fields__.keys())
        alias = {"top_k": "topk", "top_p": "topp", "max_tokens": "max_new_tokens", "stop": "stop_strings"}
        kw = {}
        for k, v in d.items():
            k = alias.get(k, k)
            if k in names and v is not None:
                kw[k] = v
        sp = cls(**kw)
        if isinstance(sp.stop_strings, str):
            sp.stop_strings = [sp.stop_strings]
        if isinstance(sp.json_schema, dict):
            import json
            sp.json_schema = json.dumps(sp.json_schema)
        sp.verify()
        return sp
