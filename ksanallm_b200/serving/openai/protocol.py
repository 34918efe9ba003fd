"""OpenAI-compatible request / response models (chat completions, completions, embeddings, models).

Field coverage follows the vLLM-style protocol classes the reference ships
(src/ksana_llm/python/openaiapi/openai_protocol.py:223-671); unknown fields are accepted and ignored.
"""
from __future__ import annotations

import time
import uuid
from typing import Any, Dict, List, Literal, Optional, Union

from pydantic import BaseModel, ConfigDict, Field


class OpenAIBase(BaseModel):
    model_config = ConfigDict(extra="allow")


def _id(prefix: str) -> str:
    return f"{prefix}-{uuid.uuid4().hex}"


class ErrorResponse(OpenAIBase):
    object: str = "error"
    message: str
    type: str = "invalid_request_error"
    param: Optional[str] = None
    code: int = 400


class ModelCard(OpenAIBase):
    id: str
    object: str = "model"
    created: int = Field(default_factory=lambda: int(time.time()))
    owned_by: str = "ksanallm_b200"
    root: Optional[str] = None
    parent: Optional[str] = None
    max_model_len: Optional[int] = None


class ModelList(OpenAIBase):
    object: str = "list"
    data: List[ModelCard] = Field(default_factory=list)


class UsageInfo(OpenAIBase):
    prompt_tokens: int = 0
    total_tokens: int = 0
    completion_tokens: Optional[int] = 0


class FunctionDef(OpenAIBase):
    name: str
    description: Optional[str] = None
    parameters: Optional[Dict[str, Any]] = None


class ToolDef(OpenAIBase):
    type: Literal["function"] = "function"
    function: FunctionDef


class ResponseFormat(OpenAIBase):
    type: Literal["text", "json_object", "json_schema"] = "text"
    json_schema: Optional[Dict[str, Any]] = None


class StreamOptions(OpenAIBase):
    include_usage: Optional[bool] = False
    continuous_usage_stats: Optional[bool] = False


class ChatCompletionRequest(OpenAIBase):
    messages: List[Dict[str, Any]]
    model: Optional[str] = None
    frequency_penalty: Optional[float] = 0.0
    logit_bias: Optional[Dict[str, float]] = None
    logprobs: Optional[bool] = False
    top_logprobs: Optional[int] = 0
    max_tokens: Optional[int] = None
    max_completion_tokens: Optional[int] = None
    n: Optional[int] = 1
    presence_penalty: Optional[float] = 0.0
    min_tokens: Optional[int] = 0
    response_format: Optional[ResponseFormat] = None
    seed: Optional[int] = None
    stop: Optional[Union[str, List[str]]] = None
    stream: Optional[bool] = False
    stream_options: Optional[StreamOptions] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    tools: Optional[List[ToolDef]] = None
    tool_choice: Optional[Union[Literal["none", "auto", "required"], Dict[str, Any]]] = None
    user: Optional[str] = None
    # extensions
    repetition_penalty: Optional[float] = None
    stop_token_ids: Optional[List[int]] = None
    ignore_eos: Optional[bool] = False
    use_beam_search: Optional[bool] = False
    best_of: Optional[int] = None
    length_penalty: Optional[float] = 1.0
    add_generation_prompt: Optional[bool] = True
    chat_template: Optional[str] = None
    chat_template_kwargs: Optional[Dict[str, Any]] = None
    guided_json: Optional[Union[str, Dict[str, Any]]] = None
    guided_regex: Optional[str] = None
    enable_thinking: Optional[bool] = None
    skip_special_tokens: Optional[bool] = True


class CompletionRequest(OpenAIBase):
    prompt: Union[str, List[str], List[int], List[List[int]]]
    model: Optional[str] = None
    best_of: Optional[int] = None
    echo: Optional[bool] = False
    frequency_penalty: Optional[float] = 0.0
    logprobs: Optional[int] = None
    max_tokens: Optional[int] = 16
    n: Optional[int] = 1
    presence_penalty: Optional[float] = 0.0
    min_tokens: Optional[int] = 0
    seed: Optional[int] = None
    stop: Optional[Union[str, List[str]]] = None
    stream: Optional[bool] = False
    stream_options: Optional[StreamOptions] = None
    suffix: Optional[str] = None
    temperature: Optional[float] = None
    top_p: Optional[float] = None
    top_k: Optional[int] = None
    user: Optional[str] = None
    repetition_penalty: Optional[float] = None
    stop_token_ids: Optional[List[int]] = None
    ignore_eos: Optional[bool] = False
    use_beam_search: Optional[bool] = False
    length_penalty: Optional[float] = 1.0
    response_format: Optional[ResponseFormat] = None
    guided_json: Optional[Union[str, Dict[str, Any]]] = None
    guided_regex: Optional[str] = None


class EmbeddingRequest(OpenAIBase):
    input: Union[str, List[str], List[int], List[List[int]]]
    model: Optional[str] = None
    encoding_format: Literal["float", "base64"] = "float"
    dimensions: Optional[int] = None
    user: Optional[str] = None
