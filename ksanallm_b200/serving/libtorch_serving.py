"""The blocking serving surface of the reference's extension module, over this engine.

The reference's Python package talks to its C++ runtime through one extension module whose names user code and the
server both rely on (src/ksana_llm/torch_op/serving_op.cpp:80-255: ``Serving`` with ``init_serving`` / ``generate`` /
``generate_streaming`` / ``forward``, the value classes ``KsanaPythonInput``, ``SamplingConfig``, ``EmbeddingSlice``,
``TargetDescribe``, ``PythonTensor``, ``KsanaPythonOutput``, ``StreamingIterator.GetNext``, ``EndpointConfig``, the
enums ``RetCode``, ``TokenReduceMode``, ``EndpointType``). A program written against that module runs here with::

    from ksanallm_b200.serving import libtorch_serving
    serving = libtorch_serving.Serving()
    serving.init_serving("config.yaml")
    status, out = serving.generate(libtorch_serving.KsanaPythonInput(...), {})

Calls block the calling thread (the extension releases the GIL while it waits; here the engine's own step thread does
the work and the caller sleeps on the request's condition variable), and may be issued from many threads at once.
"""
from __future__ import annotations

import asyncio
import threading
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .ksana_engine import EngineArgs, KsanaLLMEngine, KsanaPythonOutput, RetCode, Status  # noqa: F401  (re-exported)


class TokenReduceMode:
    GATHER_ALL = "GATHER_ALL"
    GATHER_TOKEN_ID = "GATHER_TOKEN_ID"


class EndpointType:
    LOCAL = "LOCAL"
    RPC = "RPC"


@dataclass
class SamplingConfig:
    topk: int = 1
    topp: float = 0.0
    temperature: float = 0.0
    max_new_tokens: int = 1024
    logprobs_num: int = 0
    repetition_penalty: float = 1.0
    no_repeat_ngram_size: int = 0
    encoder_no_repeat_ngram_size: int = 0
    decoder_no_repeat_ngram_size: int = 0
    num_beams: int = 1
    num_return_sequences: int = 1
    length_penalty: float = 1.0
    stop_token_ids: List[int] = field(default_factory=list)
    ignore_eos: bool = False
    stop_strings: List[str] = field(default_factory=list)
    enable_structured_output: bool = False
    json_schema: str = ""
    enable_thinking: Optional[bool] = None


@dataclass
class EmbeddingSlice:
    pos: List[int] = field(default_factory=list)
    embeddings: List[List[float]] = field(default_factory=list)
    embedding_tensors: List[Any] = field(default_factory=list)  # torch tensors [n, hidden], one per position
    additional_tensors: List[Any] = field(default_factory=list)


@dataclass
class TargetDescribe:
    token_id: List[int] = field(default_factory=list)
    slice_pos: List[Tuple[int, int]] = field(default_factory=list)
    token_reduce_mode: str = TokenReduceMode.GATHER_ALL


@dataclass
class PythonTensor:
    data: bytes = b""
    shape: List[int] = field(default_factory=list)
    dtype: str = "float32"


@dataclass
class KsanaPythonInput:
    model_name: str = ""
    sampling_config: SamplingConfig = field(default_factory=SamplingConfig)
    input_tokens: List[int] = field(default_factory=list)
    request_target: Dict[str, TargetDescribe] = field(default_factory=dict)
    input_refit_embedding: EmbeddingSlice = field(default_factory=EmbeddingSlice)
    structured_output_regex: str = ""


@dataclass
class EndpointConfig:
    type: str = EndpointType.LOCAL
    rpc_plugin_name: str = ""
    host: str = "0.0.0.0"
    port: int = 8080
    access_log: bool = True


class StreamingIterator:
    """``GetNext()`` blocks until the request has produced more tokens and returns ``(Status, KsanaPythonOutput)``;
    after the last item it returns a ``RET_STOP_ITERATION`` status with ``None``."""

    def __init__(self, engine: KsanaLLMEngine, req):
        self._engine, self._req = engine, req
        self._version, self._done = -1, False

    def GetNext(self):  # noqa: N802  (name kept for API compatibility)
        if self._done:
            return Status(RetCode.RET_STOP_ITERATION, "iteration finished"), None
        req = self._req
        seen = self._version
        while self._version == seen and not req.finished:
            self._version = req.wait(seen, 1.0)
        out = self._engine._snapshot(req)
        if req.finished:
            self._done = True
        return out.finish_status, out

    def abort(self) -> None:
        if not self._req.finished:
            self._engine.llm.abort(self._req)
        self._done = True


def _request_dict(inp: KsanaPythonInput) -> Dict[str, Any]:
    sc = inp.sampling_config
    cfg = {k: getattr(sc, k) for k in sc.__dataclass_fields__ if getattr(sc, k) is not None}
    # the extension's defaults (topp 0, temperature 0) mean "not set": the engine's own defaults apply
    for k in ("topp", "temperature"):
        if cfg.get(k, 0) <= 0:
            cfg.pop(k, None)
    d: Dict[str, Any] = {"input_tokens": list(inp.input_tokens), "sampling_config": cfg}
    if inp.structured_output_regex:
        d["structured_output_regex"] = inp.structured_output_regex
    emb = inp.input_refit_embedding
    if emb.pos and (emb.embeddings or emb.embedding_tensors):
        d["input_refit_embedding"] = {"pos": list(emb.pos),
                                      "embeddings": list(emb.embedding_tensors) or list(emb.embeddings)}
    if inp.request_target:
        d["request_target"] = [{"target_name": name, "token_id": list(t.token_id),
                                "slice_pos": [list(p) for p in t.slice_pos], "token_reduce_mode": t.token_reduce_mode}
                               for name, t in inp.request_target.items()]
    return d


class Serving:
    def __init__(self):
        self.endpoint_config = EndpointConfig()
        self.engine: Optional[KsanaLLMEngine] = None
        self._loop = asyncio.new_event_loop()
        self._thread: Optional[threading.Thread] = None

    # the engine's public calls are coroutines: one private event loop thread runs them for the blocking callers
    def _run(self, coro):
        if self._thread is None:
            self._thread = threading.Thread(target=self._loop.run_forever, name="ksana-serving-loop", daemon=True)
            self._thread.start()
        return asyncio.run_coroutine_threadsafe(coro, self._loop).result()

    def init_serving(self, config_file: str, reasoning_config: Optional[Dict[str, Any]] = None, **overrides) -> None:
        """``overrides``: fields of EngineArgs (e.g. ``synthetic_model=...``, ``device=...``) for use without a
        checkpoint directory."""
        args = EngineArgs.from_config_file(config_file, **overrides) if config_file else EngineArgs(
            config_file="", **overrides)
        self.engine = KsanaLLMEngine(args)
        self.engine.initialize()
        if reasoning_config and reasoning_config.get("think_end_token_id") is not None:
            self.engine.think_end_token_id = int(reasoning_config["think_end_token_id"])

    def generate(self, ksana_python_input: KsanaPythonInput, req_ctx: Optional[Dict[str, str]] = None):
        return self._run(self.engine.generate(_request_dict(ksana_python_input), streamer=False, req_ctx=req_ctx))

    def generate_streaming(self, ksana_python_input: KsanaPythonInput, req_ctx: Optional[Dict[str, str]] = None):
        status, it = self._run(self.engine.generate(_request_dict(ksana_python_input), streamer=True, req_ctx=req_ctx))
        if not status.OK() or it is None:
            return status, None
        req = getattr(it, "req", None)
        if req is None:  # an answer that is already complete (prefill-only instance)
            return status, _Finished(it)
        it.detached = True  # the blocking iterator takes over: the async one must not abort the request when dropped
        return status, StreamingIterator(self.engine, req)

    def forward(self, request_bytes: bytes, req_ctx: Optional[Dict[str, str]] = None):
        status, data = self._run(self.engine.forward(request_bytes, req_ctx))
        return status, (data or b"")

    def shutdown(self) -> None:
        if self.engine is not None:
            self.engine.shutdown()
        if self._thread is not None:
            self._loop.call_soon_threadsafe(self._loop.stop)
            self._thread.join(timeout=5)
            self._thread = None


class _Finished:
    def __init__(self, it):
        self._out, self._done = it.out, False

    def GetNext(self):  # noqa: N802
        if self._done:
            return Status(RetCode.RET_STOP_ITERATION, "iteration finished"), None
        self._done = True
        return self._out.finish_status, self._out
