"""OpenAI-compatible routes on top of :class:`KsanaLLMEngine`:
``POST /v1/chat/completions`` (SSE streaming, tools, reasoning content, logprobs, response_format),
``POST /v1/completions``, ``POST /v1/embeddings``, ``GET /v1/models`` and ``GET /v1/models/{id}`` (also without
the ``/v1`` prefix). Reference: src/ksana_llm/python/openaiapi/openai_adapter.py:847-874, serving_chat.py,
serving_completion.py, serving_embedding.py, serving_models.py, request_converter.py.
"""
from __future__ import annotations

import base64
import json
import os
import struct
import time
from typing import Any, Dict, List, Optional

from fastapi import Request
from fastapi.responses import JSONResponse, StreamingResponse

from ..tokenizer import IncrementalDetokenizer
from .protocol import (ChatCompletionRequest, CompletionRequest, EmbeddingRequest, ErrorResponse, ModelCard,
                       ModelList, UsageInfo, _id)


def _err(msg: str, code: int = 400, typ: str = "invalid_request_error") -> JSONResponse:
    return JSONResponse(ErrorResponse(message=msg, code=code, type=typ).model_dump(), status_code=code)


def _sse(obj: Dict[str, Any]) -> bytes:
    return b"data: " + json.dumps(obj, ensure_ascii=False).encode("utf-8") + b"\n\n"


class OpenAIServing:
    def __init__(self, engine, args):
        self.engine = engine
        self.args = args
        self.model_name = os.path.basename(os.path.normpath(args.model_dir)) if args.model_dir else \
            (args.synthetic_model or "ksana-model")
        self.tool_parser_cls = None
        self.reasoning_parser_cls = None
        if args.tool_parser_plugin:
            from ..tool_parsers import import_tool_parser_plugin
            import_tool_parser_plugin(args.tool_parser_plugin)
        if args.tool_call_parser:
            from ..tool_parsers import get_tool_parser
            self.tool_parser_cls = get_tool_parser(args.tool_call_parser)
        if args.reasoning_parser:
            from ..reasoning import get_reasoning_parser
            self.reasoning_parser_cls = get_reasoning_parser(args.reasoning_parser)

    # ---- request conversion --------------------------------------------------------------------------------------
    def _sampling_config(self, r, n_logprobs: int) -> Dict[str, Any]:
        greedy = (r.temperature is not None and r.temperature == 0.0)
        sc: Dict[str, Any] = {
            "temperature": 1.0 if r.temperature is None or greedy else r.temperature,
            "topp": 1.0 if r.top_p is None else r.top_p,
            "topk": 1 if greedy else (r.top_k if r.top_k and r.top_k > 0 else 1024),
            "max_new_tokens": getattr(r, "max_completion_tokens", None) or r.max_tokens or
            self.engine.serving.setting.batch_scheduler.max_token_len // 2,
            "logprobs": n_logprobs,
            "num_return_sequences": r.n or 1,
            "ignore_eos": bool(r.ignore_eos),
            "stop_token_ids": list(r.stop_token_ids or []),
            "stop_strings": [r.stop] if isinstance(r.stop, str) else list(r.stop or []),
            "do_sample": not greedy,
        }
        if r.temperature is None and r.top_p is None and r.top_k is None:
            sc["topk"], sc["do_sample"] = 1, False  # the engine's default is greedy
        if r.repetition_penalty:
            sc["repetition_penalty"] = r.repetition_penalty
        for name in ("presence_penalty", "frequency_penalty", "min_tokens"):
            v = getattr(r, name, None)
            if v:
                sc[name] = v
        if getattr(r, "logit_bias", None):
            sc["logit_bias"] = {int(k): float(v) for k, v in r.logit_bias.items()}
        if r.seed is not None:
            sc["seed"] = r.seed
        if r.use_beam_search:
            sc["num_beams"] = max(r.best_of or r.n or 1, r.n or 1)
            sc["length_penalty"] = r.length_penalty or 1.0
        rf = r.response_format
        if rf is not None and rf.type == "json_object":
            sc["enable_structured_output"] = True
        elif rf is not None and rf.type == "json_schema" and rf.json_schema:
            schema = rf.json_schema.get("schema", rf.json_schema)
            sc["json_schema"] = json.dumps(schema)
        if getattr(r, "guided_json", None):
            gj = r.guided_json
            sc["json_schema"] = gj if isinstance(gj, str) else json.dumps(gj)
        if getattr(r, "guided_regex", None):
            sc["structured_output_regex"] = r.guided_regex
        return sc

    @staticmethod
    def _normalise_messages(messages: List[Dict[str, Any]], content_format: str) -> List[Dict[str, Any]]:
        """``string`` format flattens [{type: text, text: ...}] parts into one string (what most templates expect)."""
        out = []
        for m in messages:
            m = dict(m)
            c = m.get("content")
            if isinstance(c, list) and content_format in ("auto", "string"):
                texts = [p.get("text", "") for p in c if isinstance(p, dict) and p.get("type") == "text"]
                if len(texts) == len(c) or content_format == "string":
                    m["content"] = "\n".join(texts)
            out.append(m)
        return out

    def _logprob_entries(self, lp_list, tok) -> List[Dict[str, Any]]:
        ents = []
        for e in lp_list or []:
            t = tok.decode([e["token"]])
            ents.append({"token": t, "logprob": e["logprob"], "bytes": list(t.encode("utf-8")),
                         "top_logprobs": [{"token": tok.decode([i]), "logprob": v,
                                           "bytes": list(tok.decode([i]).encode("utf-8"))} for i, v in (e["top"] or [])]})
        return ents

    # ---- /v1/chat/completions --------------------------------------------------------------------------------------
    async def chat(self, raw: Request):
        try:
            r = ChatCompletionRequest(**(await raw.json()))
        except Exception as ex:
            return _err(f"invalid request: {ex}")
        tok = self.engine.tokenizer
        tools = [t.model_dump() for t in r.tools] if r.tools else None
        use_tools = bool(tools) and r.tool_choice != "none" and self.tool_parser_cls is not None and \
            (self.args.enable_auto_tool_choice or isinstance(r.tool_choice, dict) or r.tool_choice == "required")
        try:
            msgs = self._normalise_messages(r.messages, self.args.chat_template_content_format)
            kw = dict(r.chat_template_kwargs or {})
            enable_thinking = r.enable_thinking if r.enable_thinking is not None else kw.get("enable_thinking")
            if enable_thinking is not None:
                kw["enable_thinking"] = enable_thinking
            if r.chat_template:
                kw["chat_template"] = r.chat_template
            prompt = tok.apply_chat_template(msgs, bool(r.add_generation_prompt), tools if tools else None, **kw)
            input_tokens = tok.encode(prompt, add_special_tokens=False)
        except Exception as ex:
            return _err(f"chat template failed: {ex}")
        n_lp = max(int(r.top_logprobs or 0), 1) if r.logprobs else 0
        req_dict = {"input_tokens": input_tokens, "sampling_config": self._sampling_config(r, n_lp)}
        if any(isinstance(m.get("content"), list) and any(isinstance(p, dict) and p.get("type") != "text"
                                                          for p in m["content"]) for m in r.messages):
            # image / video / audio parts: the model's plugin turns them into spliced embeddings
            # (reference: openaiapi/request_converter.py multimodal message parsing -> plugin preprocess)
            req_dict["messages"] = r.messages
        if enable_thinking is not None:
            req_dict["sampling_config"]["enable_thinking"] = enable_thinking
        rid, created = _id("chatcmpl"), int(time.time())
        model = r.model or self.model_name
        status, out = await self.engine.generate(req_dict, streamer=bool(r.stream), req_ctx={})
        if not status.OK():
            return _err(status.GetMessage(), 500 if status.GetCode().value >= 4 else 400, "engine_error")

        if not r.stream:
            choices = []
            comp_tokens = 0
            for i, toks in enumerate(out.output_tokens):
                text = tok.decode(toks)
                comp_tokens += len(toks)
                reasoning, content = (None, text)
                if self.reasoning_parser_cls is not None:
                    reasoning, content = self.reasoning_parser_cls(tok.tokenizer).extract(text, enable_thinking)
                msg: Dict[str, Any] = {"role": "assistant", "content": content}
                if reasoning is not None:
                    msg["reasoning_content"] = reasoning
                finish = (out.finish_reasons[i] if i < len(out.finish_reasons) else None) or "stop"
                if use_tools and content:
                    ext = self.tool_parser_cls(tok.tokenizer).extract_tool_calls(content, r)
                    if ext.tools_called:
                        msg["content"], msg["tool_calls"], finish = ext.content, ext.tool_calls, "tool_calls"
                ch: Dict[str, Any] = {"index": i, "message": msg, "finish_reason": finish, "logprobs": None}
                if n_lp and out.logprobs:
                    ch["logprobs"] = {"content": self._logprob_entries(out.logprobs[i], tok)}
                choices.append(ch)
            usage = UsageInfo(prompt_tokens=len(input_tokens), completion_tokens=comp_tokens,
                              total_tokens=len(input_tokens) + comp_tokens)
            return JSONResponse({"id": rid, "object": "chat.completion", "created": created, "model": model,
                                 "choices": choices, "usage": usage.model_dump()})

        async def gen():
            n = r.n or 1
            detoks: Dict[int, IncrementalDetokenizer] = {}
            sent: Dict[int, int] = {}
            full: Dict[int, str] = {}
            tparsers: Dict[int, Any] = {}
            rstates: Dict[int, Any] = {}
            rparser = self.reasoning_parser_cls(tok.tokenizer) if self.reasoning_parser_cls else None
            finished_idx = set()
            comp_tokens = 0
            for i in range(n):
                yield _sse({"id": rid, "object": "chat.completion.chunk", "created": created, "model": model,
                            "choices": [{"index": i, "delta": {"role": "assistant", "content": ""},
                                         "finish_reason": None}]})
            async for o in out:
                for i, toks in enumerate(o.output_tokens):
                    if i in finished_idx:
                        continue
                    d = detoks.setdefault(i, IncrementalDetokenizer(tok))
                    new = toks[sent.get(i, 0):]
                    sent[i] = len(toks)
                    comp_tokens += len(new)
                    delta_text = d.push(new) if new else ""
                    delta: Dict[str, Any] = {}
                    content_delta = delta_text
                    if rparser is not None and delta_text:
                        st = rstates.setdefault(i, rparser.new_stream_state(enable_thinking))
                        rd, content_delta = rparser.extract_streaming(st, delta_text)
                        if rd:
                            delta["reasoning_content"] = rd
                        content_delta = content_delta or ""
                    if content_delta:
                        prev = full.get(i, "")
                        full[i] = prev + content_delta
                        if use_tools:
                            tp = tparsers.setdefault(i, self.tool_parser_cls(tok.tokenizer))
                            td = tp.extract_tool_calls_streaming(prev, full[i], content_delta, r)
                            if td:
                                delta.update(td)
                        else:
                            delta["content"] = content_delta
                    fin = None
                    if o.finished or (i < len(o.finish_reasons) and o.finish_reasons[i]):
                        fin = (o.finish_reasons[i] if i < len(o.finish_reasons) else None) or "stop"
                        if use_tools and i in tparsers and tparsers[i]._sent:
                            fin = "tool_calls"
                        finished_idx.add(i)
                    if delta or fin:
                        yield _sse({"id": rid, "object": "chat.completion.chunk", "created": created, "model": model,
                                    "choices": [{"index": i, "delta": delta, "finish_reason": fin}]})
            if r.stream_options and r.stream_options.include_usage:
                yield _sse({"id": rid, "object": "chat.completion.chunk", "created": created, "model": model,
                            "choices": [], "usage": {"prompt_tokens": len(input_tokens),
                                                     "completion_tokens": comp_tokens,
                                                     "total_tokens": len(input_tokens) + comp_tokens}})
            yield b"data: [DONE]\n\n"

        return StreamingResponse(gen(), media_type="text/event-stream")

    # ---- /v1/completions --------------------------------------------------------------------------------------------
    async def completions(self, raw: Request):
        try:
            r = CompletionRequest(**(await raw.json()))
        except Exception as ex:
            return _err(f"invalid request: {ex}")
        tok = self.engine.tokenizer
        p = r.prompt
        if isinstance(p, str):
            prompts = [tok.encode(p)]
        elif p and isinstance(p[0], int):
            prompts = [list(p)]
        elif p and isinstance(p[0], str):
            prompts = [tok.encode(s) for s in p]
        else:
            prompts = [list(x) for x in p]
        if r.stream and len(prompts) > 1:
            return _err("streaming supports a single prompt")
        n_lp = int(r.logprobs or 0)
        rid, created, model = _id("cmpl"), int(time.time()), r.model or self.model_name
        sc = self._sampling_config(r, n_lp)
        if not r.stream:
            choices, ptoks, ctoks = [], 0, 0
            for pi, ids in enumerate(prompts):
                status, out = await self.engine.generate({"input_tokens": ids, "sampling_config": sc}, streamer=False)
                if not status.OK():
                    return _err(status.GetMessage(), 500, "engine_error")
                ptoks += len(ids)
                for i, toks in enumerate(out.output_tokens):
                    ctoks += len(toks)
                    text = tok.decode(toks)
                    if r.echo:
                        text = tok.decode(ids) + text
                    lp = None
                    if n_lp and out.logprobs:
                        ents = out.logprobs[i]
                        lp = {"tokens": [tok.decode([e["token"]]) for e in ents],
                              "token_logprobs": [e["logprob"] for e in ents],
                              "top_logprobs": [{tok.decode([a]): b for a, b in (e["top"] or [])} for e in ents],
                              "text_offset": []}
                    choices.append({"index": len(choices), "text": text, "logprobs": lp,
                                    "finish_reason": (out.finish_reasons[i] if i < len(out.finish_reasons) else None)
                                    or "stop"})
            return JSONResponse({"id": rid, "object": "text_completion", "created": created, "model": model,
                                 "choices": choices, "usage": {"prompt_tokens": ptoks, "completion_tokens": ctoks,
                                                               "total_tokens": ptoks + ctoks}})
        status, out = await self.engine.generate({"input_tokens": prompts[0], "sampling_config": sc}, streamer=True)
        if not status.OK():
            return _err(status.GetMessage(), 500, "engine_error")

        async def gen():
            detoks: Dict[int, IncrementalDetokenizer] = {}
            sent: Dict[int, int] = {}
            done = set()
            async for o in out:
                for i, toks in enumerate(o.output_tokens):
                    if i in done:
                        continue
                    d = detoks.setdefault(i, IncrementalDetokenizer(tok))
                    new = toks[sent.get(i, 0):]
                    sent[i] = len(toks)
                    text = d.push(new) if new else ""
                    fin = None
                    if o.finished or (i < len(o.finish_reasons) and o.finish_reasons[i]):
                        fin = (o.finish_reasons[i] if i < len(o.finish_reasons) else None) or "stop"
                        done.add(i)
                    if text or fin:
                        yield _sse({"id": rid, "object": "text_completion", "created": created, "model": model,
                                    "choices": [{"index": i, "text": text, "logprobs": None, "finish_reason": fin}]})
            yield b"data: [DONE]\n\n"

        return StreamingResponse(gen(), media_type="text/event-stream")

    # ---- /v1/embeddings ------------------------------------------------------------------------------------------------
    async def embeddings(self, raw: Request):
        """Embedding = final-norm hidden state of the last prompt token (one prefill step through /forward's
        ``layernorm`` probe)."""
        import msgpack
        try:
            r = EmbeddingRequest(**(await raw.json()))
        except Exception as ex:
            return _err(f"invalid request: {ex}")
        tok = self.engine.tokenizer
        x = r.input
        if isinstance(x, str):
            items = [tok.encode(x)]
        elif x and isinstance(x[0], int):
            items = [list(x)]
        elif x and isinstance(x[0], str):
            items = [tok.encode(s) for s in x]
        else:
            items = [list(i) for i in x]
        body = {"requests": [{"input_tokens": ids, "request_target": [
            {"target_name": "layernorm", "token_id": [len(ids) - 1], "token_reduce_mode": "GATHER_ALL"}]}
            for ids in items]}
        status, data = await self.engine.forward(msgpack.packb(body, use_bin_type=True), {})
        if not status.OK():
            return _err(status.GetMessage(), 500, "engine_error")
        resp = msgpack.unpackb(data, raw=False)
        out, ntok = [], 0
        for i, rr in enumerate(resp["responses"]):
            t = rr["response"][0]["tensor"]
            raw_bytes = base64.b64decode(t["data"])
            vec = list(struct.unpack(f"<{len(raw_bytes) // 4}f", raw_bytes))
            if r.dimensions:
                vec = vec[: r.dimensions]
            norm = sum(v * v for v in vec) ** 0.5 or 1.0
            vec = [v / norm for v in vec]
            emb: Any = vec
            if r.encoding_format == "base64":
                emb = base64.b64encode(struct.pack(f"<{len(vec)}f", *vec)).decode("ascii")
            out.append({"object": "embedding", "index": i, "embedding": emb})
            ntok += len(rr["input_token_ids"])
        return JSONResponse({"object": "list", "data": out, "model": r.model or self.model_name,
                             "usage": {"prompt_tokens": ntok, "total_tokens": ntok}})

    # ---- /v1/models ------------------------------------------------------------------------------------------------------
    def _card(self) -> ModelCard:
        return ModelCard(id=self.model_name, root=self.args.model_dir or self.model_name,
                         max_model_len=self.engine.serving.setting.batch_scheduler.max_token_len)

    async def models(self):
        return JSONResponse(ModelList(data=[self._card()]).model_dump())

    async def model(self, model_id: str):
        if model_id != self.model_name:
            return _err(f"model {model_id!r} not found", 404, "not_found")
        return JSONResponse(self._card().model_dump())


def add_openai_routes(app, engine, args) -> OpenAIServing:
    s = OpenAIServing(engine, args)
    for prefix in ("/v1", ""):
        app.post(prefix + "/chat/completions")(s.chat)
        app.post(prefix + "/completions")(s.completions)
        app.post(prefix + "/embeddings")(s.embeddings)
        app.get(prefix + "/models")(s.models)
        app.get(prefix + "/models/{model_id}")(s.model)
    return s
