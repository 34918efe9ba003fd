"""HTTP front end: ``/generate``, ``/forward``, ``/health`` plus the OpenAI-compatible routes.

Wire contract kept from the reference server (src/ksana_llm/python/serving_server.py:37-276):
``POST /generate`` takes a JSON body, ``stream`` defaults to true and streams ``json + b"\\0"`` chunks each carrying
the FULL output so far (``texts``, ``output_token_ids``, ``logprobs``, ``input_token_ids``); errors are HTTP 500
with ``{message, code}``; ``POST /forward`` takes/returns msgpack (JSON when the Content-Type says so);
``GET /health`` -> ``{"status": "healthy"}``. Request headers ``x-remote-ip``, ``kv-comm-group-key``,
``kv-comm-request-id`` and ``Content-Type`` are forwarded to the engine as the request context.
"""
from __future__ import annotations

import json
import os
import signal
import sys
from typing import Any, Dict, Optional

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, Response, StreamingResponse

from .ksana_engine import EngineArgs, KsanaLLMEngine

FIELDS_TO_EXTRACT = ("x-remote-ip", "kv-comm-group-key", "kv-comm-request-id", "Content-Type")

try:  # orjson is optional; the stdlib encoder produces the same bytes for these payloads
    import orjson

    def _dumps(obj) -> bytes:
        return orjson.dumps(obj)

    def _loads(b):
        return orjson.loads(b)
except Exception:  # pragma: no cover
    def _dumps(obj) -> bytes:
        return json.dumps(obj, ensure_ascii=False, separators=(",", ":")).encode("utf-8")

    def _loads(b):
        return json.loads(b)


class LLMServer:
    def __init__(self, args: EngineArgs, engine: Optional[KsanaLLMEngine] = None):
        self.args = args
        self.app = FastAPI(root_path=args.root_path or "")
        self.model = engine or KsanaLLMEngine.from_engine_args(args)
        self._setup_routes()

    def initialize(self) -> None:
        if self.model.llm is None:
            self.model.initialize()
        self._setup_reasoning()
        from .openai.adapter import add_openai_routes
        from ..utils.metrics import Metrics, add_metrics_route
        metrics = Metrics.from_serving_config(self.model.serving)
        self.model.llm.metrics = metrics
        add_metrics_route(self.app, metrics, self.model.llm)
        add_openai_routes(self.app, self.model, self.args)

    def _setup_reasoning(self) -> None:
        """A reasoning parser supplies the token id that ends the thinking section, so that grammar constraints
        are switched on only after it."""
        name = self.args.reasoning_parser
        if not name:
            return
        from .reasoning import get_reasoning_parser
        parser = get_reasoning_parser(name)(self.model.tokenizer.tokenizer)
        self.model.think_end_token_id = getattr(parser, "think_end_token_id", None)

    def _setup_routes(self) -> None:
        self.app.post("/generate")(self.generate)
        self.app.post("/forward")(self.forward)
        self.app.get("/health")(self.health_check)

    @staticmethod
    def get_trace_context(request: Request) -> Dict[str, str]:
        return {f: request.headers.get(f) for f in FIELDS_TO_EXTRACT if request.headers.get(f) is not None}

    def _texts(self, out, streaming: bool):
        texts = []
        for toks in out.output_tokens:
            try:
                texts.append(self.model.tokenizer.decode(toks))
            except Exception as ex:
                raise ValueError("Invalid token ids!") from ex
        return texts

    def _payload(self, out, streaming: bool) -> Dict[str, Any]:
        return {"texts": self._texts(out, streaming), "output_token_ids": out.output_tokens, "logprobs": out.logprobs,
                "input_token_ids": out.input_tokens}

    async def generate(self, request: Request) -> Response:
        try:
            req_ctx = self.get_trace_context(request)
            request_dict = _loads(await request.body())
            enable_streaming = request_dict.get("stream", True)
            status, output = await self.model.generate(request_dict=request_dict, streamer=enable_streaming,
                                                       req_ctx=req_ctx)
            if not status.OK():
                raise HTTPException(status_code=500, detail={"message": status.GetMessage(),
                                                             "code": status.GetCode().value})
            if enable_streaming:
                async def stream_results():
                    async for o in output:
                        if o is None:
                            return
                        yield _dumps(self._payload(o, True)) + b"\0"
                return StreamingResponse(stream_results())
            return JSONResponse(self._payload(output, False))
        except HTTPException:
            raise
        except Exception as ex:
            raise HTTPException(status_code=500, detail=str(ex))

    async def forward(self, request: Request) -> Response:
        try:
            req_ctx = self.get_trace_context(request)
            status, data = await self.model.forward(await request.body(), req_ctx)
            if not status.OK() or data is None:
                raise HTTPException(status_code=500, detail={"message": status.GetMessage(),
                                                             "code": status.GetCode().value})
            is_json = "json" in (req_ctx.get("Content-Type", "") or "").lower()
            return Response(content=data, media_type="application/json" if is_json else "application/x-msgpack")
        except HTTPException:
            raise
        except Exception as ex:
            raise HTTPException(status_code=500, detail=str(ex))

    async def health_check(self) -> Dict[str, str]:
        return {"status": "healthy"}


def main(argv=None) -> None:
    """``python serving_server.py --config_file X.yaml --port N ...``. With WORLD_SIZE > 1 (one process per GPU,
    e.g. under torchrun) only rank 0 opens the port; the other ranks run the follower loop."""
    import uvicorn
    args = EngineArgs.from_command_line(argv)
    server = LLMServer(args)
    rank = int(os.environ.get("RANK", os.environ.get("NODE_RANK", "0")))
    from ..utils.logger import StateReporter, setup_logging
    log = setup_logging(rank=rank)
    log.info("starting: config %s, model %s", args.config_file, args.model_dir or args.synthetic_model)
    server.model.initialize()
    if rank == 0:
        StateReporter(server.model.llm).start()
    def _leave():
        import gc
        import torch.distributed as dist
        server.model.llm = None  # the engine's references to the process groups go first ...
        gc.collect()
        if dist.is_initialized():
            dist.destroy_process_group()  # ... then the backend's threads are joined before the interpreter exits

    if rank != 0:
        server.model.serve_follower()
        _leave()
        return
    server.initialize()

    def _term(signum, frame):
        server.model.shutdown()
        _leave()
        sys.exit(0)

    signal.signal(signal.SIGTERM, _term)
    uvicorn.run(server.app, host=args.host, port=args.port, log_level="info" if args.access_log else "warning",
                access_log=args.access_log, ssl_keyfile=args.ssl_keyfile, ssl_certfile=args.ssl_certfile)
    server.model.shutdown()
    _leave()


if __name__ == "__main__":
    main()
