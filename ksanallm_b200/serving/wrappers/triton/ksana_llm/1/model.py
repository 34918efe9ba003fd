"""Triton Inference Server python backend over the serving engine.

Model repository layout: ``<repo>/ksana_llm/config.pbtxt``, ``<repo>/ksana_llm/1/model.py`` (this file) and
``<repo>/ksana_llm/1/ksana_llm.yaml`` (the usual serving configuration). Tensor names follow the TensorRT-LLM
convention the reference's backend uses (src/ksana_llm/endpoints/wrapper/triton/config/ksana_llm/1/model.py,
config.pbtxt): ``text_input`` / ``input_ids`` / ``messages``, ``request_output_len``, ``runtime_top_k``,
``runtime_top_p``, ``temperature``, ``random_seed``, ``beam_width``, ``len_penalty`` ..., ``streaming``; a request with
``request_type == "forward"`` carries a msgpack /forward body in ``request_bytes``.

The engine batches by itself, so ``execute`` only hands every request to an asyncio loop running in a thread and
returns; answers go out through the request's response sender (decoupled transaction policy), one per step when
``streaming`` is set, else one at the end, always closed by the FINAL flag.
"""
import asyncio
import json
import os
import threading

import numpy as np

import triton_python_backend_utils as pb_utils  # provided by the Triton python backend at run time

CONFIG_FILENAME = "ksana_llm.yaml"

# triton input name -> key of the engine's request dict / sampling_config
TOP_LEVEL = {"text_input": "prompt", "input_ids": "input_tokens", "messages": "messages",
             "input_refit_embedding": "input_refit_embedding", "streaming": "stream"}
SAMPLING = {"request_output_len": "max_new_tokens", "num_return_sequences": "num_return_sequences",
            "presence_penalty": "presence_penalty", "repetition_penalty": "repetition_penalty",
            "temperature": "temperature", "runtime_top_k": "topk", "runtime_top_p": "topp", "random_seed": "seed",
            "len_penalty": "length_penalty", "beam_width": "num_beams", "min_length": "min_tokens",
            "stop_token_ids": "stop_token_ids"}
JSON_INPUTS = ("sampling_parameters", "messages", "input_refit_embedding")


def _scalar(a: np.ndarray):
    v = a.reshape(-1)[0]
    if isinstance(v, (bytes, bytearray)):
        return v.decode("utf-8")
    return v.item() if hasattr(v, "item") else v


def parse_request(request) -> dict:
    """Triton tensors -> {"request_type", "request_bytes"} or the engine's /generate request dict."""
    out, sampling = {}, {}
    for t in request.inputs():
        name, a = t.name(), t.as_numpy()
        if a is None or a.size == 0:
            continue
        if name in JSON_INPUTS:
            raw = a.reshape(-1)[0]
            val = json.loads(raw.decode("utf-8") if isinstance(raw, (bytes, bytearray)) else raw)
            if name == "sampling_parameters":
                sampling.update(val)
            else:
                out[TOP_LEVEL[name]] = val
        elif name == "request_bytes":
            raw = a.reshape(-1)[0]
            out["request_bytes"] = bytes(raw) if isinstance(raw, (bytes, bytearray)) else str(raw).encode("latin-1")
        elif name == "request_type":
            out["request_type"] = _scalar(a)
        elif name == "return_log_probs":
            if bool(_scalar(a)):
                sampling["logprobs"] = 1
        elif name in ("input_ids", "stop_token_ids"):
            ids = [int(x) for x in a.reshape(-1).tolist()]
            if name == "input_ids":
                out["input_tokens"] = ids
            else:
                sampling["stop_token_ids"] = ids
        elif name in TOP_LEVEL:
            out[TOP_LEVEL[name]] = _scalar(a)
        elif name in SAMPLING:
            sampling[SAMPLING[name]] = _scalar(a)
    out["sampling_config"] = sampling
    return out


class TritonPythonModel:
    def initialize(self, args):
        self.logger = pb_utils.Logger
        model_config = json.loads(args["model_config"])
        if not pb_utils.using_decoupled_model_transaction_policy(model_config):
            raise pb_utils.TritonModelException("ksana_llm needs model_transaction_policy { decoupled: True }")
        self.output_dtypes = {o["name"]: pb_utils.triton_string_to_numpy(o["data_type"]) for o in model_config["output"]}
        model_dir = os.path.join(args["model_repository"], args["model_version"])
        yaml_path = os.path.join(model_dir, CONFIG_FILENAME)
        if not os.path.isfile(yaml_path):
            raise pb_utils.TritonModelException(f"'{CONFIG_FILENAME}' must be provided in '{model_dir}'")
        from ksanallm_b200.serving.ksana_engine import EngineArgs, KsanaLLMEngine
        overrides = json.loads(os.environ.get("KSANA_TRITON_ENGINE_OVERRIDES", "{}"))  # e.g. a synthetic model
        self.engine = KsanaLLMEngine.from_engine_args(EngineArgs.from_config_file(yaml_path, **overrides))
        self.engine.initialize()
        self.loop = asyncio.new_event_loop()
        self.in_flight = 0
        self.lock = threading.Lock()
        self.thread = threading.Thread(target=self.loop.run_forever, name="ksana-triton-loop", daemon=True)
        self.thread.start()
        self.logger.log_info("ksana_llm engine started")

    # ---- answers ------------------------------------------------------------------------------------------
    def _generate_response(self, out, length_penalty: float):
        tok = self.engine.tokenizer
        lens = [len(t) for t in out.output_tokens] or [0]
        width = max(lens)
        pad = self.engine.model_config.eos_token_ids[0] if self.engine.model_config.eos_token_ids else 0
        ids = [list(t) + [pad] * (width - len(t)) for t in out.output_tokens] or [[]]
        texts = [tok.decode(list(t)).rstrip("�").encode("utf-8") for t in out.output_tokens] or [b""]
        cum = []
        for n, lp in zip(lens, out.logprobs or []):  # length-normalised sum of the chosen tokens' log-probs
            total = sum(float(e["logprob"]) for e in (lp or []) if e)
            cum.append(total / (max(n, 1) ** length_penalty))
        if not cum:
            cum = [float("nan")] * len(lens)
        dt = self.output_dtypes
        return pb_utils.InferenceResponse(output_tensors=[
            pb_utils.Tensor("text_output", np.asarray(texts, dtype=dt.get("text_output", np.object_))),
            pb_utils.Tensor("output_ids", np.asarray(ids, dtype=dt.get("output_ids", np.int32))),
            pb_utils.Tensor("completion_tokens", np.asarray(lens, dtype=dt.get("completion_tokens", np.uint32))),
            pb_utils.Tensor("sequence_length", np.asarray(lens, dtype=dt.get("sequence_length", np.uint32))),
            pb_utils.Tensor("cum_log_probs", np.asarray(cum, dtype=dt.get("cum_log_probs", np.float32))),
            pb_utils.Tensor("finish_reason", np.asarray([int(out.finish_status.GetCode())],
                                                        dtype=dt.get("finish_reason", np.int32)))])

    @staticmethod
    def _error(message: str):
        return pb_utils.InferenceResponse(error=pb_utils.TritonError(message))

    async def _serve(self, request) -> None:
        sender = request.get_response_sender()
        try:
            rd = parse_request(request)
            if rd.get("request_type") == "forward":
                status, data = await self.engine.forward(rd.get("request_bytes") or b"")
                if not status.OK():
                    sender.send(self._error(status.GetMessage()))
                else:
                    sender.send(pb_utils.InferenceResponse(output_tensors=[pb_utils.Tensor(
                        "forward_response", np.asarray([data], dtype=self.output_dtypes.get("forward_response",
                                                                                            np.object_)))]))
                return
            stream = bool(rd.pop("stream", False))
            lp = float(rd["sampling_config"].get("length_penalty", 1.0))
            status, res = await self.engine.generate(rd, streamer=stream)
            if not status.OK() or res is None:
                sender.send(self._error(status.GetMessage() or "request failed"))
            elif stream:
                async for out in res:
                    sender.send(self._generate_response(out, lp))
            else:
                sender.send(self._generate_response(res, lp))
        except Exception as ex:  # one bad request must not take the backend down
            sender.send(self._error(f"{type(ex).__name__}: {ex}"))
        finally:
            sender.send(flags=pb_utils.TRITONSERVER_RESPONSE_COMPLETE_FINAL)
            with self.lock:
                self.in_flight -= 1

    def execute(self, requests):
        for request in requests:
            with self.lock:
                self.in_flight += 1
            asyncio.run_coroutine_threadsafe(self._serve(request), self.loop)
        return None  # decoupled: every answer goes through the response senders

    def finalize(self):
        import time
        deadline = time.time() + 30
        while self.in_flight and time.time() < deadline:
            time.sleep(0.05)
        self.loop.call_soon_threadsafe(self.loop.stop)
        self.thread.join(timeout=10)
        self.engine.shutdown()
