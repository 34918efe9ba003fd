"""The Triton Inference Server python backend, run against a stand-in for ``triton_python_backend_utils``: TensorRT-LLM
style input tensors become an engine request, answers leave through the response sender (one per step when
streaming, FINAL flag last), a ``forward`` request carries a msgpack body, and a bad request yields an error answer
instead of taking the backend down."""
import base64
import importlib.util
import json
import os
import shutil
import sys
import threading
import types

import msgpack
import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WRAP = os.path.join(ROOT, "ksanallm_b200", "serving", "wrappers", "triton", "ksana_llm")


class _Tensor:
    def __init__(self, name, array):
        self._name, self._a = name, array

    def name(self):
        return self._name

    def as_numpy(self):
        return self._a


class _Response:
    def __init__(self, output_tensors=None, error=None):
        self.tensors = {t.name(): t.as_numpy() for t in (output_tensors or [])}
        self.error = error


class _Error:
    def __init__(self, message):
        self.message = message


class _Sender:
    def __init__(self):
        self.responses, self.final = [], threading.Event()

    def send(self, response=None, flags=0):
        if response is not None:
            self.responses.append(response)
        if flags == 1:
            self.final.set()


class _Request:
    def __init__(self, **tensors):
        self._inputs = [_Tensor(k, v) for k, v in tensors.items()]
        self.sender = _Sender()

    def inputs(self):
        return self._inputs

    def get_response_sender(self):
        return self.sender


@pytest.fixture(scope="module")
def backend(tmp_path_factory):
    fake = types.ModuleType("triton_python_backend_utils")
    fake.Tensor, fake.InferenceResponse, fake.TritonError = _Tensor, _Response, _Error
    fake.TritonModelException = RuntimeError
    fake.TRITONSERVER_RESPONSE_COMPLETE_FINAL = 1
    fake.Logger = types.SimpleNamespace(log_info=lambda m: None, log_error=lambda m: None)
    fake.using_decoupled_model_transaction_policy = \
        lambda cfg: bool(cfg.get("model_transaction_policy", {}).get("decoupled"))
    fake.triton_string_to_numpy = lambda s: {"TYPE_STRING": np.object_, "TYPE_INT32": np.int32, "TYPE_UINT32": np.uint32,
                                             "TYPE_FP32": np.float32}[s]
    sys.modules["triton_python_backend_utils"] = fake
    repo = tmp_path_factory.mktemp("repo")
    os.makedirs(repo / "1")
    shutil.copy(os.path.join(ROOT, "examples", "tiny_cpu.yaml"), repo / "1" / "ksana_llm.yaml")
    spec = importlib.util.spec_from_file_location("ksana_triton_model", os.path.join(WRAP, "1", "model.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    os.environ["KSANA_TRITON_ENGINE_OVERRIDES"] = json.dumps({"synthetic_model": "tiny-llama", "device": "cpu"})
    os.environ["KSANA_SKIP_WARMUP"] = "1"
    cfg = {"model_transaction_policy": {"decoupled": True},
           "output": [{"name": n, "data_type": t} for n, t in (
               ("forward_response", "TYPE_STRING"), ("text_output", "TYPE_STRING"), ("output_ids", "TYPE_INT32"),
               ("completion_tokens", "TYPE_UINT32"), ("sequence_length", "TYPE_UINT32"),
               ("cum_log_probs", "TYPE_FP32"), ("finish_reason", "TYPE_INT32"))]}
    model = mod.TritonPythonModel()
    model.initialize({"model_config": json.dumps(cfg), "model_repository": str(repo), "model_version": "1"})
    yield mod, model
    model.finalize()
    del sys.modules["triton_python_backend_utils"]
    os.environ.pop("KSANA_TRITON_ENGINE_OVERRIDES", None)


def _run(model, req):
    assert model.execute([req]) is None
    assert req.sender.final.wait(60)
    return req.sender.responses


def test_config_declares_the_tensors_the_backend_reads():
    text = open(os.path.join(WRAP, "config.pbtxt")).read()
    assert 'backend: "python"' in text and "decoupled: True" in text
    mod_src = open(os.path.join(WRAP, "1", "model.py")).read()
    import re
    for name in re.findall(r'name: "(\w+)"', text)[1:]:
        assert f'"{name}"' in mod_src, name


def test_generate_streaming_and_not(backend):
    _, model = backend
    common = dict(input_ids=np.array([[5, 9, 77, 120]], dtype=np.uint32),
                  request_output_len=np.array([6], dtype=np.uint32), runtime_top_k=np.array([1], dtype=np.uint32),
                  sampling_parameters=np.array([[json.dumps({"ignore_eos": True}).encode()]], dtype=np.object_),
                  return_log_probs=np.array([True]))
    whole = _run(model, _Request(streaming=np.array([False]), **common))
    assert len(whole) == 1 and whole[0].error is None
    ids = whole[0].tensors["output_ids"]
    assert ids.shape == (1, 6) and whole[0].tensors["sequence_length"].tolist() == [6]
    assert whole[0].tensors["finish_reason"].tolist() == [0] and np.isfinite(whole[0].tensors["cum_log_probs"]).all()
    assert isinstance(whole[0].tensors["text_output"].reshape(-1)[0], bytes)
    parts = _run(model, _Request(streaming=np.array([True]), **common))
    assert len(parts) >= 2 and parts[-1].tensors["output_ids"].tolist() == ids.tolist()
    text = _run(model, _Request(text_input=np.array([[b"hello"]], dtype=np.object_),
                                request_output_len=np.array([3], dtype=np.uint32)))
    assert text[0].error is None and text[0].tensors["completion_tokens"].tolist()[0] <= 3


def test_forward_request_and_error_answer(backend):
    _, model = backend
    body = msgpack.packb({"requests": [{"input_tokens": [1, 2, 3, 4], "request_target": [
        {"target_name": "layernorm", "slice_pos": [[-1, -1]], "token_reduce_mode": "GATHER_ALL"}]}]})
    out = _run(model, _Request(request_type=np.array([b"forward"], dtype=np.object_),
                               request_bytes=np.array([body], dtype=np.object_)))
    assert out[0].error is None
    t = msgpack.unpackb(out[0].tensors["forward_response"].reshape(-1)[0], raw=False)["responses"][0]["response"][0]
    a = np.frombuffer(base64.b64decode(t["tensor"]["data"]), dtype=np.float32)
    assert t["target_name"] == "layernorm" and a.size == int(np.prod(t["tensor"]["shape"]))
    bad = _run(model, _Request(request_output_len=np.array([3], dtype=np.uint32)))  # neither text nor tokens
    assert bad[0].error is not None and bad[0].error.message
