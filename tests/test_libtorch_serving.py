"""The blocking ``Serving`` surface (names of the reference's extension module) over the engine, on CPU."""
import json
import threading

import pytest

from ksanallm_b200.config.schema import parse_serving_config
from ksanallm_b200.serving import libtorch_serving as lts


@pytest.fixture(scope="module")
def serving():
    cfg = parse_serving_config({"setting": {"global": {}, "batch_scheduler": {
        "max_batch_size": 8, "max_step_tokens": 128, "max_token_len": 256},
        "block_manager": {"block_token_num": 16}}})
    s = lts.Serving()
    s.init_serving("", synthetic_model="tiny-llama", device="cpu", serving=cfg)
    yield s
    s.shutdown()


def _input(n=24, new=6):
    inp = lts.KsanaPythonInput()
    inp.input_tokens = [(5 * i + 7) % 200 + 3 for i in range(n)]
    inp.sampling_config.max_new_tokens = new
    inp.sampling_config.ignore_eos = True
    return inp


def test_generate_blocks_and_returns_status_and_output(serving):
    status, out = serving.generate(_input(), {})
    assert status.OK() and out.input_tokens == _input().input_tokens
    assert len(out.output_tokens) == 1 and len(out.output_tokens[0]) == 6


def test_streaming_iterator_yields_growing_outputs_then_stop_iteration(serving):
    want = serving.generate(_input(), {})[1].output_tokens[0]
    status, it = serving.generate_streaming(_input(), {})
    assert status.OK()
    seen = []
    while True:
        st, out = it.GetNext()
        if st.GetCode() == lts.RetCode.RET_STOP_ITERATION:
            assert out is None
            break
        assert st.OK()
        seen.append(list(out.output_tokens[0]))
    assert seen and seen[-1] == want
    assert all(a == b[:len(a)] for a, b in zip(seen, seen[1:]))  # every item carries the full output so far


def test_calls_from_many_threads(serving):
    res = [None] * 4

    def run(i):
        res[i] = serving.generate(_input(20 + i, 4), {})
    ts = [threading.Thread(target=run, args=(i,)) for i in range(4)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(60)
    assert all(r is not None and r[0].OK() and len(r[1].output_tokens[0]) == 4 for r in res)


def test_forward_and_invalid_argument(serving):
    body = {"requests": [{"input_tokens": _input().input_tokens,
                          "request_target": [{"target_name": "logits", "slice_pos": [[23, 23]],
                                              "token_reduce_mode": "GATHER_ALL"}]}]}
    status, data = serving.forward(json.dumps(body).encode(), {"Content-Type": "application/json"})
    assert status.OK(), status.GetMessage()
    resp = json.loads(data)["responses"][0]
    assert resp["input_token_ids"] == _input().input_tokens and resp["response"]
    bad = lts.KsanaPythonInput()
    bad.input_tokens = []
    st, _ = serving.generate(bad, {})
    assert not st.OK()
