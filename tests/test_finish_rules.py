"""How requests end, through the serving-level engine on CPU: EOS, stop token ids, stop strings (text match across
token boundaries), length limit, abort of a streaming request when its iterator is dropped (client disconnect),
input longer than max_token_len, invalid sampling parameters."""
import asyncio
import os

import pytest

from ksanallm_b200.serving.ksana_engine import EngineArgs, KsanaLLMEngine

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def eng():
    os.environ["KSANA_SKIP_WARMUP"] = "1"
    args = EngineArgs.from_config_file(os.path.join(ROOT, "examples", "tiny_cpu.yaml"), synthetic_model="tiny-llama",
                                       device="cpu")
    e = KsanaLLMEngine(args)
    e.initialize()
    yield e
    e.shutdown()


def _gen(eng, **sc):
    body = {"input_tokens": [5, 9, 77, 120, 33], "stream": False, "sampling_config": dict({"topk": 1}, **sc)}
    return asyncio.run(eng.generate(body, streamer=False))


def test_length_eos_and_stop_tokens(eng):
    st, free = _gen(eng, max_new_tokens=12, ignore_eos=True)
    toks = free.output_tokens[0]
    assert st.OK() and len(toks) == 12 and free.finish_reasons == ["length"]
    # a stop token id ends the request AT that token (it is part of the output, as in the reference)
    st, out = _gen(eng, max_new_tokens=12, ignore_eos=True, stop_token_ids=[toks[4]])
    assert out.output_tokens[0] == toks[:toks.index(toks[4]) + 1] and out.finish_reasons == ["stop"]
    # the model's EOS id behaves the same unless ignore_eos is set
    eos = eng.model_config.eos_token_ids
    eng.model_config.eos_token_ids = [toks[2]]
    try:
        st, out = _gen(eng, max_new_tokens=12)
        assert out.output_tokens[0] == toks[:toks.index(toks[2]) + 1] and out.finish_reasons == ["stop"]
        st, out = _gen(eng, max_new_tokens=12, ignore_eos=True)
        assert out.output_tokens[0] == toks
    finally:
        eng.model_config.eos_token_ids = eos


def test_stop_strings_match_decoded_text(eng, monkeypatch):
    # the stand-in tokenizer only knows byte tokens; give every id a letter so that the random model "writes" text
    monkeypatch.setattr(eng.tokenizer, "decode", lambda ids, **kw: "".join(chr(97 + int(t) % 26) for t in ids))
    st, free = _gen(eng, max_new_tokens=12, ignore_eos=True)
    text = eng.tokenizer.decode(free.output_tokens[0])
    needle = text[3:5]  # spans two tokens
    st, out = _gen(eng, max_new_tokens=12, ignore_eos=True, stop_strings=[needle])
    got = eng.tokenizer.decode(out.output_tokens[0])
    assert st.OK() and out.finish_reasons == ["stop"]
    assert got.endswith(needle) and len(out.output_tokens[0]) == text.index(needle) + 2


def test_invalid_requests_are_rejected(eng):
    st, out = _gen(eng, max_new_tokens=4, topk=5000)
    assert not st.OK() and out is None
    body = {"input_tokens": list(range(3, 400)), "stream": False, "sampling_config": {"max_new_tokens": 4}}
    st, out = asyncio.run(eng.generate(body, streamer=False))
    assert not st.OK() and "max_token_len" in st.GetMessage()
    st, out = asyncio.run(eng.generate({"stream": False}, streamer=False))
    assert not st.OK()


def test_dropping_the_stream_aborts_the_request(eng):
    async def run():
        body = {"input_tokens": [5, 9, 77, 120, 33], "stream": True,
                "sampling_config": {"topk": 1, "max_new_tokens": 200, "ignore_eos": True}}
        st, it = await eng.generate(body, streamer=True)
        assert st.OK()
        first = await it.__anext__()
        req = it.req
        del it  # the client went away
        for _ in range(200):
            if req.finished:
                break
            await asyncio.sleep(0.02)
        return first, req

    first, req = asyncio.run(run())
    assert req.finished and len(req.seqs[0].output_tokens) < 200
    assert req.seqs[0].finish_reason == "abort"
    assert not eng.llm.has_unfinished()


def test_many_concurrent_requests_complete_and_match_sequential_runs(eng):
    """More requests in flight than the event loop's default executor has threads: each parks a waiter thread in the
    engine's own pool; all finish, and batching changes no token."""
    import time
    bodies = [{"input_tokens": [5 + (i % 7), 9, 77 + i, 120, 33], "stream": False,
               "sampling_config": {"topk": 1, "max_new_tokens": 6, "ignore_eos": True}} for i in range(72)]
    seq = [asyncio.run(eng.generate(dict(b), streamer=False))[1].output_tokens[0] for b in bodies[:6]]

    async def burst():
        return await asyncio.gather(*[eng.generate(dict(b), streamer=False) for b in bodies])

    t0 = time.time()
    res = asyncio.run(burst())
    assert all(st.OK() for st, _ in res) and time.time() - t0 < 60
    assert [o.output_tokens[0] for _, o in res[:6]] == seq
