"""Prefill/decode disaggregation through the serving layer: two engine instances (roles prefill and decode); the
request goes to both with one ``kv-comm-request-id``. The decode instance must answer with exactly what a single
instance generates, after receiving the prompt's KV blocks and the first token from the prefill instance. One case
wires the two statically, the other finds the decode listener through the router's node registry."""
import asyncio
import os
import socket
import threading
import time

import pytest

from ksanallm_b200.serving.ksana_engine import EngineArgs, KsanaLLMEngine

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BODY = {"input_tokens": [(7 * i + 3) % 200 + 3 for i in range(40)], "stream": False,
        "sampling_config": {"max_new_tokens": 6, "topk": 1, "ignore_eos": True}}


def _make(role, router="", group="", enable_async=None, **extra):
    args = EngineArgs.from_config_file(os.path.join(ROOT, "examples", "tiny_cpu.yaml"), synthetic_model="tiny-llama",
                                       device="cpu")
    if enable_async is not None:
        args.serving.setting.batch_scheduler.enable_async = enable_async
    cs = args.serving.setting.connector
    cs.group_role, cs.router_addr, cs.group_name, cs.connector_waiting_sec = role, router, group, 30
    cs.heartbeat_interval_ms = 200
    cs.extra.update(extra)
    eng = KsanaLLMEngine(args)
    eng.initialize()
    return eng


def _run_pair(prefill, decode, ctx, body):
    async def both():
        d = asyncio.create_task(decode.generate(dict(body), streamer=False, req_ctx=ctx))
        p = asyncio.create_task(prefill.generate(dict(body), streamer=False, req_ctx=ctx))
        return await asyncio.gather(p, d)
    return asyncio.run(both())


@pytest.fixture(scope="module")
def want():
    single = _make("none")
    st, out = asyncio.run(single.generate(dict(BODY), streamer=False))
    assert st.OK()
    single.shutdown()
    return out


def test_static_peer(want):
    decode = _make("decode")
    prefill = _make("prefill", peer_transfer_addr="%s:%d" % decode.connector.transfer_addr)
    try:
        (pst, pout), (dst, dout) = _run_pair(prefill, decode, {"kv-comm-request-id": "r1"}, BODY)
        assert pst.OK() and dst.OK()
        assert pout.output_tokens == [want.output_tokens[0][:1]]
        assert dout.output_tokens == want.output_tokens and dout.input_tokens == want.input_tokens
        assert prefill.connector.exported == 1 and decode.connector.imported == 1
        assert decode.llm.cache.stats.prefix_hit_tokens >= 32  # two full blocks arrived instead of being computed
        # a request without the header is served locally by either instance
        st, out = asyncio.run(decode.generate(dict(BODY), streamer=False))
        assert st.OK() and out.output_tokens == want.output_tokens
    finally:
        decode.shutdown()
        prefill.shutdown()


def test_streaming_requests_and_first_token_stop(want):
    """The router forwards the client's body unchanged, so both instances may see stream=true: the prefill instance
    still completes and exports, the decode instance streams. A first token that is a stop token ends the request on
    the decode side without another step."""
    decode = _make("decode")
    prefill = _make("prefill", peer_transfer_addr="%s:%d" % decode.connector.transfer_addr)
    try:
        async def both(body, ctx):
            d = asyncio.create_task(decode.generate(dict(body), streamer=True, req_ctx=ctx))
            p = asyncio.create_task(prefill.generate(dict(body), streamer=True, req_ctx=ctx))
            (pst, pit), (dst, dit) = await asyncio.gather(p, d)
            assert pst.OK() and dst.OK()
            last = None
            async for item in dit:
                last = item
            return [x async for x in pit], last

        p_items, last = asyncio.run(both(BODY, {"kv-comm-request-id": "s1"}))
        assert len(p_items) == 1 and last.finished and last.output_tokens == want.output_tokens
        stop_body = dict(BODY, sampling_config=dict(BODY["sampling_config"], ignore_eos=False,
                                                    stop_token_ids=[want.output_tokens[0][0]]))
        steps = decode.llm.stats["steps"]
        _, last = asyncio.run(both(stop_body, {"kv-comm-request-id": "s2"}))
        assert last.finished and last.output_tokens == [want.output_tokens[0][:1]] and last.finish_reasons == ["stop"]
        assert decode.llm.stats["steps"] == steps
    finally:
        decode.shutdown()
        prefill.shutdown()


def test_decode_times_out_without_prefill():
    decode = _make("decode")
    decode.serving.setting.connector.connector_waiting_sec = 1
    try:
        st, out = asyncio.run(decode.generate(dict(BODY), streamer=False, req_ctx={"kv-comm-request-id": "nobody"}))
        assert not st.OK() and out is None and "KV transfer" in st.GetMessage()
    finally:
        decode.shutdown()


def test_lookup_through_router(want):
    import uvicorn
    from ksanallm_b200.serving.simple_router import create_app, NodeRegistry
    reg = NodeRegistry()
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    server = uvicorn.Server(uvicorn.Config(create_app(reg), host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    for _ in range(100):
        if server.started:
            break
        time.sleep(0.05)
    decode = _make("decode", router=f"127.0.0.1:{port}", group="dg")
    prefill = _make("prefill", router=f"127.0.0.1:{port}", group="pg")
    try:
        nodes = {n["role"]: n for n in reg.nodes()}
        assert set(nodes) == {"prefill", "decode"}
        assert nodes["decode"]["transfer_addr"] == "%s:%d" % decode.connector.transfer_addr
        hb0 = nodes["decode"]["last_heartbeat"]
        time.sleep(0.5)
        assert {n["role"]: n for n in reg.nodes()}["decode"]["last_heartbeat"] > hb0
        ctx = {"kv-comm-request-id": "r2", "kv-comm-group-key": "pg__dg"}
        (pst, _), (dst, dout) = _run_pair(prefill, decode, ctx, BODY)
        assert pst.OK() and dst.OK() and dout.output_tokens == want.output_tokens
    finally:
        decode.shutdown()
        prefill.shutdown()
        server.should_exit = True
        th.join(timeout=5)


@pytest.mark.parametrize("enable_async", [False, True])
def test_kv_leaves_layer_by_layer_during_the_last_prefill_chunk(want, monkeypatch, enable_async):
    """The prefill instance ships each layer's blocks from the layer tracker's callbacks while its forward pass runs
    (chunked prefill: the blocks of earlier chunks go with the first layers of the last chunk), the first token
    follows as a trailer; with synchronous and with asynchronous stepping."""
    monkeypatch.setenv("KSANA_PD_LAYERWISE_WAIT_MS", "5000")
    decode = _make("decode")
    prefill = _make("prefill", enable_async=enable_async, peer_transfer_addr="%s:%d" % decode.connector.transfer_addr)
    order = []
    try:
        assert prefill.llm.async_mode == enable_async
        from ksanallm_b200.parallel import transfer
        real = transfer.TransferEngine.send_layer

        def spy(self, layer, peer):
            order.append(("layer", layer, prefill.llm.step_count))
            return real(self, layer, peer)
        monkeypatch.setattr(transfer.TransferEngine, "send_layer", spy)
        real_fin = transfer.TransferEngine.finish_export
        monkeypatch.setattr(transfer.TransferEngine, "finish_export",
                            lambda self, first, peer: (order.append(("trailer", list(first))), real_fin(self, first, peer))[1])
        (pst, pout), (dst, dout) = _run_pair(prefill, decode, {"kv-comm-request-id": "lw1"}, BODY)
        assert pst.OK() and dst.OK()
        assert dout.output_tokens == want.output_tokens and dout.input_tokens == want.input_tokens
        assert prefill.connector.layerwise_exports == 1 and decode.connector.imported == 1
        n_layers = len(prefill.llm.runner.kv_caches)
        assert [o[:2] for o in order[:n_layers]] == [("layer", l) for l in range(n_layers)]
        assert len({o[2] for o in order[:n_layers]}) == 1        # all within one step of the prefill instance
        assert order[n_layers] == ("trailer", want.output_tokens[0][:1])
        assert decode.llm.cache.stats.prefix_hit_tokens >= 32
        assert prefill.llm.runner.model.progress is None or not prefill.connector._sessions
    finally:
        decode.shutdown()
        prefill.shutdown()
