"""PD router registry: registration, heartbeat expiry (host-side fault: a node that stops beating), pair choice by
load, first-writer-wins communication ids."""
import time

from fastapi.testclient import TestClient

from ksanallm_b200.serving.simple_router import NodeRegistry, create_app


def test_registry_and_http_surface():
    reg = NodeRegistry(heartbeat_timeout=0.3)
    c = TestClient(create_app(reg))
    p = c.post("/RegisterNode", json={"group_name": "pg", "role": "prefill", "addr": "127.0.0.1:1"}).json()["node_id"]
    d1 = c.post("/RegisterNode", json={"group_name": "dg1", "role": "decode", "addr": "127.0.0.1:2"}).json()["node_id"]
    d2 = c.post("/RegisterNode", json={"group_name": "dg2", "role": "decode", "addr": "127.0.0.1:3"}).json()["node_id"]
    assert c.post("/RegisterNode", json={"group_name": "x", "role": "nope", "addr": "a"}).status_code == 400
    reg.add_inflight(d1, 3)
    pair = reg.pick_pair()
    assert pair[0][0] == p and pair[1][0] == d2  # least loaded decode node
    a = c.post("/RegisterCommId", json={"group_key": "pg__dg2", "comm_id": "AAA"}).json()["comm_id"]
    b = c.post("/RegisterCommId", json={"group_key": "pg__dg2", "comm_id": "BBB"}).json()["comm_id"]
    assert a == b == "AAA"
    time.sleep(0.4)
    assert c.post("/Heartbeat", json={"node_id": p}).status_code == 200
    assert c.post("/Heartbeat", json={"node_id": "ghost"}).status_code == 404
    nodes = {n["node_id"]: n for n in c.get("/nodes").json()}
    assert nodes[p]["online"] == 1 and nodes[d1]["online"] == 0 and nodes[d2]["online"] == 0
    assert c.post("/generate", json={"prompt": "x"}).status_code == 503  # no decode node alive any more


def test_static_provider_round_robin_and_penalty():
    from ksanallm_b200.serving.simple_router.name_service import StaticProvider
    sp = StaticProvider([("p0:1", "d0:1"), ("p1:1", "d1:1")], penalty=2)
    first = [sp.get_available_nodes()[0]["addr"] for _ in range(4)]
    assert first == ["p0:1", "p1:1", "p0:1", "p1:1"]
    bad = sp.pairs[0]
    sp.update_call_result(bad[0], bad[1], False, True)
    assert [sp.get_available_nodes()[0]["addr"] for _ in range(3)] == ["p1:1", "p1:1", "p0:1"]


def _free_port():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _serve(app, port):
    import threading
    import uvicorn
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    for _ in range(200):
        if server.started:
            break
        time.sleep(0.05)
    return server, th


def test_generate_through_the_router_with_two_live_instances():
    """Router + a prefill instance + a decode instance, all over real HTTP on loopback: the client's /generate goes
    to the router, which fans it out; the decode instance's answer (streamed back) equals a single instance's."""
    import json
    import os
    import httpx
    from ksanallm_b200.serving.ksana_engine import EngineArgs
    from ksanallm_b200.serving.server import LLMServer
    os.environ["KSANA_SKIP_WARMUP"] = "1"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    rport = _free_port()
    reg = NodeRegistry()
    router, rth = _serve(create_app(reg), rport)
    servers = []
    try:
        for role in ("decode", "prefill", "none"):
            port = _free_port()
            args = EngineArgs.from_config_file(os.path.join(root, "examples", "tiny_cpu.yaml"),
                                               synthetic_model="tiny-llama", device="cpu")
            cs = args.serving.setting.connector
            if role != "none":
                cs.group_role, cs.router_addr, cs.group_name = role, f"127.0.0.1:{rport}", role + "_group"
                cs.inference_addr, cs.inference_port, cs.heartbeat_interval_ms = "127.0.0.1", port, 200
                cs.connector_waiting_sec = 30
            srv = LLMServer(args)
            srv.initialize()
            servers.append((srv, port) + _serve(srv.app, port))
        assert {n["role"] for n in reg.nodes()} == {"prefill", "decode"}
        body = {"input_tokens": [(7 * i + 3) % 200 + 3 for i in range(40)], "stream": False,
                "sampling_config": {"max_new_tokens": 6, "topk": 1, "ignore_eos": True}}
        want = httpx.post(f"http://127.0.0.1:{servers[2][1]}/generate", content=json.dumps(body), timeout=60).json()
        got = httpx.post(f"http://127.0.0.1:{rport}/generate", content=json.dumps(body), timeout=60)
        assert got.status_code == 200
        got = json.loads(got.content.split(b"\0")[0])
        assert got["output_token_ids"] == want["output_token_ids"] and len(got["output_token_ids"][0]) == 6
        assert servers[1][0].model.connector.exported == 1 and servers[0][0].model.connector.imported == 1
    finally:
        for srv, _, us, th in servers:
            us.should_exit = True
            srv.model.shutdown()
        router.should_exit = True
