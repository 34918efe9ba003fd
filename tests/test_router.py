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
