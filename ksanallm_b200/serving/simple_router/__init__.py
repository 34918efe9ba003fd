"""PD-disaggregation router: registry of prefill / decode nodes, heartbeats, communication-id registration and
request fan-out to a (prefill, decode) pair with merged streaming.

Capability parity with the reference's ``simple_router`` FastAPI service
(src/ksana_llm/python/simple_router/{main,services,node,generate,models,database}.py): nodes register themselves
with ``POST /RegisterNode`` and keep alive with ``POST /Heartbeat``; ``POST /RegisterCommId`` stores the NCCL/ZMQ
communication id of a prefill-decode group pair; ``POST /generate`` picks the least-loaded alive pair, tags both
sub-requests with ``kv-comm-group-key`` / ``kv-comm-request-id`` headers and streams the decode node's output.
Storage is sqlite3 from the standard library (the reference uses SQLAlchemy).
"""
from __future__ import annotations

import asyncio
import json
import sqlite3
import threading
import time
import uuid
from typing import Any, Dict, List, Optional, Tuple

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, StreamingResponse

HEARTBEAT_TIMEOUT_S = 30.0


class NodeRegistry:
    def __init__(self, path: str = ":memory:", heartbeat_timeout: float = HEARTBEAT_TIMEOUT_S):
        self.transfer_addrs: Dict[str, str] = {}
        self.db = sqlite3.connect(path, check_same_thread=False)
        self.lock = threading.Lock()
        self.timeout = heartbeat_timeout
        with self.lock:
            self.db.execute("CREATE TABLE IF NOT EXISTS nodes (node_id TEXT PRIMARY KEY, group_name TEXT, role TEXT, "
                            "addr TEXT, world_size INTEGER, last_heartbeat REAL, inflight INTEGER DEFAULT 0, "
                            "online INTEGER DEFAULT 1)")
            self.db.execute("CREATE TABLE IF NOT EXISTS comm_ids (group_key TEXT PRIMARY KEY, comm_id TEXT, created REAL)")
            self.db.commit()

    def register(self, group_name: str, role: str, addr: str, world_size: int = 1, node_id: Optional[str] = None,
                 transfer_addr: str = "") -> str:
        if role not in ("prefill", "decode", "both"):
            raise ValueError("role must be prefill, decode or both")
        node_id = node_id or uuid.uuid4().hex
        self.transfer_addrs[node_id] = transfer_addr  # where a decode node accepts KV transfers
        with self.lock:
            self.db.execute("INSERT OR REPLACE INTO nodes VALUES (?, ?, ?, ?, ?, ?, 0, 1)",
                            (node_id, group_name, role, addr, world_size, time.time()))
            self.db.commit()
        return node_id

    def heartbeat(self, node_id: str) -> bool:
        with self.lock:
            cur = self.db.execute("UPDATE nodes SET last_heartbeat = ?, online = 1 WHERE node_id = ?",
                                  (time.time(), node_id))
            self.db.commit()
            return cur.rowcount > 0

    def sweep(self) -> List[str]:
        """Marks nodes without a recent heartbeat offline; returns their ids."""
        dead_before = time.time() - self.timeout
        with self.lock:
            rows = self.db.execute("SELECT node_id FROM nodes WHERE online = 1 AND last_heartbeat < ?",
                                   (dead_before,)).fetchall()
            self.db.execute("UPDATE nodes SET online = 0 WHERE last_heartbeat < ?", (dead_before,))
            self.db.commit()
        return [r[0] for r in rows]

    def alive(self, role: str) -> List[Tuple[str, str, str, int]]:
        self.sweep()
        with self.lock:
            return self.db.execute("SELECT node_id, group_name, addr, inflight FROM nodes WHERE online = 1 AND "
                                   "(role = ? OR role = 'both') ORDER BY inflight ASC", (role,)).fetchall()

    def pick_pair(self) -> Optional[Tuple[Tuple, Tuple]]:
        p, d = self.alive("prefill"), self.alive("decode")
        if not p or not d:
            return None
        return p[0], d[0]

    def add_inflight(self, node_id: str, delta: int) -> None:
        with self.lock:
            self.db.execute("UPDATE nodes SET inflight = MAX(inflight + ?, 0) WHERE node_id = ?", (delta, node_id))
            self.db.commit()

    def register_comm_id(self, group_key: str, comm_id: str) -> str:
        """First writer wins: both sides of a pair call this and end up with the same id."""
        with self.lock:
            row = self.db.execute("SELECT comm_id FROM comm_ids WHERE group_key = ?", (group_key,)).fetchone()
            if row:
                return row[0]
            self.db.execute("INSERT INTO comm_ids VALUES (?, ?, ?)", (group_key, comm_id, time.time()))
            self.db.commit()
            return comm_id

    def nodes(self) -> List[Dict[str, Any]]:
        with self.lock:
            rows = self.db.execute("SELECT node_id, group_name, role, addr, world_size, last_heartbeat, inflight, "
                                   "online FROM nodes").fetchall()
        keys = ["node_id", "group_name", "role", "addr", "world_size", "last_heartbeat", "inflight", "online"]
        out = [dict(zip(keys, r)) for r in rows]
        for n in out:
            n["transfer_addr"] = self.transfer_addrs.get(n["node_id"], "")
        return out


def create_app(registry: Optional[NodeRegistry] = None, http_client_factory=None, provider=None) -> FastAPI:
    """``provider``: a name_service.NameServiceProvider choosing the prefill / decode pair of every request; the
    default reads this router's own registry."""
    from .name_service import RegistryProvider
    reg = registry or NodeRegistry()
    app = FastAPI()
    app.state.registry = reg
    ns = provider or RegistryProvider(reg)
    app.state.provider = ns

    def client():
        if http_client_factory is not None:
            return http_client_factory()
        import httpx
        return httpx.AsyncClient(timeout=None)

    @app.post("/RegisterNode")
    async def register_node(req: Request):
        b = await req.json()
        try:
            nid = reg.register(b["group_name"], b["role"], b["addr"], int(b.get("world_size", 1)), b.get("node_id"),
                               str(b.get("transfer_addr", "") or ""))
        except (KeyError, ValueError) as ex:
            raise HTTPException(400, str(ex))
        return {"node_id": nid, "heartbeat_timeout_s": reg.timeout}

    @app.post("/Heartbeat")
    async def heartbeat(req: Request):
        b = await req.json()
        if not reg.heartbeat(b.get("node_id", "")):
            raise HTTPException(404, "unknown node")
        return {"status": "ok", "time": time.time()}

    @app.post("/RegisterCommId")
    async def register_comm(req: Request):
        b = await req.json()
        return {"comm_id": reg.register_comm_id(b["group_key"], b["comm_id"])}

    @app.get("/nodes")
    async def nodes():
        reg.sweep()
        return reg.nodes()

    @app.get("/health")
    async def health():
        return {"status": "healthy"}

    @app.post("/generate")
    async def generate(req: Request):
        pair = ns.get_available_nodes()
        if pair is None:
            raise HTTPException(503, "no alive prefill/decode pair")
        pn, dn = pair
        p_id, p_group, p_addr = pn["node_id"], pn["group_name"], pn["addr"]
        d_id, d_group, d_addr = dn["node_id"], dn["group_name"], dn["addr"]
        body = await req.body()
        headers = {"kv-comm-group-key": f"{p_group}__{d_group}", "kv-comm-request-id": uuid.uuid4().hex,
                   "Content-Type": "application/json"}
        reg.add_inflight(p_id, 1)
        reg.add_inflight(d_id, 1)
        c = client()

        async def run():
            p_ok = d_ok = False
            try:
                # the prefill node computes the prompt and pushes KV to the decode node; its own reply is dropped
                prefill_task = asyncio.create_task(c.post(f"http://{p_addr}/generate", content=body, headers=headers))
                async with c.stream("POST", f"http://{d_addr}/generate", content=body, headers=headers) as r:
                    d_ok = r.status_code == 200
                    async for chunk in r.aiter_bytes():
                        yield chunk
                p_ok = (await prefill_task).status_code == 200
            finally:
                reg.add_inflight(p_id, -1)
                reg.add_inflight(d_id, -1)
                ns.update_call_result(pn, dn, p_ok, d_ok)
                await c.aclose()

        return StreamingResponse(run())

    return app


def main(argv=None) -> None:
    import argparse
    import uvicorn
    ap = argparse.ArgumentParser(description="ksanallm_b200 PD router")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=9080)
    ap.add_argument("--db", default="router.sqlite3")
    ap.add_argument("--name-service", default="", help="module exposing create_provider() (default: own registry)")
    ap.add_argument("--static-pairs", default="", help="prefill_addr=decode_addr[,prefill_addr=decode_addr...]")
    ns = ap.parse_args(argv)
    provider = None
    if ns.name_service:
        from .name_service import load_provider
        provider = load_provider(ns.name_service)
    elif ns.static_pairs:
        from .name_service import StaticProvider
        provider = StaticProvider([tuple(x.split("=", 1)) for x in ns.static_pairs.split(",")])
    uvicorn.run(create_app(NodeRegistry(ns.db), provider=provider), host=ns.host, port=ns.port)


if __name__ == "__main__":
    main()
