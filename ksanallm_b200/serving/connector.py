"""Prefill / decode disaggregation at the serving level.

A *prefill* instance computes the prompt, returns the first token and pushes the request's KV blocks to a *decode*
instance, which continues the generation; a router (serving/simple_router) sends every request to one instance of
each role with a shared ``kv-comm-request-id`` header. The reference implements this with its Connector /
TaskManager / TaskDispatcher and NCCL / ZMQ / TCP communicators plus a router client with heartbeats
(src/ksana_llm/connector/**, src/ksana_llm/transfer/transfer_engine.h). Here:

* every decode instance runs a transfer listener (TCP); its address is part of the node's registration,
* the prefill instance looks the decode group's listener up (router ``/nodes`` or the static ``peer_transfer_addr``),
  sends ``request id`` + the request's blocks through parallel.transfer.TransferEngine,
* the decode instance's ``/generate`` waits for the import with that id, then admits prompt + first token(s); the
  imported blocks are found again as a cached prefix.
"""
from __future__ import annotations

import json
import socket
import struct
import threading
import time
import urllib.request
from typing import Dict, List, Optional, Tuple

from ..parallel.transfer import TcpTransport, TransferEngine


def _send_str(sock: socket.socket, s: str) -> None:
    b = s.encode()
    sock.sendall(struct.pack("<i", len(b)) + b)


def _connect(host: str, port: int, patience: float = 30.0) -> socket.socket:
    """A peer instance may still be starting: refused connections are retried for a while."""
    deadline = time.time() + patience
    while True:
        try:
            return socket.create_connection((host, port), timeout=30)
        except ConnectionRefusedError:
            if time.time() > deadline:
                raise
            time.sleep(0.2)


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    out = b""
    while len(out) < n:
        c = sock.recv(n - len(out))
        if not c:
            raise ConnectionError("peer closed")
        out += c
    return out


def _recv_str(sock: socket.socket) -> str:
    n = struct.unpack("<i", _recv_exact(sock, 4))[0]
    return _recv_exact(sock, n).decode()


class PDConnector:
    def __init__(self, llm, setting, inference_addr: str = ""):
        """``llm``: engine.LLMEngine; ``setting``: config.schema.ConnectorSetting."""
        self.llm, self.cfg = llm, setting
        self.role = setting.group_role
        self.inference_addr = inference_addr or f"{setting.inference_addr or '127.0.0.1'}:{setting.inference_port}"
        self.transfer_addr: Optional[Tuple[str, int]] = None
        self.node_id: Optional[str] = None
        self._imports: Dict[str, Tuple[List[int], List[int], int]] = {}
        self._cv = threading.Condition()
        self._stop = threading.Event()
        self._threads: List[threading.Thread] = []
        self._srv: Optional[socket.socket] = None
        self.exported = self.imported = 0

    # ---- lifecycle ---------------------------------------------------------------------------------------------------
    def start(self) -> None:
        if self.role in ("decode", "both"):
            host = str(self.cfg.extra.get("transfer_host", "127.0.0.1"))
            self._srv = socket.socket()
            self._srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            self._srv.bind((host, int(self.cfg.extra.get("transfer_port", 0))))
            self._srv.listen(64)
            self._srv.settimeout(0.5)
            self.transfer_addr = (host, self._srv.getsockname()[1])
            t = threading.Thread(target=self._listen, daemon=True)
            t.start()
            self._threads.append(t)
        if self.cfg.router_addr:
            self._register()
            t = threading.Thread(target=self._heartbeat, daemon=True)
            t.start()
            self._threads.append(t)

    def stop(self) -> None:
        self._stop.set()
        if self._srv is not None:
            try:
                self._srv.close()
            except OSError:
                pass

    # ---- router client -----------------------------------------------------------------------------------------------
    def _post(self, path: str, body: dict) -> dict:
        req = urllib.request.Request(f"http://{self.cfg.router_addr}{path}", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=5) as r:
            return json.loads(r.read() or b"{}")

    def _register(self) -> None:
        body = {"group_name": self.cfg.group_name or self.role, "role": self.role, "addr": self.inference_addr,
                "transfer_addr": "%s:%d" % self.transfer_addr if self.transfer_addr else ""}
        try:
            self.node_id = self._post("/RegisterNode", body).get("node_id")
        except OSError:
            self.node_id = None

    def _heartbeat(self) -> None:
        while not self._stop.wait(self.cfg.heartbeat_interval_ms / 1000.0):
            try:
                if self.node_id is None:
                    self._register()
                else:
                    self._post("/Heartbeat", {"node_id": self.node_id})
            except OSError:
                self.node_id = None

    def _decode_transfer_addr(self, group_key: str) -> Tuple[str, int]:
        static = self.cfg.extra.get("peer_transfer_addr")
        if static:
            h, p = str(static).rsplit(":", 1)
            return h, int(p)
        d_group = group_key.split("__", 1)[1] if "__" in group_key else ""
        with urllib.request.urlopen(f"http://{self.cfg.router_addr}/nodes", timeout=5) as r:
            nodes = json.loads(r.read())
        for n in (nodes if isinstance(nodes, list) else nodes.get("nodes", [])):
            if not n.get("online", 1):
                continue
            if n.get("role") in ("decode", "both") and (not d_group or n.get("group_name") == d_group) and \
                    n.get("transfer_addr"):
                h, p = n["transfer_addr"].rsplit(":", 1)
                return h, int(p)
        raise ConnectionError(f"no decode instance with a transfer listener for group key {group_key!r}")

    # ---- prefill side -------------------------------------------------------------------------------------------------
    def export(self, request_id: str, group_key: str, prompt_tokens: List[int], first_tokens: List[int]) -> int:
        host, port = self._decode_transfer_addr(group_key)
        sock = _connect(host, port)
        try:
            _send_str(sock, request_id)
            te = TransferEngine(self.llm.runner.kv_caches, self.llm.cache, TcpTransport(sock), self.llm.block_size)
            pending = []

            def shards(blocks):
                # a tensor-parallel instance: every other rank sends its shard of the same blocks to the decode
                # instance's rank of the same index (listening on port + rank); the message travels in the plan
                # stream, so it reaches the followers before any later step can overwrite those blocks
                pending.append(self.llm.enqueue_control({"op": "pd_export", "rid": request_id, "blocks": list(blocks),
                                                         "host": host, "port": port}))

            with self.llm.lock:
                n = te.export_request(prompt_tokens, first_tokens, 0, on_blocks=shards)
            for ev in pending:
                ev.wait(60.0)
            _recv_exact(sock, 1)  # the decode side acknowledges after committing the blocks
            self.exported += 1
            return n
        finally:
            sock.close()

    # ---- decode side --------------------------------------------------------------------------------------------------
    def _listen(self) -> None:
        while not self._stop.is_set():
            try:
                conn, _ = self._srv.accept()
            except (socket.timeout, OSError):
                continue
            threading.Thread(target=self._serve_import, args=(conn,), daemon=True).start()

    def _serve_import(self, conn: socket.socket) -> None:
        try:
            conn.settimeout(60)
            rid = _recv_str(conn)
            te = TransferEngine(self.llm.runner.kv_caches, self.llm.cache, TcpTransport(conn), self.llm.block_size)
            with self.llm.lock:  # the scheduler thread uses the same cache manager
                toks, first, placed = te.import_request(0)
                have, blocks = te.last_import
                # the other ranks of a tensor-parallel instance place their shard into the same blocks; enqueued
                # under the lock: no step that could read those blocks is planned before the message went out
                ev = self.llm.enqueue_control({"op": "pd_import", "rid": rid, "skip": have, "blocks": list(blocks)})
            ev.wait(60.0)
            conn.sendall(b"\x01")
            with self._cv:
                self._imports[rid] = (toks, first, placed)
                self.imported += 1
                self._cv.notify_all()
        except (OSError, ConnectionError, AssertionError):
            pass
        finally:
            conn.close()

    def wait_import(self, request_id: str, timeout: float) -> Optional[Tuple[List[int], List[int], int]]:
        deadline = time.time() + timeout
        with self._cv:
            while request_id not in self._imports:
                left = deadline - time.time()
                if left <= 0:
                    return None
                self._cv.wait(min(left, 0.5))
            return self._imports.pop(request_id)


class PDShardWorker:
    """Ranks > 0 of a tensor-parallel prefill / decode instance. The driving rank owns the request bookkeeping and
    the block tables; these ranks only move their shard of the KV blocks it names (control messages ``pd_export`` /
    ``pd_import`` arriving in the plan stream). Decode side: a listener on ``transfer_port + rank`` buffers incoming
    shards by request id until the driving rank says where they go."""

    def __init__(self, llm, setting, rank: int):
        self.llm, self.cfg, self.rank = llm, setting, rank
        self.role = setting.group_role
        self._shards: Dict[str, list] = {}
        self._cv = threading.Condition()
        self._stop = threading.Event()
        self._srv: Optional[socket.socket] = None
        self.exported = self.imported = 0
        llm.on_control = self.handle

    def start(self) -> None:
        if self.role in ("decode", "both"):
            host = str(self.cfg.extra.get("transfer_host", "127.0.0.1"))
            base = int(self.cfg.extra.get("transfer_port", 0))
            if base <= 0:
                raise ValueError("a tensor-parallel decode instance needs setting.connector.transfer_port "
                                 "(rank r listens on transfer_port + r)")
            self._srv = socket.socket()
            self._srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            self._srv.bind((host, base + self.rank))
            self._srv.listen(64)
            self._srv.settimeout(0.5)
            threading.Thread(target=self._listen, daemon=True).start()

    def stop(self) -> None:
        self._stop.set()
        if self._srv is not None:
            try:
                self._srv.close()
            except OSError:
                pass

    def _engine(self, sock) -> TransferEngine:
        return TransferEngine(self.llm.runner.kv_caches, None, TcpTransport(sock) if sock is not None else None,
                              self.llm.block_size)

    def _listen(self) -> None:
        while not self._stop.is_set():
            try:
                conn, _ = self._srv.accept()
            except (socket.timeout, OSError):
                continue
            try:
                conn.settimeout(60)
                rid = _recv_str(conn)
                bufs = self._engine(conn).import_shard()
                with self._cv:
                    self._shards[rid] = bufs
                    self._cv.notify_all()
            except (OSError, ConnectionError, AssertionError):
                pass
            finally:
                conn.close()

    def handle(self, msg: Dict) -> None:
        """Runs inside the follower's step loop, in plan order."""
        if msg.get("op") == "pd_export":
            sock = _connect(msg["host"], int(msg["port"]) + self.rank)
            try:
                _send_str(sock, msg["rid"])
                self._engine(sock).export_shard(msg["blocks"])
                self.exported += 1
            finally:
                sock.close()
        elif msg.get("op") == "pd_import":
            deadline = time.time() + 60.0
            with self._cv:
                while msg["rid"] not in self._shards and time.time() < deadline:
                    self._cv.wait(0.5)
                bufs = self._shards.pop(msg["rid"], None)
            if bufs is None:
                raise RuntimeError(f"KV shard of request {msg['rid']} did not arrive on rank {self.rank}")
            self._engine(None).place_shard(bufs, int(msg["skip"]), msg["blocks"])
            self.imported += 1
