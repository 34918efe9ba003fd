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
import os
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
        # layer-by-layer hand-over (prefill side): request id -> session; see expect_export
        self._sessions: Dict[int, "_LayerwiseExport"] = {}
        self._by_rid: Dict[str, "_LayerwiseExport"] = {}
        self._tracker = None
        self.layerwise_exports = 0
        self.layerwise = os.environ.get("KSANA_PD_LAYERWISE", "1") != "0"

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
    def expect_export(self, req, request_id: str, group_key: str) -> None:
        """Announces that ``req`` will be handed over: the connection to the decode instance is opened now (off the
        step thread), and when the scheduler plans the prompt's last chunk the KV blocks leave layer by layer while
        the forward pass is still running (``LayerProgressTracker`` events), instead of all at once after the first
        token. Used on single-rank instances, with synchronous or asynchronous stepping (through the native executor
        the layers report together at the end of the stack, so the transfer then overlaps the sampling and the next
        step's scheduling only); tensor-parallel instances keep the one-piece export, their shards travel after the
        step. Reference: the prefill side's layer-wise sends in
        src/ksana_llm/transfer/transfer_engine.h:63-190."""
        if not self.layerwise or self.llm.tp.size > 1:
            return
        sess = _LayerwiseExport(self, req, request_id, group_key)
        self._by_rid[request_id] = sess
        for s_ in req.seqs:
            self._sessions[s_.seq_id] = sess
        self.llm.before_forward = self._on_plan
        self.llm.before_resolve = self._before_resolve
        threading.Thread(target=sess.connect, daemon=True).start()

    def _on_plan(self, plan) -> None:
        """Engine hook, step thread, right before the forward pass of ``plan``."""
        model = self.llm.runner.model
        armed = []
        for e in plan.entries:
            sess = self._sessions.get(e.seq_id)
            if sess is not None and e.num_logits > 0 and not sess.armed:
                if sess.arm(e.seq_id):
                    armed.append(sess)
                else:
                    self._drop(sess)
        if not armed:
            if model.progress is not None and not any(s_.armed and not s_.layers_done.is_set()
                                                      for s_ in self._by_rid.values()):
                model.progress = None
            return
        from ..parallel.transfer import LayerProgressTracker
        if self._tracker is None:
            self._tracker = LayerProgressTracker(len(self.llm.runner.kv_caches), self.llm.runner.device)
        self._tracker.reset()
        self._tracker.set_callbacks([s_.on_layer for s_ in armed])
        model.progress = self._tracker

    def cancel_export(self, request_id: str) -> None:
        """The request ended without a hand-over (error, abort): close its session, if any."""
        sess = self._by_rid.get(request_id)
        if sess is not None:
            self._drop(sess)

    def _before_resolve(self, plan) -> None:
        """Engine hook: the step's results are about to reach the scheduler, which may finish the request and return
        its blocks to the pool. The layers of a session armed for this step are read from those blocks by the
        tracker's thread: wait until the last one has been copied out (the device finished this forward pass before
        its tokens could be read, so this is the copy time of the last layers at most)."""
        for e in plan.entries:
            sess = self._sessions.get(e.seq_id)
            if sess is not None and sess.armed and not sess.failed:
                sess.layers_done.wait(30.0)

    def _drop(self, sess) -> None:
        self._by_rid.pop(sess.request_id, None)
        for k in [k for k, v in self._sessions.items() if v is sess]:
            self._sessions.pop(k, None)
        sess.close()

    def export(self, request_id: str, group_key: str, prompt_tokens: List[int], first_tokens: List[int]) -> int:
        sess = self._by_rid.get(request_id)
        if sess is not None:
            try:
                if sess.armed and sess.finish(first_tokens):
                    self.exported += 1
                    self.layerwise_exports += 1
                    return sess.n_blocks
            finally:
                self._drop(sess)
            # the session never started (connection not ready in time, request pre-empted, ...): one-piece export
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
            evs = []

            def committed(have, blocks):
                # the other ranks of a tensor-parallel instance place their shard into the same blocks; enqueued
                # under the lock that covers the commit: no step that could read those blocks is planned before
                # the message went out
                evs.append(self.llm.enqueue_control({"op": "pd_import", "rid": rid, "skip": have,
                                                     "blocks": list(blocks)}))

            # the engine's lock (the scheduler thread uses the same cache manager) is taken for the reservation and
            # for the commit only: a layer-by-layer export keeps this connection busy for a whole forward pass
            toks, first, placed = te.import_request(0, lock=self.llm.lock, after_commit=committed)
            if not evs:
                with self.llm.lock:
                    committed(*te.last_import)
            evs[0].wait(60.0)
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


class _LayerwiseExport:
    """One request leaving the prefill instance layer by layer."""

    def __init__(self, conn: PDConnector, req, request_id: str, group_key: str):
        self.c, self.req, self.request_id, self.group_key = conn, req, request_id, group_key
        self.sock: Optional[socket.socket] = None
        self.ready = threading.Event()
        self.layers_done = threading.Event()
        self.armed = False
        self.failed = False
        self.te: Optional[TransferEngine] = None
        self.n_blocks = 0

    def connect(self) -> None:
        try:
            host, port = self.c._decode_transfer_addr(self.group_key)
            self.sock = _connect(host, port)
            _send_str(self.sock, self.request_id)
        except (OSError, ConnectionError):
            self.failed = True
        self.ready.set()

    def arm(self, seq_id: int) -> bool:
        """Step thread, the prompt's last chunk is about to run: header + tokens go out now, the layers follow from
        the tracker's callbacks. False: not possible (no connection yet), the caller falls back."""
        # the connection is opened when the request arrives; a short wait here (step thread) is cheaper than losing
        # the overlap when the very first step already runs the prompt's last chunk
        self.ready.wait(float(os.environ.get("KSANA_PD_LAYERWISE_WAIT_MS", "20")) / 1000.0)
        if not self.ready.is_set() or self.failed or self.sock is None:
            return False
        llm = self.c.llm
        toks = list(self.req.prompt_tokens)
        n_full = len(toks) // llm.block_size
        with llm.lock:
            blocks = list(llm.cache.block_table(seq_id))[:n_full]
        self.n_blocks = len(blocks)
        try:
            self.te = TransferEngine(llm.runner.kv_caches, llm.cache, TcpTransport(self.sock), llm.block_size)
            self.te.begin_export(toks, blocks, 0)
        except (OSError, ConnectionError):
            self.failed = True
            return False
        self.armed = True
        return True

    def on_layer(self, layer: int) -> None:
        if self.failed:
            return
        try:
            self.te.send_layer(layer, 0)
        except (OSError, ConnectionError):
            self.failed = True
            self.layers_done.set()  # nobody needs to wait for the rest
        if layer == len(self.te.kv) - 1:
            self.layers_done.set()

    def finish(self, first_tokens: List[int]) -> bool:
        if not self.layers_done.wait(60.0) or self.failed:
            return False
        try:
            self.te.finish_export(first_tokens, 0)
            _recv_exact(self.sock, 1)  # the decode side acknowledges after committing the blocks
            return True
        except (OSError, ConnectionError):
            return False

    def close(self) -> None:
        if self.sock is not None:
            try:
                self.sock.close()
            except OSError:
                pass


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
        # layer-by-layer hand-over (prefill side): request id -> session; see expect_export
        self._sessions: Dict[int, "_LayerwiseExport"] = {}
        self._by_rid: Dict[str, "_LayerwiseExport"] = {}
        self._tracker = None
        self.layerwise_exports = 0
        self.layerwise = os.environ.get("KSANA_PD_LAYERWISE", "1") != "0"
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
