"""Inter-node control plane over TCP: node registration, barrier, layer-range allocation, KV block-count
synchronisation (min over nodes), heartbeat with timeout, shutdown broadcast.

Capability parity with the reference's ControlChannel / DistributedCoordinator
(src/ksana_llm/distributed/control_channel.cpp:70-118, 215-252, 433-494, 577-792; packet types in packet_type.h):
the master listens on MASTER_HOST:MASTER_PORT, workers connect and exchange length-prefixed JSON packets. On a
missed heartbeat the failing peer is reported through ``on_failure`` (the reference shuts the whole cluster down;
here the engine fails in-flight requests and keeps the decision to the caller). Every blocking wait has a timeout.
"""
from __future__ import annotations

import json
import socket
import struct
import threading
import time
from typing import Any, Callable, Dict, List, Optional, Tuple

HEARTBEAT_INTERVAL_S = 30.0
HEARTBEAT_TIMEOUT_S = 120.0


def _send(sock: socket.socket, obj: Dict[str, Any]) -> None:
    data = json.dumps(obj).encode()
    sock.sendall(struct.pack("<I", len(data)) + data)


def _recv(sock: socket.socket) -> Optional[Dict[str, Any]]:
    hdr = b""
    while len(hdr) < 4:
        chunk = sock.recv(4 - len(hdr))
        if not chunk:
            return None
        hdr += chunk
    (n,) = struct.unpack("<I", hdr)
    buf = b""
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            return None
        buf += chunk
    return json.loads(buf)


def split_layers(num_layers: int, world: int, master_offload: int = 0) -> List[Tuple[int, int]]:
    """Contiguous [lo, hi) layer ranges per node; ``master_offload`` layers are moved off node 0 (it also runs the
    embedding, lm_head and sampling; reference env MASTER_OFFLOAD_LAYER_NUM)."""
    base, rem = divmod(num_layers, world)
    counts = [base + (1 if i < rem else 0) for i in range(world)]
    if world > 1 and master_offload > 0:
        take = min(master_offload, counts[0] - 1)
        counts[0] -= take
        for i in range(take):
            counts[1 + i % (world - 1)] += 1
    out, lo = [], 0
    for c in counts:
        out.append((lo, lo + c))
        lo += c
    return out


class ControlMaster:
    def __init__(self, host: str, port: int, world_size: int, heartbeat_interval: float = HEARTBEAT_INTERVAL_S,
                 heartbeat_timeout: float = HEARTBEAT_TIMEOUT_S, on_failure: Optional[Callable[[int], None]] = None):
        self.world = world_size
        self.hb_interval, self.hb_timeout = heartbeat_interval, heartbeat_timeout
        self.on_failure = on_failure
        self.srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self.srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self.srv.bind((host, port))
        self.srv.listen(world_size)
        self.port = self.srv.getsockname()[1]
        self.conns: Dict[int, socket.socket] = {}
        self.last_seen: Dict[int, float] = {}
        self.lock = threading.Lock()
        self.cond = threading.Condition(self.lock)
        self.barriers: Dict[str, set] = {}
        self.values: Dict[str, Dict[int, Any]] = {}
        self.failed: List[int] = []
        self._stop = threading.Event()
        self._threads: List[threading.Thread] = []
        t = threading.Thread(target=self._accept_loop, daemon=True)
        t.start()
        self._threads.append(t)
        t = threading.Thread(target=self._watchdog, daemon=True)
        t.start()
        self._threads.append(t)

    def _accept_loop(self) -> None:
        self.srv.settimeout(0.2)
        while not self._stop.is_set():
            try:
                conn, _ = self.srv.accept()
            except socket.timeout:
                continue
            except OSError:
                return
            msg = _recv(conn)
            if not msg or msg.get("type") != "add_node":
                conn.close()
                continue
            rank = int(msg["rank"])
            with self.cond:
                self.conns[rank] = conn
                self.last_seen[rank] = time.time()
                self.cond.notify_all()
            t = threading.Thread(target=self._serve, args=(rank, conn), daemon=True)
            t.start()
            self._threads.append(t)

    def _serve(self, rank: int, conn: socket.socket) -> None:
        while not self._stop.is_set():
            try:
                msg = _recv(conn)
            except OSError:
                msg = None
            if msg is None:
                return
            with self.cond:
                self.last_seen[rank] = time.time()
                typ = msg.get("type")
                if typ == "barrier":
                    self.barriers.setdefault(msg["name"], set()).add(rank)
                elif typ == "value":
                    self.values.setdefault(msg["name"], {})[rank] = msg["value"]
                self.cond.notify_all()

    def _watchdog(self) -> None:
        while not self._stop.wait(min(self.hb_interval, 0.5)):
            now = time.time()
            with self.cond:
                for r, t in list(self.last_seen.items()):
                    if r not in self.failed and now - t > self.hb_timeout:
                        self.failed.append(r)
                        if self.on_failure:
                            self.on_failure(r)
                        self.cond.notify_all()

    def wait_nodes(self, timeout: float = 60.0) -> bool:
        with self.cond:
            return self.cond.wait_for(lambda: len(self.conns) >= self.world - 1, timeout)

    def broadcast(self, obj: Dict[str, Any]) -> None:
        with self.lock:
            for r, c in self.conns.items():
                if r in self.failed:
                    continue
                try:
                    _send(c, obj)
                except OSError:
                    pass

    def barrier(self, name: str, timeout: float = 60.0) -> bool:
        """Master side of a barrier: waits for every worker, then releases them."""
        with self.cond:
            ok = self.cond.wait_for(lambda: len(self.barriers.get(name, ())) >= self.world - 1 or self.failed, timeout)
            ok = ok and not self.failed
            self.barriers.pop(name, None)
        self.broadcast({"type": "barrier_release", "name": name, "ok": ok})
        return ok

    def allocate_layers(self, num_layers: int, master_offload: int = 0, nccl_id: Optional[str] = None):
        ranges = split_layers(num_layers, self.world, master_offload)
        self.broadcast({"type": "layers", "ranges": ranges, "nccl_id": nccl_id})
        return ranges

    def sync_min(self, name: str, my_value: int, timeout: float = 60.0) -> Optional[int]:
        """All nodes report a number (e.g. KV block count); everybody receives the minimum."""
        with self.cond:
            ok = self.cond.wait_for(lambda: len(self.values.get(name, {})) >= self.world - 1 or self.failed, timeout)
            if not ok or self.failed:
                return None
            vals = list(self.values.pop(name).values()) + [my_value]
        m = min(vals)
        self.broadcast({"type": "value_result", "name": name, "value": m})
        return m

    def shutdown(self) -> None:
        self.broadcast({"type": "shutdown"})
        self._stop.set()
        with self.lock:
            for c in self.conns.values():
                try:
                    c.close()
                except OSError:
                    pass
        self.srv.close()


class ControlWorker:
    def __init__(self, host: str, port: int, rank: int, heartbeat_interval: float = HEARTBEAT_INTERVAL_S,
                 heartbeat_timeout: float = HEARTBEAT_TIMEOUT_S, on_shutdown: Optional[Callable[[], None]] = None,
                 connect_timeout: float = 30.0):
        self.rank = rank
        self.hb_interval, self.hb_timeout = heartbeat_interval, heartbeat_timeout
        self.on_shutdown = on_shutdown
        deadline = time.time() + connect_timeout
        while True:
            try:
                self.sock = socket.create_connection((host, port), timeout=2.0)
                break
            except OSError:
                if time.time() > deadline:
                    raise
                time.sleep(0.05)
        self.sock.settimeout(None)
        _send(self.sock, {"type": "add_node", "rank": rank})
        self.inbox: List[Dict[str, Any]] = []
        self.cond = threading.Condition()
        self.last_master = time.time()
        self.master_lost = False
        self._stop = threading.Event()
        self.paused = False  # test hook: stop sending heartbeats
        threading.Thread(target=self._reader, daemon=True).start()
        threading.Thread(target=self._heartbeat, daemon=True).start()

    def _reader(self) -> None:
        while not self._stop.is_set():
            try:
                msg = _recv(self.sock)
            except OSError:
                msg = None
            if msg is None:
                with self.cond:
                    self.master_lost = True
                    self.cond.notify_all()
                return
            with self.cond:
                self.last_master = time.time()
                if msg.get("type") == "shutdown":
                    self._stop.set()
                    if self.on_shutdown:
                        self.on_shutdown()
                self.inbox.append(msg)
                self.cond.notify_all()

    def _heartbeat(self) -> None:
        while not self._stop.wait(self.hb_interval):
            if self.paused:
                continue
            try:
                _send(self.sock, {"type": "heartbeat", "rank": self.rank, "t": time.time()})
            except OSError:
                return

    def _wait_msg(self, pred, timeout: float) -> Optional[Dict[str, Any]]:
        with self.cond:
            def find():
                for i, m in enumerate(self.inbox):
                    if pred(m):
                        return self.inbox.pop(i)
                return None
            end = time.time() + timeout
            while True:
                m = find()
                if m is not None or self.master_lost:
                    return m
                left = end - time.time()
                if left <= 0:
                    return None
                self.cond.wait(left)

    def barrier(self, name: str, timeout: float = 60.0) -> bool:
        _send(self.sock, {"type": "barrier", "name": name, "rank": self.rank})
        m = self._wait_msg(lambda x: x.get("type") == "barrier_release" and x.get("name") == name, timeout)
        return bool(m and m.get("ok"))

    def wait_layers(self, timeout: float = 60.0):
        m = self._wait_msg(lambda x: x.get("type") == "layers", timeout)
        return (m["ranges"][self.rank], m.get("nccl_id")) if m else None

    def sync_min(self, name: str, value: int, timeout: float = 60.0) -> Optional[int]:
        _send(self.sock, {"type": "value", "name": name, "value": value, "rank": self.rank})
        m = self._wait_msg(lambda x: x.get("type") == "value_result" and x.get("name") == name, timeout)
        return None if m is None else int(m["value"])

    def wait_shutdown(self, timeout: float) -> bool:
        return self._wait_msg(lambda x: x.get("type") == "shutdown", timeout) is not None

    def close(self) -> None:
        self._stop.set()
        try:
            self.sock.close()
        except OSError:
            pass
