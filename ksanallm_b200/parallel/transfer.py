"""Prefill / decode disaggregation: moving a request's KV blocks (and its first token) from the prefill instance to
the decode instance, layer by layer as the layers finish.

Reference: TransferEngine (src/ksana_llm/transfer/transfer_engine.h:63-190) is driven by LayerProgressTracker
(runtime/layer_progress_tracker.{h,cpp}: one CUDA event per layer, a monitor thread, a callback that pushes the
layer's blocks) over the connector's NCCL / ZMQ / TCP communicators (connector/communicator/**); the first token and
draft tokens follow the blocks (runtime/llm_runtime.cpp:253-279).

Both sides go through the prefix tree of their KV cache manager: the exporter pins the request's full blocks by
matching its tokens, the importer allocates blocks for the same tokens, receives into them and commits them, after
which the ordinary admission path finds them as a cached prefix and only recomputes the unfinished tail block.
"""
from __future__ import annotations

import socket
import struct
import threading
import time
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist


class LayerProgressTracker:
    """Per-layer completion events. ``record(layer)`` is called right after a layer's kernels were launched; a
    monitor thread fires the callbacks in layer order once the device has actually finished them (CUDA events), or
    immediately on CPU. Recording layer L implies every layer below it was launched before."""

    def __init__(self, num_layers: int, device: torch.device):
        self.num_layers, self.device = num_layers, torch.device(device)
        self._callbacks: List[Callable[[int], None]] = []
        self._events: Dict[int, "torch.cuda.Event"] = {}
        self._lock = threading.Condition()
        self._next = 0          # next layer whose completion has not been reported
        self._recorded = -1     # highest layer recorded in this pass
        self._stop = False
        self._thread: Optional[threading.Thread] = None

    def register_callback(self, fn: Callable[[int], None]) -> None:
        self._callbacks.append(fn)

    def set_callbacks(self, fns: Sequence[Callable[[int], None]]) -> None:
        """Replaces the callbacks (one forward pass = one set: the blocks to ship differ from step to step)."""
        with self._lock:
            self._callbacks = list(fns)

    def reset(self) -> None:
        with self._lock:
            self._events.clear()
            self._next, self._recorded = 0, -1

    def record(self, layer: int) -> None:
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            with self._lock:
                self._events[layer] = ev
                self._recorded = max(self._recorded, layer)
                self._lock.notify_all()
            if self._thread is None:
                self._thread = threading.Thread(target=self._monitor, daemon=True)
                self._thread.start()
        else:
            with self._lock:
                self._recorded = max(self._recorded, layer)
            self._drain(layer)

    def _drain(self, upto: int) -> None:
        while self._next <= upto:
            for fn in self._callbacks:
                fn(self._next)
            self._next += 1

    def _monitor(self) -> None:
        while True:
            with self._lock:
                self._lock.wait_for(lambda: self._stop or any(l >= self._next for l in self._events), timeout=0.5)
                if self._stop:
                    return
                ready = sorted(l for l in self._events if l >= self._next)
            for layer in ready:
                self._events[layer].synchronize()
                self._drain(layer)

    def wait_all(self, timeout: float = 30.0) -> bool:
        t0 = time.time()
        while self._next <= self._recorded:
            if time.time() - t0 > timeout:
                return False
            time.sleep(0.0005)
        return True

    def close(self) -> None:
        with self._lock:
            self._stop = True
            self._lock.notify_all()


# ---- transports -----------------------------------------------------------------------------------------------------
class DistTransport:
    """torch.distributed point-to-point (NCCL between GPUs, gloo on CPU)."""

    def __init__(self, group=None):
        self.group = group

    def send(self, t: torch.Tensor, peer: int) -> None:
        dist.send(t.contiguous(), dst=peer, group=self.group)

    def recv(self, t: torch.Tensor, peer: int) -> None:
        dist.recv(t, src=peer, group=self.group)


class TcpTransport:
    """Host-staged TCP stream for instances that share no process group (the reference's TCP communicator)."""

    def __init__(self, sock: socket.socket):
        self.sock = sock
        self.sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)

    @staticmethod
    def listen(host: str, port: int) -> "TcpTransport":
        srv = socket.socket()
        srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        srv.bind((host, port))
        srv.listen(1)
        conn, _ = srv.accept()
        srv.close()
        return TcpTransport(conn)

    @staticmethod
    def connect(host: str, port: int, retries: int = 100) -> "TcpTransport":
        for _ in range(retries):
            try:
                return TcpTransport(socket.create_connection((host, port)))
            except OSError:
                time.sleep(0.05)
        raise ConnectionError(f"cannot reach {host}:{port}")

    def send(self, t: torch.Tensor, peer: int = 0) -> None:
        raw = t.detach().to("cpu").contiguous().view(torch.uint8).numpy().tobytes()
        self.sock.sendall(struct.pack("<q", len(raw)) + raw)

    def recv(self, t: torch.Tensor, peer: int = 0) -> None:
        n = struct.unpack("<q", self._read(8))[0]
        buf = torch.frombuffer(bytearray(self._read(n)), dtype=torch.uint8)
        t.copy_(buf.view(t.dtype).view(t.shape))

    def _read(self, n: int) -> bytes:
        chunks = []
        while n:
            c = self.sock.recv(min(n, 1 << 20))
            if not c:
                raise ConnectionError("peer closed")
            chunks.append(c)
            n -= len(c)
        return b"".join(chunks)


# ---- engine ------------------------------------------------------------------------------------------------------------
class TransferEngine:
    def __init__(self, kv_caches: Sequence[torch.Tensor], cache_manager, transport, block_size: int):
        self.kv, self.cache, self.tr, self.block_size = list(kv_caches), cache_manager, transport, block_size
        self._tmp_ids = iter(range(-2, -(1 << 40), -1))
        self.sent_blocks = self.recv_blocks = 0

    def _hdr(self) -> torch.Tensor:
        return torch.zeros(4, dtype=torch.int64)

    def export_request(self, tokens: Sequence[int], first_tokens: Sequence[int], peer: int,
                       tracker: Optional[LayerProgressTracker] = None, on_blocks=None) -> int:
        """Sends the KV of every FULL block of ``tokens`` (they must still be in the prefix tree: the request was
        just prefilled with prefix caching on) followed by the tokens generated so far. Returns blocks sent."""
        toks = [int(t) for t in tokens]
        tmp = next(self._tmp_ids)
        hit = self.cache.create_seq(tmp, toks + [0])  # + 1: matching never covers the whole sequence
        n_blocks = hit // self.block_size
        blocks = list(self.cache.block_table(tmp))[:n_blocks]
        try:
            if on_blocks is not None:
                on_blocks(blocks)  # tensor-parallel instances: the other ranks send their shard of the same blocks
            h = self._hdr()
            h[0], h[1], h[2], h[3] = len(toks), n_blocks, len(first_tokens), len(self.kv)
            self.tr.send(h, peer)
            self.tr.send(torch.tensor(toks + [int(t) for t in first_tokens], dtype=torch.int32), peer)
            if n_blocks:
                idx = torch.tensor(blocks, dtype=torch.long, device=self.kv[0].device)
                send_layer = lambda l: self.tr.send(self.kv[l].index_select(0, idx), peer)  # noqa: E731
                if tracker is not None:
                    # layers are pushed as the device finishes them
                    done = threading.Event()

                    def cb(layer, _n=len(self.kv)):
                        send_layer(layer)
                        if layer == _n - 1:
                            done.set()
                    tracker.register_callback(cb)
                    done.wait(60.0)
                else:
                    for l in range(len(self.kv)):
                        send_layer(l)
            self.sent_blocks += n_blocks
        finally:
            self.cache.free_seq(tmp)
        return n_blocks

    # ---- layer-by-layer export: header + tokens first, each layer when the device has finished it, the tokens
    # generated so far last (they do not exist yet while the layers leave) -------------------------------------------
    def begin_export(self, tokens: Sequence[int], blocks: Sequence[int], peer: int) -> None:
        toks = [int(t) for t in tokens]
        h = self._hdr()
        h[0], h[1], h[2], h[3] = len(toks), len(blocks), -1, len(self.kv)  # -1: the generated tokens follow the layers
        self.tr.send(h, peer)
        self.tr.send(torch.tensor(toks, dtype=torch.int32), peer)
        self._lw_idx = torch.tensor(list(blocks), dtype=torch.long, device=self.kv[0].device) if blocks else None

    def send_layer(self, layer: int, peer: int) -> None:
        if self._lw_idx is not None:
            self.tr.send(self.kv[layer].index_select(0, self._lw_idx), peer)

    def finish_export(self, first_tokens: Sequence[int], peer: int) -> None:
        t = torch.tensor([len(first_tokens)] + [int(x) for x in first_tokens], dtype=torch.int32)
        self.tr.send(torch.tensor([t.numel()], dtype=torch.int64), peer)
        self.tr.send(t, peer)
        self.sent_blocks += 0 if self._lw_idx is None else int(self._lw_idx.numel())

    def import_request(self, peer: int, lock=None, after_commit=None) -> Tuple[List[int], List[int], int]:
        """Receives one exported request. Returns (prompt tokens, tokens already generated, blocks placed in the
        prefix tree). ``lock``: held only while the cache manager is touched (block reservation before the layers
        arrive, commit after them), not while the layers are in flight: a layer-by-layer export lasts as long as the
        sender's forward pass. ``after_commit(first_block_kept, blocks)`` runs under the same hold as the commit."""
        import contextlib
        guard = lock if lock is not None else contextlib.nullcontext()
        h = self._hdr()
        self.last_import = (0, [])
        self.tr.recv(h, peer)
        n_tok, n_blocks, n_first, n_layers = (int(x) for x in h)
        assert n_layers == len(self.kv), "both instances must hold the same layers"
        trailer = n_first < 0  # layer-by-layer export: the generated tokens arrive after the layers
        tt = torch.zeros(n_tok + max(n_first, 0), dtype=torch.int32)
        self.tr.recv(tt, peer)
        toks, first = tt[:n_tok].tolist(), tt[n_tok:].tolist()

        def read_trailer():
            n = torch.zeros(1, dtype=torch.int64)
            self.tr.recv(n, peer)
            t = torch.zeros(int(n[0]), dtype=torch.int32)
            self.tr.recv(t, peer)
            return t[1:1 + int(t[0])].tolist()

        if n_blocks == 0:
            return toks, (read_trailer() if trailer else first), 0
        tmp = next(self._tmp_ids)
        covered = n_blocks * self.block_size
        with guard:
            hit = self.cache.create_seq(tmp, toks[:covered] + [0])
            have = hit // self.block_size
            ok = self.cache.ensure_capacity(tmp, covered)
            table = list(self.cache.block_table(tmp)) if ok else []
        dev = self.kv[0].device
        for l in range(n_layers):
            buf = torch.empty((n_blocks,) + tuple(self.kv[l].shape[1:]), dtype=self.kv[l].dtype, device=dev)
            self.tr.recv(buf, peer)
            if ok and have < n_blocks:
                idx = torch.tensor(table[have:n_blocks], dtype=torch.long, device=dev)
                self.kv[l].index_copy_(0, idx, buf[have:])
        if trailer:
            first = read_trailer()
        placed = 0
        with guard:
            if ok:
                self.cache.commit_filled(tmp, toks[:covered] + [0], covered)
                placed = n_blocks - have
            self.last_import = (have, table[have:n_blocks] if ok else [])  # which received blocks went where
            self.cache.free_seq(tmp)
            if after_commit is not None:
                after_commit(*self.last_import)
        self.recv_blocks += placed
        return toks, first, placed

    # ---- shards of a tensor-parallel instance: same block ids on every rank, no token metadata ----------------
    def export_shard(self, blocks: Sequence[int], peer: int = 0) -> None:
        h = self._hdr()
        h[1], h[3] = len(blocks), len(self.kv)
        self.tr.send(h, peer)
        if blocks:
            idx = torch.tensor(list(blocks), dtype=torch.long, device=self.kv[0].device)
            for l in range(len(self.kv)):
                self.tr.send(self.kv[l].index_select(0, idx), peer)

    def import_shard(self, peer: int = 0) -> List[torch.Tensor]:
        """Receives one shard into host tensors (one per layer, [n_blocks, ...]); ``place_shard`` puts them into the
        cache once the driving rank has said which blocks they belong to."""
        h = self._hdr()
        self.tr.recv(h, peer)
        n_blocks, n_layers = int(h[1]), int(h[3])
        assert n_layers == len(self.kv), "both instances must hold the same layers"
        bufs = []
        for l in range(n_layers):
            buf = torch.empty((n_blocks,) + tuple(self.kv[l].shape[1:]), dtype=self.kv[l].dtype)
            if n_blocks:
                self.tr.recv(buf, peer)
            bufs.append(buf)
        return bufs

    def place_shard(self, bufs: Sequence[torch.Tensor], skip: int, blocks: Sequence[int]) -> None:
        if not blocks:
            return
        dev = self.kv[0].device
        idx = torch.tensor(list(blocks), dtype=torch.long, device=dev)
        for l, buf in enumerate(bufs):
            self.kv[l].index_copy_(0, idx, buf[skip:skip + len(blocks)].to(dev))
