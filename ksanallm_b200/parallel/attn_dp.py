"""Attention data parallelism with expert parallelism for the MoE blocks.

Every rank (DP group of one rank here) owns its own requests, scheduler and KV cache and holds the full attention /
dense weights; only the routed experts are sharded over the ranks. All ranks step in lock-step: each MoE block is
a collective exchange (tokens to the ranks hosting their experts, weighted outputs back), so a rank without work
still runs a "mock" step with zero tokens. This mirrors the reference's attn_data_para_size mode: per-DP-group
strategies and cache managers (src/ksana_llm/service/inference_engine.cpp:201-260), mock requests so idle EP ranks
still run a step (batch_scheduler/batch_scheduler.cpp:472-519) and the cross-DP synchronisation of step sizes.
"""
from __future__ import annotations

import time
import threading
import struct
import socket
import json
from typing import Any, Dict, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops


class DPCoordinator:
    """Per-step agreement between the DP ranks: the largest token count of any rank (the slot stride of the
    expert exchange) and whether anybody still has work."""

    def __init__(self, group=None, device: Optional[torch.device] = None):
        self.group = group
        self.device = device or torch.device("cpu")
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)

    def sync(self, local_tokens: int, has_unfinished: bool) -> Tuple[int, bool]:
        t = torch.tensor([local_tokens, 1 if has_unfinished else 0, 1 if self.stop_requested else 0],
                         dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        self.stopping = bool(t[2])  # every rank learns of a shutdown in the same step and leaves the loop together
        return int(t[0]), bool(t[1])

    stop_requested = False
    stopping = False


class ADPBalance:
    """Lines the DP ranks' prefills up. The ranks step in lock-step (the MoE exchange joins them), so one rank's
    long prefill stretches the decode step of all the others; holding new prompts back until EVERY rank has one to
    start - or some rank has nothing to decode, or the wait has lasted too long, or traffic is high enough that
    prompts arrive everywhere anyway - makes the long steps coincide. Reference: BatchScheduler::BalanceADPRequests,
    IsADPBalanceTimeout, UpdateQPS (batch_scheduler/batch_scheduler.cpp:588-737) and
    setting.batch_scheduler.attention_dp_lb_config.

    Every rank owns its requests here, so the rule reads "every rank has a waiting request" where the reference,
    which re-deals one global waiting pool, counts them. Clocks differ between processes: rank 0 evaluates the
    time-based conditions and its verdict travels with the gathered counts, so all ranks decide alike."""

    def __init__(self, coord: DPCoordinator, max_waiting_steps: int = 50, max_waiting_time_ms: int = 1000,
                 min_qps_for_waiting: float = -1.0, qps_window_s: float = 1.0, clock=time.monotonic):
        self.coord = coord
        self.max_steps, self.max_ms, self.min_qps = int(max_waiting_steps), int(max_waiting_time_ms), float(min_qps_for_waiting)
        self.window, self.clock = float(qps_window_s), clock
        self.waiting_iters = 0
        self.hold_started = 0.0
        self.qps = 0.0
        self._arrivals, self._window_start = 0, clock()
        self.held_steps = self.released_by_timeout = 0

    def _update_qps(self, arrivals: int) -> None:
        self._arrivals += arrivals
        now = self.clock()
        if now - self._window_start >= self.window:
            self.qps = self._arrivals / (now - self._window_start)
            self._arrivals, self._window_start = 0, now

    def decide(self, num_waiting: int, num_running: int, arrivals: int = 0) -> bool:
        """One call per step on every rank (a collective). True: this step may start new prompts."""
        t = torch.tensor([num_waiting, num_running, arrivals, 0, 0], dtype=torch.int64, device=self.coord.device)
        rows = [torch.empty_like(t) for _ in range(self.coord.size)]
        if self.coord.rank == 0:
            self._update_qps(0)  # the window also closes in steps without arrivals
            busy = self.min_qps >= 0 and self.qps > self.min_qps
            timed_out = self.waiting_iters > 0 and (self.clock() - self.hold_started) * 1000.0 >= self.max_ms
            t[3], t[4] = int(timed_out), int(busy)
        dist.all_gather(rows, t, group=self.coord.group)
        g = torch.stack(rows).tolist()
        if self.coord.rank == 0:
            self._update_qps(sum(r[2] for r in g))
        waiting, running = [r[0] for r in g], [r[1] for r in g]
        timed_out, busy = bool(g[0][3]), bool(g[0][4])
        if sum(waiting) == 0:
            self.waiting_iters = 0
            return True
        timeout = busy or timed_out or self.waiting_iters >= self.max_steps
        proceed = all(w > 0 for w in waiting) or not all(r > 0 for r in running) or timeout
        if proceed:
            if timeout and not all(w > 0 for w in waiting):
                self.released_by_timeout += 1
            self.waiting_iters = 0
            return True
        if self.waiting_iters == 0:
            self.hold_started = self.clock()
        self.waiting_iters += 1
        self.held_steps += 1
        return False


class GatherEPExchange:
    """Same contract as parallel.ep.EPExchange.moe, built from torch.distributed collectives (works on gloo and
    NCCL): all-gather the padded token slots, run the local experts on everything, sum the partial outputs and keep
    the rank's own rows. Used on CPU and wherever symmetric memory is not available."""

    def __init__(self, group, rank: int, size: int, top_k: int, num_experts: int):
        assert num_experts % size == 0
        self.group, self.rank, self.size, self.top_k = group, rank, size, top_k
        self.e_local = num_experts // size
        self.step_stride = 0

    custom_experts = True  # moe() accepts experts_fn (quantised expert weights)

    def moe(self, x, ids, weights, w_gate_up, w_down, t_stride, add=None, experts_fn=None):
        """``experts_fn(x_all, ids_all, weights_all) -> y_all``: the rank's local experts over the gathered tokens,
        for expert weights that are not plain bf16 / fp32 tensors (fp8 block-scaled, 4-bit)."""
        T, H = x.shape
        k = self.top_k
        xp = x.new_zeros(t_stride, H)
        ip = torch.full((t_stride, k), -1, dtype=torch.int32, device=x.device)
        wp = torch.zeros(t_stride, k, dtype=torch.float32, device=x.device)
        if T:
            xp[:T], ip[:T], wp[:T] = x, ids.to(torch.int32), weights.float()
        xg = [torch.empty_like(xp) for _ in range(self.size)]
        ig = [torch.empty_like(ip) for _ in range(self.size)]
        wg = [torch.empty_like(wp) for _ in range(self.size)]
        dist.all_gather(xg, xp, group=self.group)
        dist.all_gather(ig, ip, group=self.group)
        dist.all_gather(wg, wp, group=self.group)
        if experts_fn is not None:
            y = experts_fn(torch.cat(xg), torch.cat(ig), torch.cat(wg))
        else:
            y = ops.moe_experts(torch.cat(xg), torch.cat(ig), torch.cat(wg), w_gate_up, w_down, self.rank * self.e_local)
        y = y.float()
        dist.all_reduce(y, group=self.group)
        out = y[self.rank * t_stride:self.rank * t_stride + T].to(x.dtype)
        return out if add is None else out + add


# ---- request distribution for a served DP instance ------------------------------------------------------------------
# One process per GPU means one scheduler per DP rank, but a served instance has ONE HTTP front-end (rank 0). Rank 0
# deals every request to the least loaded rank (the reference: BatchScheduler::BalanceWaitingReqs deals its waiting
# pool over the attention-DP groups by token load, batch_scheduler_balance_reqs_algo.cpp:11-55); remote ranks run the
# request in their own engine and stream the new tokens back over a TCP link.

def _send_msg(sock: socket.socket, obj) -> None:
    data = json.dumps(obj).encode()
    sock.sendall(struct.pack("<I", len(data)) + data)


def _recv_msg(sock: socket.socket):
    hdr = b""
    while len(hdr) < 4:
        c = sock.recv(4 - len(hdr))
        if not c:
            return None
        hdr += c
    n = struct.unpack("<I", hdr)[0]
    buf = bytearray()
    while len(buf) < n:
        c = sock.recv(min(n - len(buf), 1 << 20))
        if not c:
            return None
        buf += c
    return json.loads(bytes(buf))


class DPRequestRouter:
    """Rank 0: owns the links to the other DP ranks, places requests, mirrors remote progress into local Request
    objects so that the serving layer streams them like its own."""

    def __init__(self, engine, host: str, port: int, world: int, accept_timeout: float = 120.0):
        self.engine, self.world = engine, world
        self.links: Dict[int, socket.socket] = {}
        self.load = [0] * world          # outstanding prompt + budgeted output tokens per rank
        self.remote: Dict[int, Tuple[Any, int, int]] = {}  # rid -> (Request, rank, weight)
        self.lock = threading.Lock()
        self._rid = 0
        self.placed = [0] * world
        srv = socket.socket()
        srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        srv.bind((host, port))
        srv.listen(world)
        srv.settimeout(accept_timeout)
        self.port = srv.getsockname()[1]
        self._srv = srv

    def accept_all(self) -> None:
        while len(self.links) < self.world - 1:
            conn, _ = self._srv.accept()
            hello = _recv_msg(conn)
            self.links[int(hello["rank"])] = conn
            threading.Thread(target=self._reader, args=(int(hello["rank"]), conn), daemon=True).start()
        self._srv.close()

    def place(self, n_tokens: int) -> int:
        with self.lock:
            r = min(range(self.world), key=lambda i: (self.load[i], i))
            self.load[r] += n_tokens
            self.placed[r] += 1
            return r

    def release(self, rank: int, n_tokens: int) -> None:
        with self.lock:
            self.load[rank] -= n_tokens

    def submit(self, rank: int, req, weight: int) -> None:
        import dataclasses
        with self.lock:
            self._rid += 1
            rid = self._rid
            self.remote[rid] = (req, rank, weight)
        req.dp_remote = (rank, rid)
        _send_msg(self.links[rank], {"op": "add", "rid": rid, "tokens": list(req.prompt_tokens),
                                     "params": dataclasses.asdict(req.params)})

    def abort(self, req) -> None:
        rank, rid = req.dp_remote
        try:
            _send_msg(self.links[rank], {"op": "abort", "rid": rid})
        except OSError:
            pass

    def _reader(self, rank: int, conn: socket.socket) -> None:
        while True:
            try:
                m = _recv_msg(conn)
            except OSError:
                m = None
            if m is None:
                break
            with self.lock:
                ent = self.remote.get(m["rid"])
            if ent is None:
                continue
            req, _, weight = ent
            so = req.seqs[0]
            so.output_tokens.extend(m.get("tokens", []))
            now = time.time()
            if m.get("tokens") and req.first_token_time is None:
                req.first_token_time = now
            req.token_times.extend([now] * len(m.get("tokens", [])))
            if m.get("finished"):
                so.finished, so.finish_reason = True, m.get("reason")
                if m.get("error"):
                    from ..engine.llm_engine import EngineError
                    req.error = EngineError(int(m.get("code", 7)), m["error"])
                req.finished, req.finish_time = True, now
                with self.lock:
                    self.remote.pop(m["rid"], None)
                self.release(rank, weight)
            req.notify()
        # a lost link fails what that rank still owed
        with self.lock:
            lost = [(rid, e) for rid, e in self.remote.items() if e[1] == rank]
        for rid, (req, _, weight) in lost:
            from ..engine.llm_engine import EngineError
            req.error = EngineError(7, f"attention-DP rank {rank} is gone")
            req.seqs[0].finished = req.finished = True
            req.notify()

    def close(self) -> None:
        for c in self.links.values():
            try:
                c.close()
            except OSError:
                pass


class DPRequestWorker:
    """Ranks > 0: receives requests from rank 0, runs them in the local engine, reports progress after every step."""

    def __init__(self, engine, host: str, port: int, rank: int, connect_timeout: float = 120.0):
        self.engine, self.rank = engine, rank
        deadline = time.time() + connect_timeout
        while True:
            try:
                self.sock = socket.create_connection((host, port), timeout=5)
                break
            except OSError:
                if time.time() > deadline:
                    raise
                time.sleep(0.1)
        self.sock.settimeout(None)
        _send_msg(self.sock, {"rank": rank})
        self.active: Dict[int, Tuple[Any, int]] = {}  # rid -> (Request, tokens already reported)
        self.lock = threading.Lock()
        threading.Thread(target=self._reader, daemon=True).start()

    def _reader(self) -> None:
        from ..engine.sampling_params import SamplingParams
        while True:
            try:
                m = _recv_msg(self.sock)
            except OSError:
                m = None
            if m is None:
                return
            if m["op"] == "add":
                try:
                    req = self.engine.add_request(m["tokens"], SamplingParams.from_dict(m["params"]), local=True)
                    with self.lock:
                        self.active[m["rid"]] = (req, 0)
                except Exception as ex:  # reported back instead of killing the link
                    _send_msg(self.sock, {"rid": m["rid"], "finished": True, "reason": "error", "error": str(ex),
                                          "code": getattr(ex, "code", 7)})
            elif m["op"] == "abort":
                with self.lock:
                    ent = self.active.get(m["rid"])
                if ent is not None:
                    self.engine.abort(ent[0])

    def report(self) -> None:
        """Called by the step loop after every step."""
        with self.lock:
            items = list(self.active.items())
        for rid, (req, sent) in items:
            toks = req.seqs[0].output_tokens if req.seqs else []
            if len(toks) == sent and not req.finished:
                continue
            msg = {"rid": rid, "tokens": list(toks[sent:]), "finished": bool(req.finished)}
            if req.finished:
                msg["reason"] = req.seqs[0].finish_reason if req.seqs else "error"
                if req.error is not None:
                    msg["error"], msg["code"] = str(req.error), req.error.code
            try:
                _send_msg(self.sock, msg)
            except OSError:
                return
            with self.lock:
                if req.finished:
                    self.active.pop(rid, None)
                else:
                    self.active[rid] = (req, len(toks))
