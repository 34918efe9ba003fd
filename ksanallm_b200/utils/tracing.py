"""Tracing: NVTX ranges and the scheduler event tracer.

* ``profile_scope(name)``: NVTX push/pop around a region when ``ENABLE_PROFILE_EVENT`` is set (reference:
  src/ksana_llm/profiler/profile_event.cpp:12-43, macro PROFILE_EVENT_SCOPE).
* ``ScheduleEventTracer``: ``KLLM_SCHED_TRACE_LEVEL=1|2`` records Begin/End events per step (level 1) and per
  request (level 2) into ``sched_events_node_<rank>.csv`` from a writer thread (reference:
  src/ksana_llm/profiler/sched_event_tracer.cpp:17-45); ``summarise_trace`` is the post-processor
  (reference: tools/profiler/sched_event_trace_process.py) and can also emit a Chrome trace JSON.
"""
from __future__ import annotations

import contextlib
import csv
import json
import os
import queue
import threading
import time
from typing import Dict, List, Optional

_NVTX = os.environ.get("ENABLE_PROFILE_EVENT") is not None


@contextlib.contextmanager
def profile_scope(name: str):
    if not _NVTX:
        yield
        return
    import torch
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


class ScheduleEventTracer:
    FIELDS = ["time_ns", "node_rank", "event", "phase", "step", "req_id", "batch_size", "token_num"]

    def __init__(self, rank: int = 0, level: Optional[int] = None, directory: str = "."):
        self.level = int(os.environ.get("KLLM_SCHED_TRACE_LEVEL", "0")) if level is None else level
        self.rank = rank
        self.path = os.path.join(directory, f"sched_events_node_{rank}.csv")
        self.q: "queue.Queue" = queue.Queue()
        self._thread = None
        if self.level > 0:
            self._thread = threading.Thread(target=self._writer, daemon=True, name="ksana-sched-trace")
            self._thread.start()

    @property
    def enabled(self) -> bool:
        return self.level > 0

    def record(self, event: str, phase: str, step: int = 0, req_id: int = -1, batch_size: int = 0,
               token_num: int = 0, level: int = 1) -> None:
        if self.level >= level:
            self.q.put((time.time_ns(), self.rank, event, phase, step, req_id, batch_size, token_num))

    @contextlib.contextmanager
    def span(self, event: str, step: int = 0, batch_size: int = 0, token_num: int = 0):
        self.record(event, "B", step, -1, batch_size, token_num)
        try:
            yield
        finally:
            self.record(event, "E", step, -1, batch_size, token_num)

    def _writer(self) -> None:
        with open(self.path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(self.FIELDS)
            while True:
                item = self.q.get()
                if item is None:
                    break
                w.writerow(item)
                if self.q.empty():
                    f.flush()

    def close(self) -> None:
        if self._thread is not None:
            self.q.put(None)
            self._thread.join(timeout=5)
            self._thread = None


def summarise_trace(csv_path: str, chrome_trace_path: Optional[str] = None) -> Dict[str, Dict[str, float]]:
    """Per-event count / total / mean / max duration in ms; optionally writes a Chrome trace (chrome://tracing)."""
    open_ev: Dict[tuple, int] = {}
    stats: Dict[str, List[float]] = {}
    chrome = []
    with open(csv_path, newline="") as f:
        for row in csv.DictReader(f):
            key = (row["event"], row["step"], row["req_id"])
            t = int(row["time_ns"])
            if row["phase"] == "B":
                open_ev[key] = t
            elif key in open_ev:
                t0 = open_ev.pop(key)
                stats.setdefault(row["event"], []).append((t - t0) / 1e6)
                chrome.append({"name": row["event"], "ph": "X", "ts": t0 / 1e3, "dur": (t - t0) / 1e3,
                               "pid": int(row["node_rank"]), "tid": 0 if row["req_id"] == "-1" else int(row["req_id"]),
                               "args": {"step": row["step"], "batch": row["batch_size"], "tokens": row["token_num"]}})
    if chrome_trace_path:
        with open(chrome_trace_path, "w") as f:
            json.dump({"traceEvents": chrome}, f)
    return {k: {"count": len(v), "total_ms": sum(v), "mean_ms": sum(v) / len(v), "max_ms": max(v)}
            for k, v in stats.items()}


if __name__ == "__main__":
    import sys
    print(json.dumps(summarise_trace(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else None), indent=1))
