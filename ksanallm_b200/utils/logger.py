"""Process logging set up from the reference's environment variables.

* ``KLLM_LOG_LEVEL``: a base level (DEBUG / INFO / WARNING / ERROR) and / or comma-separated categories that get
  DEBUG output - ATTENTION, COMMUNICATION, MOE, MODEL, SCHEDULER, MAIN, MULTI_BATCH (e.g. ``INFO,SCHEDULER``);
* ``KLLM_LOG_FILE``: log file (default ``log/ksana_llm.log``; ``-`` or ``stderr`` for the console only);
* ``KLLM_STAT_FILE``: append one JSON line of engine state every ``state_interval_s`` seconds.

Reference: src/ksana_llm/utils/logger.h:39-160 (levels + categories), batch_scheduler.cpp:423-470 (a state line
every 10 s), profiler/writer.cpp (KLLM_STAT_FILE).
"""
from __future__ import annotations

import json
import logging
import os
import threading
import time
from typing import Optional

CATEGORIES = ("ATTENTION", "COMMUNICATION", "MOE", "MODEL", "SCHEDULER", "MAIN", "MULTI_BATCH")
_ROOT = "ksanallm"
_configured = False


def get_logger(category: str = "MAIN") -> logging.Logger:
    return logging.getLogger(f"{_ROOT}.{category.upper()}")


def setup_logging(level_spec: Optional[str] = None, log_file: Optional[str] = None, rank: int = 0) -> logging.Logger:
    """Idempotent. Returns the MAIN logger."""
    global _configured
    spec = level_spec if level_spec is not None else os.environ.get("KLLM_LOG_LEVEL", "INFO")
    path = log_file if log_file is not None else os.environ.get("KLLM_LOG_FILE", "log/ksana_llm.log")
    root = logging.getLogger(_ROOT)
    if _configured:
        return get_logger("MAIN")
    base, debug_cats = logging.INFO, []
    for part in (p.strip().upper() for p in spec.split(",") if p.strip()):
        if part in CATEGORIES:
            debug_cats.append(part)
        elif part in ("DEBUG", "INFO", "WARNING", "ERROR", "CRITICAL"):
            base = getattr(logging, part)
    root.setLevel(base)
    for cat in debug_cats:
        get_logger(cat).setLevel(logging.DEBUG)
    fmt = logging.Formatter(f"%(asctime)s rank{rank} %(levelname)s %(name)s: %(message)s")
    handler: logging.Handler
    if path in ("-", "stderr", ""):
        handler = logging.StreamHandler()
    else:
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        handler = logging.FileHandler(path if rank == 0 else f"{path}.rank{rank}")
    handler.setFormatter(fmt)
    handler.setLevel(logging.DEBUG)
    root.addHandler(handler)
    root.propagate = False
    _configured = True
    return get_logger("MAIN")


def engine_state(llm) -> dict:
    st, cs = llm.sched.stats, llm.cache.stats
    total = llm.cache.num_device_blocks
    free = llm.cache.num_available_blocks
    return {"time": round(time.time(), 3), "step": llm.step_count, "waiting": llm.sched.num_waiting,
            "running": llm.sched.num_running, "swapped": llm.sched.num_swapped,
            "blocks_used": total - free, "blocks_total": total,
            "generated_tokens": llm.stats["generated_tokens"], "prompt_tokens": llm.stats["prompt_tokens"],
            "prefix_hit_tokens": cs.prefix_hit_tokens, "flexible_hit_tokens": cs.flexible_hit_tokens,
            "preempt_recompute": st.preempt_recompute, "preempt_swap": st.preempt_swap,
            "draft_proposed": st.draft_proposed, "draft_accepted": st.draft_accepted}


class StateReporter:
    """Logs one scheduler state line every ``interval_s`` seconds (and appends it to KLLM_STAT_FILE when set)."""

    def __init__(self, llm, interval_s: float = 10.0, stat_file: Optional[str] = None):
        self.llm, self.interval = llm, interval_s
        self.stat_file = stat_file if stat_file is not None else os.environ.get("KLLM_STAT_FILE", "")
        self.log = get_logger("SCHEDULER")
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="ksana-state", daemon=True)

    def start(self) -> "StateReporter":
        self._thread.start()
        return self

    def report_once(self) -> dict:
        s = engine_state(self.llm)
        self.log.info("state " + " ".join(f"{k}={v}" for k, v in s.items() if k != "time"))
        if self.stat_file:
            with open(self.stat_file, "a", encoding="utf-8") as f:
                f.write(json.dumps(s) + "\n")
        return s

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self.report_once()
            except Exception:  # a reporter never takes the server down
                self.log.exception("state report failed")

    def stop(self) -> None:
        self._stop.set()
