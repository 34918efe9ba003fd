"""The serving engine: request intake, the step loop, output delivery.

Rank 0 owns the native scheduler (C++), plans every step, broadcasts the packed plan to the other
tensor-parallel ranks (one int32 buffer over the CPU process group), runs its shard of the model and
samples. Other ranks run :meth:`LLMEngine.follow`. Reference counterparts: InferenceEngine
(src/ksana_llm/service/inference_engine.cpp:56-370, 418-561), BatchManager::MainProcess
(batch_manager/batch_manager.cpp:119-214), LlmRuntime::StepOnChief (runtime/llm_runtime.cpp:290-338).
"""
from __future__ import annotations

import contextlib
import itertools
import json
import os
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from .. import host as _host
from ..config.model_config import ModelConfig
from ..config.schema import ServingConfig
from ..models.transformer import TransformerModel
from ..parallel.comm import TPGroup
from ..utils import tracing as _tracing
from .model_runner import ModelRunner
from .sampler import SampleRow
from .sampling_params import SamplingParams

FINISH_NAMES = {
    _host.FINISH_NONE: None, _host.FINISH_EOS: "stop", _host.FINISH_STOP_TOKEN: "stop", _host.FINISH_LENGTH: "length",
    _host.FINISH_ABORTED: "abort", _host.FINISH_TIMEOUT: "timeout", _host.FINISH_STOP_STRING: "stop",
    _host.FINISH_ERROR: "error",
}


class EngineError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


@dataclass
class SequenceOutput:
    seq_id: int
    output_tokens: List[int] = field(default_factory=list)
    logprobs: List[Any] = field(default_factory=list)
    finished: bool = False
    finish_reason: Optional[str] = None
    cum_logprob: float = 0.0
    text_checked: int = 0  # number of output tokens already scanned for stop strings


class Request:
    """One user request = one or more output sequences (parallel sampling / beams)."""

    def __init__(self, req_id: int, prompt_tokens: List[int], params: SamplingParams, arrival: float):
        self.req_id = req_id
        self.prompt_tokens = prompt_tokens
        self.params = params
        self.arrival = arrival
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        self.token_times: List[float] = []
        self.seqs: List[SequenceOutput] = []
        self.finished = False
        self.error: Optional[EngineError] = None
        self.cond = threading.Condition()
        self.version = 0
        self.aborted = False
        self.refit = None
        self.grammar = None
        self.probe = None  # /forward request targets
        self.probe_result = None
        self.generators: Dict[int, torch.Generator] = {}
        self.tries: Dict[int, Any] = {}
        self.beam = None
        self.mrope = None      # [3, prompt_len] multimodal RoPE positions (None: text-only)
        self.mrope_delta = 0

    def notify(self) -> None:
        with self.cond:
            self.version += 1
            self.cond.notify_all()

    def wait(self, last_version: int, timeout: Optional[float] = None) -> int:
        with self.cond:
            if self.version == last_version and not self.finished:
                self.cond.wait(timeout)
            return self.version

    @property
    def output_token_ids(self) -> List[List[int]]:
        return [list(s.output_tokens) for s in self.seqs]


class LLMEngine:
    def __init__(self, model: TransformerModel, serving: ServingConfig, tp: Optional[TPGroup] = None,
                 num_blocks: Optional[int] = None, num_host_blocks: Optional[int] = None,
                 detokenize: Optional[Callable[[List[int]], str]] = None, seed: int = 0,
                 kv_dtype: Optional[torch.dtype] = None, block_sync_group=None):
        self.model = model
        self._block_sync_group = block_sync_group  # pipeline stages: world group for the block-count agreement
        self.cfg: ModelConfig = model.cfg
        self.serving = serving
        self.tp = tp or model.tp
        self.detokenize = detokenize
        bs_cfg, bm_cfg = serving.setting.batch_scheduler, serving.setting.block_manager
        self.block_size = 64 if self.cfg.use_mla and bm_cfg.block_token_num == 16 else bm_cfg.block_token_num
        if num_blocks is None:
            num_blocks = self._derive_num_blocks(kv_dtype)
        if num_host_blocks is None:
            num_host_blocks = int(num_blocks * bm_cfg.block_host_memory_factor) if bs_cfg.preempt_mode == 0 else 0
            num_host_blocks = min(num_host_blocks, self._host_block_cap(kv_dtype))
        self.num_blocks = num_blocks
        max_blocks_per_seq = (bs_cfg.max_token_len + self.block_size - 1) // self.block_size + 1
        self.runner = ModelRunner(model, num_blocks, self.block_size, num_host_blocks, bs_cfg.max_step_tokens,
                                  bs_cfg.max_batch_size, max_blocks_per_seq, kv_dtype, seed)
        self.runner.sampler.eos_token_ids = list(model.cfg.eos_token_ids)
        self.is_driver = self.tp.rank == 0  # with pipeline stages: re-set by attach_pipeline (global rank 0 drives)
        # drafts per step from the first next-n module (applied repeatedly for more than one; tensor-parallel peers
        # receive each further pass's rows from the driver)
        self.mtp_steps = bs_cfg.mtp_step_num if (bs_cfg.enable_speculative_decoding or bs_cfg.mtp_step_num) \
            and model.mtp_layers else 0
        self.trie_drafts = 3 if (bs_cfg.enable_speculative_decoding and not model.mtp_layers) else 0
        sc = _host.SchedulerConfig()
        sc.block_size = self.block_size
        sc.max_batch_size = bs_cfg.max_batch_size
        sc.max_step_tokens = bs_cfg.max_step_tokens
        sc.max_token_len = bs_cfg.max_token_len
        sc.max_waiting_queue_len = bs_cfg.max_waiting_queue_len
        sc.waiting_timeout_ms = bs_cfg.waiting_timeout_in_ms
        sc.split_fuse_token_num = bs_cfg.split_fuse_token_num
        sc.preempt_mode = bs_cfg.preempt_mode if num_host_blocks > 0 else 1
        sc.launch_block_threshold = bs_cfg.launch_block_threshold
        sc.swapin_block_threshold = bs_cfg.swapin_block_threshold
        # parallel token prediction (config.json: num_register_token / reg_token_id): N register tokens follow the
        # last real token and every position yields a token (reference: runtime/draft_generator/ptp_generator.cpp)
        self.ptp_steps = int(getattr(model.cfg, "num_register_token", 0) or 0)
        self.ptp_token = int(getattr(model.cfg, "reg_token_id", 0) or 0)
        if self.ptp_steps:
            self.mtp_steps = self.trie_drafts = 0
        sc.max_draft_tokens = max(self.mtp_steps, self.trie_drafts, self.ptp_steps)
        sc.ptp_mode = self.ptp_steps > 0
        sc.pp_wb_strategy = int(getattr(bs_cfg, "pp_multibatch_wb_strategy", 0) or 0)
        sc.lookahead_slots = max(self.mtp_steps - 1, 0)
        sc.min_flexible_cache_num = self._flexible_cache_min(bs_cfg, model, kv_dtype)
        sc.decode_token_threshold = 1 + sc.max_draft_tokens
        self.cache = _host.KVCacheManager(num_blocks, num_host_blocks, self.block_size,
                                          bool(bs_cfg.enable_auto_prefix_cache))
        self.sched = _host.Scheduler(sc, self.cache)
        self.sched_cfg = sc
        self._ids = itertools.count(1)
        self._seq_ids = itertools.count(1)
        self.requests: Dict[int, Request] = {}
        self.seq_owner: Dict[int, Tuple[Request, SequenceOutput]] = {}
        self.lock = threading.RLock()
        self._loop_thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self._wake = threading.Event()
        self.step_count = 0
        self.metrics = None  # utils.metrics.Metrics, attached by the server
        # KLLM_SCHED_TRACE_LEVEL=1|2: Begin / End events of every step's phases (and, at level 2, of every request)
        # go to sched_events_node_<rank>.csv; ENABLE_PROFILE_EVENT adds NVTX ranges around the same phases
        from ..utils.tracing import ScheduleEventTracer
        self.tracer = ScheduleEventTracer(self.tp.rank, directory=os.environ.get("KLLM_SCHED_TRACE_DIR", "."))
        self._ctl = None  # CPU process group for plan broadcast
        self._ctl_src = 0
        self._hdr = np.zeros(64, dtype=np.int32)
        self.stats = {"generated_tokens": 0, "prompt_tokens": 0, "steps": 0, "forward_time": 0.0, "schedule_time": 0.0,
                      "t_broadcast": 0.0, "t_launch": 0.0, "t_sample_sync": 0.0, "t_apply": 0.0}
        self.on_step: Optional[Callable[[Dict[str, Any]], None]] = None
        self.pipeline = None  # parallel.pipeline.PipelineStage when the model is split over stages
        # asynchronous scheduling (setting.batch_scheduler.enable_async): step N + 1 is planned and launched while
        # step N still runs; its tokens reach the host one step late
        self.async_mode = bool(bs_cfg.enable_async) and not self.mtp_steps and not self.trie_drafts and \
            not self.ptp_steps
        self._inflight = None       # (plan, token handle) of the step whose tokens are not on the host yet
        self._complex_requests = 0  # live requests that need per-token host state (grammar, beams, penalties, ...)
        self.dp = None              # parallel.attn_dp.DPCoordinator under attention data parallelism
        self.adp_balance = None     # parallel.attn_dp.ADPBalance (attention_dp_lb_config.enable_balance)
        self._check_blocks = bool(getattr(bm_cfg, "enable_block_checksum", False))
        self._status_every = int(os.environ.get("KSANA_STATUS_CHECK_STEPS", "64"))  # 0: never read the status word
        # A step that took longer than this is suspected of having sat in a bounded peer wait (8 s in the kernels):
        # the status word is then read right away instead of at the next periodic check. Kept below the kernels' bound
        # and far below the heartbeat timeout, so a lost peer is reported by whichever notices first.
        self._slow_step_s = float(os.environ.get("KSANA_STATUS_SLOW_STEP_S", "4"))
        self._last_apply = time.perf_counter()
        # set when the device status word was found non-zero: what the kernels of recent steps produced is not to be
        # trusted. A multi-rank instance then refuses new requests (its ranks no longer agree on what they computed).
        self.device_fault: Optional[str] = None
        self.before_forward = None  # optional hook(plan), called on the step thread right before a forward pass
        # optional hook(plan), called before a step's results reach the scheduler, i.e. before any sequence of the
        # plan can finish and release its cache blocks
        self.before_resolve = None
        self._ctl_ops: List[Tuple[Dict[str, Any], threading.Event]] = []  # control messages for the follower ranks
        self.on_control: Optional[Callable[[Dict[str, Any]], None]] = None   # follower side: handler of such messages
        self.dp_router = None       # parallel.attn_dp.DPRequestRouter on the rank that owns the HTTP front-end
        self.dp_worker = None       # parallel.attn_dp.DPRequestWorker on the other DP ranks
        self._dp_arrivals = 0
        self.dp_any_work = True

    @staticmethod
    def _flexible_cache_min(bs_cfg, model, kv_dtype) -> int:
        """setting.batch_scheduler.min_flexible_cache_num when the model's cached keys can be moved to another
        position by a rotation (or do not depend on the position at all) and the cache keeps the model's own dtype;
        0 (off) otherwise."""
        want = int(getattr(bs_cfg, "min_flexible_cache_num", 0) or 0)
        cfg = model.cfg
        if want <= 0 or not bs_cfg.enable_auto_prefix_cache:
            return 0
        movable = (cfg.position_encoding in ("rope", "alibi") and not cfg.qk_norm_after_rope and not cfg.qk_l2_norm
                   and not cfg.rope_layers and not cfg.rope_scaling.mrope_section and not cfg.index_topk
                   and not cfg.cla_share_factor)
        return want if movable and kv_dtype is None else 0

    # ---- sizing ----------------------------------------------------------------------------------------
    def _derive_num_blocks(self, kv_dtype) -> int:
        bm = self.serving.setting.block_manager
        per_block = self.model.kv_block_bytes(self.block_size, kv_dtype)
        if self.model.device.type == "cuda":
            free, total = torch.cuda.mem_get_info(self.model.device)
            budget = free - int(total * bm.reserved_device_memory_ratio) - (8 << 30)
            if bm.block_device_memory_ratio > 0:
                budget = min(budget, int(total * bm.block_device_memory_ratio))
            n = max(int(budget // per_block), 16)
        else:
            n = 512
        # every rank that shares block tables must own the same number of blocks: the smallest offer wins
        # (tensor-parallel peers; pipeline stages hold different layers, so their offers differ too)
        for grp in ([self.tp.group] if self.tp.size > 1 else []) + \
                ([self._block_sync_group] if self._block_sync_group is not None else []):
            t = torch.tensor([n], dtype=torch.int64, device=self.model.device)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=grp)
            n = int(t.item())
        cap = self.serving.setting.batch_scheduler
        need = (cap.max_token_len // self.block_size + 2) * max(cap.max_batch_size, 1) * 4
        return int(min(n, max(need, 64)))

    def _host_block_cap(self, kv_dtype) -> int:
        per_block = self.model.kv_block_bytes(self.block_size, kv_dtype)
        return max(int((8 << 30) // max(per_block, 1)), 0)

    # ---- request intake --------------------------------------------------------------------------------
    def add_request(self, prompt_tokens: Sequence[int], params: Optional[SamplingParams] = None,
                    refit=None, grammar=None, probe=None, mrope_positions=None, local: bool = False) -> Request:
        """``mrope_positions``: [3, prompt_len] (temporal, height, width) positions of the prompt tokens for models
        with multimodal RoPE; generated tokens continue from max + 1 on all three axes. Under served attention data
        parallelism the request may be placed on another DP rank (``local`` forces this rank)."""
        params = params or SamplingParams()
        params.verify()
        if self.refusing_requests():
            raise EngineError(_host.FINISH_ERROR, f"this instance no longer accepts requests: {self.device_fault}")
        now = time.time()
        req = Request(next(self._ids), list(int(t) for t in prompt_tokens), params, now)
        req.refit, req.grammar, req.probe = refit, grammar, probe
        if self.dp_router is not None and not local:
            weight = len(req.prompt_tokens) + params.max_new_tokens
            plain = (refit is None and grammar is None and probe is None and mrope_positions is None and
                     max(params.num_beams, params.num_return_sequences, 1) == 1 and not params.logprobs and
                     not self._needs_host_tokens(params, req))
            rank = self.dp_router.place(weight) if plain else 0
            if not plain:
                self.dp_router.load[0] += weight
            req.dp_weight = weight
            if rank != 0:
                # runs in another rank's engine; its progress is mirrored into this object by the router's reader
                if len(req.prompt_tokens) >= self.sched_cfg.max_token_len:
                    self.dp_router.release(rank, weight)
                    raise EngineError(_host.RET_INPUT_LENGTH_EXCEEDED, "input length exceeds max_token_len")
                req.seqs.append(SequenceOutput(-req.req_id))
                self.stats["prompt_tokens"] += len(req.prompt_tokens)
                self.dp_router.submit(rank, req, weight)
                return req
        if mrope_positions is not None:
            axes = self._rope_axes()
            mp = torch.as_tensor(mrope_positions, dtype=torch.int32).reshape(axes, -1)
            if mp.shape[1] != len(req.prompt_tokens):
                raise EngineError(_host.RET_INVALID_ARGUMENT, f"mrope_positions must be [{axes}, prompt_len]")
            req.mrope = mp
            req.mrope_delta = int(mp.max()) + 1 - mp.shape[1] if mp.numel() else 0
        n_out = max(params.num_beams, params.num_return_sequences, 1)
        if params.num_beams > 1:
            import dataclasses
            from .beam_search import BeamState
            req.beam = BeamState(params.num_beams, params.num_return_sequences, params.length_penalty,
                                 params.max_new_tokens)
            req.row_params = dataclasses.replace(params, topk=1, do_sample=False, num_beams=1,
                                                 logprobs=max(params.logprobs, 2 * params.num_beams))
        with self.lock:
            first = self._enqueue_seq(req, req.prompt_tokens)
            req._pending_fanout = n_out - 1 if params.num_beams <= 1 else 0
            self.requests[req.req_id] = req
            req._complex = self._needs_host_tokens(params, req) or n_out > 1 or mrope_positions is not None
            self._complex_requests += 1 if req._complex else 0
            self.stats["prompt_tokens"] += len(req.prompt_tokens)
        self._wake.set()
        return req

    def _enqueue_seq(self, req: Request, tokens: List[int]) -> SequenceOutput:
        sid = next(self._seq_ids)
        self._dp_arrivals += 1
        p = req.params
        eos = list(self.cfg.eos_token_ids)
        # spliced embeddings (images): equal token ids no longer mean equal KV, so the prefix tree is bypassed
        no_cache = req.refit is not None
        if req.beam is not None:
            # the beam state applies EOS / length rules itself (a finished hypothesis is not a finished request)
            code = self.sched.enqueue(sid, tokens, p.max_new_tokens + 1, True, [], [], int(req.arrival * 1000),
                                      req.req_id, no_cache)
        else:
            code = self.sched.enqueue(sid, tokens, p.max_new_tokens, p.ignore_eos, eos, list(p.stop_token_ids),
                                      int(req.arrival * 1000), req.req_id, no_cache)
        if code != _host.RET_SUCCESS:
            msg = {_host.RET_EXCEED_CAPACITY: "waiting queue is full",
                   _host.RET_INPUT_LENGTH_EXCEEDED: "input length exceeds max_token_len",
                   _host.RET_OUT_OF_MEMORY: "request can never fit in the KV cache",
                   _host.RET_INVALID_ARGUMENT: "invalid request"}.get(code, "rejected")
            raise EngineError(code, msg)
        so = SequenceOutput(sid)
        req.seqs.append(so)
        self.seq_owner[sid] = (req, so)
        if p.seed is not None:
            g = torch.Generator(device=self.runner.device)
            g.manual_seed(p.seed + len(req.seqs) - 1)
            req.generators[sid] = g
        if self.trie_drafts:
            trie = _host.DraftTrie()
            trie.feed(tokens)
            req.tries[sid] = trie
        return so

    def _fork_seq(self, req: Request, parent_sid: int) -> Optional[SequenceOutput]:
        """Copy-on-write fork of a running sequence (beam search)."""
        import copy
        child_id = next(self._seq_ids)
        if not self.sched.fork(parent_sid, child_id):
            return None
        parent = self.seq_owner[parent_sid][1]
        so = SequenceOutput(child_id, list(parent.output_tokens), copy.copy(parent.logprobs))
        so.cum_logprob = parent.cum_logprob
        req.seqs.append(so)
        self.seq_owner[child_id] = (req, so)
        return so

    def abort(self, req: Request) -> None:
        if getattr(req, "dp_remote", None) is not None:
            self.dp_router.abort(req)
            return
        with self.lock:
            req.aborted = True
            for s in req.seqs:
                if not s.finished:
                    self.sched.abort(s.seq_id)
        self._wake.set()

    def has_unfinished(self) -> bool:
        return (self.sched.has_unfinished() or self._inflight is not None or
                any(x is not None for x in getattr(self, "_mb_inflight", ())))

    # ---- one step ----------------------------------------------------------------------------------------
    def refusing_requests(self) -> bool:
        """True once a device fault was seen on an instance of several ranks."""
        return self.device_fault is not None and (self.tp.size > 1 or self.pipeline is not None or self.dp is not None)

    def step(self) -> int:
        """Schedules and runs one step. Returns the number of tokens generated."""
        if self._ctl_ops:
            self._flush_control_ops()
        if self.pipeline is not None and getattr(self, "pp_micro_batches", 1) > 1 and self.is_driver:
            return self._step_pipelined()
        if self.async_mode and self.is_driver:
            if self._complex_requests == 0 and (self.pipeline is None or self.pipeline.topo.num_stages == 1):
                return self._step_async()
            drained = self._drain_inflight()
            return drained + self._step_sync()
        return self._step_sync()

    @contextlib.contextmanager
    def _phase(self, name: str, batch: int = 0, tokens: int = 0):
        """One phase of a step for the tracers (no cost when both are off)."""
        if not self.tracer.enabled and not _tracing._NVTX:
            yield
            return
        with _tracing.profile_scope(name), self.tracer.span(name, self.step_count, batch, tokens):
            yield

    def _step_sync(self) -> int:
        t0 = time.perf_counter()
        self.tracer.record("Schedule", "B", self.step_count)
        with self.lock:
            if self.adp_balance is not None:
                arrivals, self._dp_arrivals = self._dp_arrivals, 0
                allow = self.adp_balance.decide(self.sched.num_waiting, self.sched.num_running, arrivals)
                self.sched.set_hold_waiting(not allow)
            plan = self.sched.schedule(int(time.time() * 1000))
            for sid, reason in plan.dropped:
                self._finish_seq(sid, reason)
            layout = rows = refit = mrope = None
            greedy = True
            if not plan.empty():
                layout = self.sched.pack(plan, self.runner.staging.host_np, self.runner.max_blocks_per_seq)
                rows, greedy, refit = self._sample_rows(plan)
                mrope = self._build_mrope(plan)
            dp_group = self.dp is not None and self._has_followers()
            if dp_group:
                # a DP group with tensor parallelism inside: its followers hear about EVERY step, also the empty
                # ones, because the per-step agreement below and the mock steps are collectives they take part in
                self._broadcast_plan(layout, plan, greedy, refit=refit, mrope=mrope, noplan=plan.empty())
            if self.dp is not None:
                # attention data parallelism: all ranks step together; a rank without work runs a mock step
                stride, anybody = self.dp.sync(plan.total_tokens, self.sched.has_unfinished())
                self.dp_any_work = anybody
                if self.tp.ep is not None:
                    self.tp.ep.step_stride = max(stride, 1)
                if plan.empty():
                    if stride > 0:
                        self.runner.mock_forward(bool(self.mtp_steps))
                        self._mtp_idle_passes(self.mtp_steps - 1)
                        self.stats["mock_steps"] = self.stats.get("mock_steps", 0) + 1
                    self.tracer.record("Schedule", "E", self.step_count)
                    return 0
            if plan.empty():
                self.tracer.record("Schedule", "E", self.step_count)
                return 0
        t1 = time.perf_counter()
        nb, nt = len(plan.entries), plan.total_tokens
        self.tracer.record("Schedule", "E", self.step_count, -1, nb, nt)
        if self.tracer.level >= 2:
            for e in plan.entries:
                self.tracer.record("ForwardRequest", "B", self.step_count, e.seq_id, 1, e.q_len, level=2)
        if self._has_followers() and not dp_group:
            with self._phase("BroadcastPlan", nb, nt):
                self._broadcast_plan(layout, plan, greedy, refit=refit, mrope=mrope)
        ta = time.perf_counter()
        with self._phase("PrepareForwarding", nb, nt):
            self.runner.apply_flexible(plan.flexible)
            self.runner.apply_block_ops(plan.swap_out, plan.swap_in, plan.block_copies)
            meta = self.runner.upload(layout)
            if mrope is not None:
                meta.mrope_positions = mrope.to(self.runner.device)
        guard = self._checksum_guard(plan) if self._check_blocks else None
        if self.pipeline is not None and self.pipeline.topo.num_stages > 1:
            with self._phase("ForwardingLayers", nb, nt):
                out, hidden = self._pipeline_step_driver(meta, refit, rows, greedy)
            tb = time.perf_counter()
        else:
            with self._phase("ForwardingLayers", nb, nt):
                if self.before_forward is not None:
                    self.before_forward(plan)  # prefill / decode disaggregation: KV leaves layer by layer
                hidden = self.runner.forward(meta, refit)
                self._run_probes(plan, meta, hidden)
            tb = time.perf_counter()
            with self._phase("LmHeadSampling", nb, nt):
                out = self.runner.sample(hidden, meta, rows, greedy)
        if guard is not None:
            self._checksum_verify(guard)
        t2 = time.perf_counter()
        with self.lock, self._phase("UpdateResults", nb, nt):
            n_new = self._apply_results(plan, out, meta, hidden)
        if self.tracer.level >= 2:
            for e in plan.entries:
                self.tracer.record("ForwardRequest", "E", self.step_count, e.seq_id, 1, e.q_len, level=2)
        t3 = time.perf_counter()
        self.step_count += 1
        st = self.stats
        st["steps"] += 1
        st["schedule_time"] += t1 - t0
        st["forward_time"] += t2 - t1
        # host-side phase clocks (seconds, cumulative): where a step's wall time goes on the driving rank
        st["t_broadcast"] += ta - t1
        st["t_launch"] += tb - ta
        st["t_sample_sync"] += t2 - tb
        st["t_apply"] += t3 - t2
        if self.on_step is not None:
            self.on_step({"tokens": meta.total_tokens, "seqs": meta.num_seqs, "new_tokens": n_new,
                          "schedule_s": t1 - t0, "forward_s": t2 - t1, "prefill": meta.num_prefill,
                          "decode": meta.num_decode})
        return n_new

    # ---- asynchronous scheduling ---------------------------------------------------------------------------------
    @staticmethod
    def _needs_host_tokens(params, req) -> bool:
        """True when sampling this request depends on host-side per-token state, which lags one step in async mode."""
        p = params
        greedy = p.do_sample is False or p.topk == 1
        return (not greedy or p.logprobs > 0 or p.repetition_penalty != 1.0 or p.no_repeat_ngram_size > 0 or
                p.encoder_no_repeat_ngram_size > 0 or p.decoder_no_repeat_ngram_size > 0 or p.num_beams > 1 or
                p.presence_penalty != 0.0 or p.frequency_penalty != 0.0 or bool(p.logit_bias) or p.min_tokens > 0 or
                bool(p.stop_strings) or req.grammar is not None or req.probe is not None or req.refit is not None)

    def _drain_inflight(self) -> int:
        """Brings the tokens of the in-flight step to the host and applies them."""
        inf, self._inflight = self._inflight, None
        if inf is None:
            return 0
        from .sampler import SampleOutput
        plan, handle = inf
        toks = self.runner.wait_tokens(handle)
        n = len(toks)
        if self.before_resolve is not None:
            self.before_resolve(plan)
        with self.lock:
            results = self.sched.resolve(plan, toks)
            return self._apply_results(plan, SampleOutput(tokens=toks, logprobs=[None] * n, chosen_logprob=[None] * n),
                                       None, None, results=results)

    def _step_async(self) -> int:
        """One step with the host one token behind the device (reference: the async mode of ScheduleProcessor,
        src/ksana_llm/batch_manager/schedule_processor.cpp:118-199, which plans on estimated generation results).
        The plan is built from placeholder tokens; the device substitutes the real ones from the previous step's
        token vector (ModelRunner.fixup_inputs)."""
        t0 = time.perf_counter()
        with self.lock:
            plan = self.sched.schedule(int(time.time() * 1000))
            for sid, reason in plan.dropped:
                self._finish_seq(sid, reason)
            if plan.empty():
                return self._drain_inflight()
            self.runner.staging.flip()
            layout = self.sched.pack(plan, self.runner.staging.host_np, self.runner.max_blocks_per_seq)
        t1 = time.perf_counter()
        fix = self._inflight is not None
        if self._has_followers():
            self._broadcast_plan(layout, plan, True, fixup=fix)
        ta = time.perf_counter()
        nb, nt = len(plan.entries), plan.total_tokens
        with self._phase("LaunchStep", nb, nt):
            self.runner.apply_flexible(plan.flexible)
            self.runner.apply_block_ops(plan.swap_out, plan.swap_in, plan.block_copies)
            meta = self.runner.upload(layout)
            if fix:
                self.runner.fixup_inputs(meta)
            if self.before_forward is not None:
                self.before_forward(plan)  # prefill / decode disaggregation: KV leaves layer by layer
            hidden = self.runner.forward(meta, None)
            handle = self.runner.sample_greedy_async(hidden, meta)
        tb = time.perf_counter()
        with self._phase("ResolvePreviousStep", nb, nt):
            n_new = self._drain_inflight()  # the PREVIOUS step: its tokens were produced before this one started
        t2 = time.perf_counter()
        with self.lock:
            placeholders = [-(1 + i) for i in range(plan.total_logits)]
            self.sched.update(plan, placeholders, int(time.time() * 1000))
        self._inflight = (plan, handle)
        t3 = time.perf_counter()
        self.step_count += 1
        st = self.stats
        st["steps"] += 1
        st["schedule_time"] += t1 - t0
        st["forward_time"] += t2 - t1
        st["t_broadcast"] += ta - t1
        st["t_launch"] += tb - ta
        st["t_sample_sync"] += t2 - tb
        st["t_apply"] += t3 - t2
        return n_new

    def _rope_axes(self) -> int:
        """Position axes per token: 3 for M-RoPE (temporal, height, width), 4 for XD-RoPE."""
        sec = self.runner.model.cfg.rope_scaling.mrope_section
        return 4 if len(sec) == 4 else 3

    def _attach_mrope(self, plan, meta) -> None:
        mp = self._build_mrope(plan)
        if mp is not None:
            meta.mrope_positions = mp.to(self.runner.device)

    def _build_mrope(self, plan) -> Optional[torch.Tensor]:
        """The step's [axes, T] multimodal positions (host tensor) when any scheduled request carries them."""
        if not any(getattr(self.seq_owner[e.seq_id][0], "mrope", None) is not None for e in plan.entries
                   if e.seq_id in self.seq_owner):
            return None
        cols = []
        axes = self._rope_axes()
        for e in plan.entries:
            req = self.seq_owner[e.seq_id][0]
            idx = torch.arange(e.q_start, e.q_start + e.q_len, dtype=torch.int32)
            mp = getattr(req, "mrope", None)
            if mp is None:
                cols.append(idx.unsqueeze(0).expand(axes, -1))
                continue
            P = mp.shape[1]
            inside = idx.clamp(max=max(P - 1, 0)).long()
            cols.append(torch.where(idx.unsqueeze(0) < P, mp[:, inside], (idx + req.mrope_delta).unsqueeze(0).expand(axes, -1)))
        return torch.cat(cols, dim=1).to(torch.int32).contiguous()

    def _sample_rows(self, plan):
        rows: List[SampleRow] = []
        refit = None
        row0 = 0  # first row of the entry in the step's flat token order
        for e in plan.entries:
            req, so = self.seq_owner[e.seq_id]
            if req.refit is not None and e.q_start < len(req.prompt_tokens):
                # the part of every spliced run that falls into this chunk [q_start, q_start + q_len)
                for pos, emb in req.refit:
                    lo, hi = max(pos, e.q_start), min(pos + emb.shape[0], e.q_start + e.q_len)
                    if lo < hi:
                        refit = (refit or []) + [(row0 + lo - e.q_start, emb[lo - pos:hi - pos])]
            row0 += e.q_len
            for j in range(e.num_logits):
                bm = None
                if req.grammar is not None and j == 0:
                    bm = req.grammar.next_bitmask(so.seq_id)
                rows.append(SampleRow(getattr(req, "row_params", req.params), req.prompt_tokens, so.output_tokens, bm,
                                      req.generators.get(e.seq_id)))
        from .sampler import Sampler
        greedy = Sampler.all_greedy(rows)
        return rows, greedy, refit

    def _apply_results(self, plan, out, meta, hidden, results=None) -> int:
        now = time.time()
        sampled = out.tokens
        # beam search rewrites the sampled tokens from the top-2k log-probs before the scheduler sees them
        if results is None:
            if self.before_resolve is not None:
                self.before_resolve(plan)
            results = self.sched.update(plan, sampled, int(now * 1000))
        # reading the status word waits for the device: cheap after a synchronous step (it is idle), but under
        # asynchronous scheduling it would wait for the step in flight, so that path looks 16 times less often
        every = self._status_every * (16 if hidden is None else 1)
        t_now = time.perf_counter()
        slow = self._status_every > 0 and self._slow_step_s > 0 and t_now - self._last_apply > self._slow_step_s
        self._last_apply = t_now
        if slow or (every and self.step_count % every == every - 1):
            try:
                self.runner.check_device_status()
            except RuntimeError as ex:
                self.device_fault = str(ex)
                raise  # the serve loop fails what is in flight
        if self.mtp_steps and hidden is not None and meta is not None:
            self._mtp_propose(plan, meta, hidden, results)
        row = 0
        row_of = {}
        for e in plan.entries:
            row_of[e.seq_id] = row
            row += e.num_logits
        n_new = 0
        touched = set()
        for r in results:
            req, so = self.seq_owner.get(r.seq_id, (None, None))
            if req is None:
                continue
            base = row_of[r.seq_id]
            for j, tok in enumerate(r.new_tokens):
                so.output_tokens.append(int(tok))
                if out.logprobs and out.logprobs[base + j] is not None:
                    so.logprobs.append({"token": int(tok), "logprob": out.chosen_logprob[base + j],
                                        "top": out.logprobs[base + j]})
                    so.cum_logprob += out.chosen_logprob[base + j] or 0.0
                if req.grammar is not None:
                    req.grammar.accept(so.seq_id, int(tok))
                trie = req.tries.get(r.seq_id)
                if trie is not None:
                    trie.feed_one(int(tok))
            n_new += len(r.new_tokens)
            if req.first_token_time is None and r.new_tokens:
                req.first_token_time = now
            req.token_times.extend([now] * len(r.new_tokens))
            reason = r.finish_reason
            if reason == _host.FINISH_NONE and req.params.stop_strings and self.detokenize is not None:
                if self._hit_stop_string(req, so):
                    self.sched.finish(r.seq_id, _host.FINISH_STOP_STRING)
                    reason = _host.FINISH_STOP_STRING
            if reason == _host.FINISH_NONE and req.grammar is not None and req.grammar.is_terminated(so.seq_id):
                self.sched.finish(r.seq_id, _host.FINISH_EOS)
                reason = _host.FINISH_EOS
            if reason != _host.FINISH_NONE:
                self._finish_seq(r.seq_id, reason, notify=False)
            else:
                trie = req.tries.get(r.seq_id)
                if trie is not None and req.grammar is None:
                    d = trie.propose(self.trie_drafts)
                    if d:
                        self.sched.set_drafts(r.seq_id, d)
                if self.ptp_steps and req.grammar is None:
                    self.sched.set_drafts(r.seq_id, [self.ptp_token] * self.ptp_steps)
            # fan-out of parallel samples once the prompt's blocks are cached
            if getattr(req, "_pending_fanout", 0) and r.new_tokens:
                k = req._pending_fanout
                req._pending_fanout = 0
                for _ in range(k):
                    try:
                        self._enqueue_seq(req, req.prompt_tokens)
                    except EngineError as ex:
                        req.error = ex
            touched.add(req.req_id)
        self.stats["generated_tokens"] += n_new
        # ---- beam search: re-rank and fork/prune the beams of every request that advanced ----
        for rid in touched:
            req = self.requests.get(rid)
            if req is None or req.beam is None or req.beam.done:
                continue
            rows = {}
            for r in results:
                owner = self.seq_owner.get(r.seq_id)
                if owner is None or owner[0] is not req or not r.new_tokens:
                    continue
                top = out.logprobs[row_of[r.seq_id]] or []
                rows[r.seq_id] = (list(owner[1].output_tokens[:-1]), top)
            if rows:
                req.beam.step(self, req, rows, set(self.cfg.eos_token_ids) | set(req.params.stop_token_ids))
        for rid in touched:
            req = self.requests.get(rid)
            if req is not None:
                self._check_request_done(req)
                req.notify()
        return n_new

    def _hit_stop_string(self, req: Request, so: SequenceOutput) -> bool:
        window = so.output_tokens[max(0, so.text_checked - 16):]
        text = self.detokenize(window)
        so.text_checked = len(so.output_tokens)
        return any(s and s in text for s in req.params.stop_strings)

    def _finish_seq(self, sid: int, reason: int, notify: bool = True) -> None:
        owner = self.seq_owner.pop(sid, None)
        self.sched.forget(sid)
        if owner is None:
            return
        req, so = owner
        so.finished = True
        so.finish_reason = FINISH_NAMES.get(reason, "stop")
        if reason == _host.FINISH_TIMEOUT and req.error is None:
            req.error = EngineError(_host.RET_REQUEST_TIMEOUT if hasattr(_host, "RET_REQUEST_TIMEOUT") else 4,
                                    "request timed out in queue")
        if notify:
            self._check_request_done(req)
            req.notify()

    def _check_request_done(self, req: Request) -> None:
        if req.finished:
            return
        if all(s.finished for s in req.seqs) and not getattr(req, "_pending_fanout", 0):
            req.finished = True
            req.finish_time = time.time()
            self.requests.pop(req.req_id, None)
            if self.dp_router is not None and getattr(req, "dp_weight", 0):
                self.dp_router.release(0, req.dp_weight)
            if getattr(req, "_complex", False):
                req._complex = False
                self._complex_requests -= 1
            if self.metrics is not None:
                self.metrics.observe_request(req)

    def _checksum_guard(self, plan):
        """setting.block_manager.enable_block_checksum (debug): the blocks that were already full before this step -
        cached prefixes included - must come out of the step unchanged. Checksums of the first and last layer's
        pages are taken before the forward and compared after it (reference: CalculateChecksum, cache_copy.cu:407,
        verification in models/base/model_input.cpp:380-530)."""
        from ..utils.memory_checker import block_checksums
        blocks = set()
        for e in plan.entries:
            table = self.cache.block_table(e.seq_id)
            blocks.update(table[:e.q_start // self.block_size])
        blocks = sorted(blocks)
        if not blocks:
            return None
        layers = sorted({0, len(self.runner.kv_caches) - 1})
        return blocks, layers, [block_checksums(self.runner.kv_caches[l], blocks) for l in layers]

    def _checksum_verify(self, guard) -> None:
        from ..utils.memory_checker import block_checksums
        blocks, layers, before = guard
        for l, b in zip(layers, before):
            now = block_checksums(self.runner.kv_caches[l], blocks)
            bad = [blocks[i] for i in (now != b).nonzero().flatten().tolist()]
            if bad:
                raise RuntimeError(f"KV block checksum changed during step {self.step_count}: layer {l}, blocks {bad[:8]}")

    def _mtp_propose(self, plan, meta, hidden, results) -> None:
        """Multi-token prediction drafts (DeepSeek next-n module): after the main model's step the MTP layer runs
        over the same rows with every row's FOLLOWING token as its second input (the next prompt token, the next fed
        token, or - at a sequence's last accepted row - the token just generated); the arg-max at that row is the
        draft the next step verifies. The layer keeps its own KV pages under the same block tables; rows of rejected
        drafts are written again when their positions are fed again. Reference: LlmRuntime::MtpForward
        (runtime/llm_runtime.cpp:172-240), deepseek_v3_model.cpp:231-288. One draft per step."""
        model = self.model
        mtp = model.mtp_layers[0]
        by_seq = {r.seq_id: r for r in results}
        fix_rows, fix_vals, draft_rows, draft_seqs = [], [], [], []
        row0 = 0
        for e in plan.entries:
            q, real = e.q_len, e.q_len - e.n_drafts
            owner = self.seq_owner.get(e.seq_id)
            r = by_seq.get(e.seq_id)
            if e.num_logits == 0:
                if owner is not None:  # a prompt chunk: what follows it is the next prompt token
                    toks = owner[0].prompt_tokens
                    nxt_pos = e.q_start + q
                    if nxt_pos < len(toks):
                        fix_rows.append(row0 + q - 1)
                        fix_vals.append(int(toks[nxt_pos]))
            elif r is not None and len(r.new_tokens) > r.accepted_drafts:
                last = row0 + real - 1 + r.accepted_drafts
                fix_rows.append(last)
                fix_vals.append(int(r.new_tokens[r.accepted_drafts]))  # the token after the accepted drafts
                # (a grammar-constrained request takes no drafts: only its first logits row carries the token mask)
                if r.finish_reason == _host.FINISH_NONE and (owner is None or owner[0].grammar is None):
                    draft_rows.append(last)
                    draft_seqs.append(e.seq_id)
            row0 += q
        nxt = torch.roll(meta.input_ids, -1)
        if fix_rows:
            nxt[torch.tensor(fix_rows, device=nxt.device)] = torch.tensor(fix_vals, dtype=nxt.dtype, device=nxt.device)
        rows = torch.tensor(draft_rows, dtype=torch.int32, device=nxt.device)
        if self._has_followers():
            # tensor-parallel peers run the same draft pass (its collectives need them): they get the shifted ids
            n = torch.tensor([len(draft_rows)], dtype=torch.int32)
            dist.broadcast(n, src=self._ctl_src, group=self._ctl)
            dist.broadcast(nxt.to("cpu", torch.int32), src=self._ctl_src, group=self._ctl)
            if draft_rows:
                dist.broadcast(rows.cpu(), src=self._ctl_src, group=self._ctl)
        drafts = self._mtp_forward(mtp, nxt, rows, meta, hidden)
        if drafts is None:
            self._mtp_idle_passes(self.mtp_steps - 1)
            return
        chains = [[int(d)] for d in drafts.tolist()]
        if self.mtp_steps > 1:
            # further drafts: the module is applied again at the following positions, fed with its own previous
            # output and the token it just drafted (its cache entries for those positions live in the look-ahead
            # slots the scheduler reserved)
            pos0 = {}
            for e in plan.entries:
                r = by_seq.get(e.seq_id)
                if r is not None:
                    pos0[e.seq_id] = e.q_start + (e.q_len - e.n_drafts) + r.accepted_drafts
            self._mtp_chain(mtp, draft_seqs, [pos0[s_] for s_ in draft_seqs], chains, rows)
        for sid, ch in zip(draft_seqs, chains):
            self.sched.set_drafts(sid, ch)

    @torch.inference_mode()
    def _mtp_chain(self, mtp, seqs, positions, chains, rows) -> None:
        from .. import ops
        from .step_input import make_step_input
        model, bs = self.model, self.block_size
        cache = self.runner.kv_caches[len(model.layers)]
        prev = self._mtp_residual.index_select(0, rows.long())
        tables = [self.cache.block_table(s_) for s_ in seqs]
        n = len(seqs)
        peers = self._has_followers()
        for k in range(1, self.mtp_steps):
            pos = [p + k - 1 for p in positions]
            if any(p // bs >= len(t) for p, t in zip(pos, tables)):
                if peers:
                    dist.broadcast(torch.zeros(2, dtype=torch.int32), src=self._ctl_src, group=self._ctl)
                self._mtp_idle_passes(self.mtp_steps - k)
                return  # no reserved slot (end of the length budget): shorter chains for everybody
            slots = [t[p // bs] * bs + p % bs for p, t in zip(pos, tables)]
            width = max(len(t) for t in tables)
            bt = [list(t) + [0] * (width - len(t)) for t in tables]
            ids = [c[-1] for c in chains]
            if peers:  # the same pass on the tensor-parallel peers: [rows, table width], then ids | pos | slots | tables
                dist.broadcast(torch.tensor([n, width], dtype=torch.int32), src=self._ctl_src, group=self._ctl)
                flat = ids + pos + slots + [b for t in bt for b in t]
                dist.broadcast(torch.tensor(flat, dtype=torch.int32), src=self._ctl_src, group=self._ctl)
            meta = make_step_input(ids, pos, slots, list(range(n + 1)), [p + 1 for p in pos], bt, logits_idx=list(range(n)),
                                   num_prefill=0, device=self.runner.device)
            emb = ops.embedding(meta.input_ids, model.embed, model.cfg.emb_scale)
            h, prev = mtp.forward(emb, prev, meta, cache, return_residual=True)
            nxt = model.greedy_tokens(h, meta.logits_idx).tolist()
            for c, d in zip(chains, nxt):
                c.append(int(d))

    @torch.inference_mode()
    def _mtp_idle_passes(self, n: int) -> None:
        """Attention data parallelism: the other ranks may be running ``n`` more passes of the draft module, each of
        which exchanges tokens with every rank's experts; join them with empty passes."""
        if n <= 0 or self.dp is None or not getattr(self, "_dp_mtp_lockstep", False):
            return
        self.runner.mock_mtp_passes(n)

    @torch.inference_mode()
    def _mtp_forward(self, mtp, nxt, rows, meta, hidden):
        model = self.model
        from .. import ops
        embeds = ops.embedding(nxt, model.embed, model.cfg.emb_scale)
        h, self._mtp_residual = mtp.forward(embeds, hidden, meta, self.runner.kv_caches[len(model.layers)],
                                            return_residual=True)
        if rows.numel() == 0:
            return None
        return model.greedy_tokens(h, rows)

    def _mtp_follow(self, meta, hidden) -> None:
        """Follower half of ``_mtp_propose``."""
        n = torch.zeros(1, dtype=torch.int32)
        dist.broadcast(n, src=self._ctl_src, group=self._ctl)
        nxt = torch.zeros(meta.total_tokens, dtype=torch.int32)
        dist.broadcast(nxt, src=self._ctl_src, group=self._ctl)
        rows = torch.zeros(int(n[0]), dtype=torch.int32)
        if int(n[0]):
            dist.broadcast(rows, src=self._ctl_src, group=self._ctl)
        dev = self.runner.device
        model, mtp = self.model, self.model.mtp_layers[0]
        self._mtp_forward(mtp, nxt.to(dev), rows.to(dev), meta, hidden)
        if self.mtp_steps > 1 and int(n[0]):
            from .. import ops
            from .step_input import make_step_input
            cache = self.runner.kv_caches[len(model.layers)]
            prev = self._mtp_residual.index_select(0, rows.to(dev).long())
            for _ in range(1, self.mtp_steps):
                head = torch.zeros(2, dtype=torch.int32)
                dist.broadcast(head, src=self._ctl_src, group=self._ctl)
                m, width = int(head[0]), int(head[1])
                if m == 0:
                    break
                flat = torch.zeros(m * (3 + width), dtype=torch.int32)
                dist.broadcast(flat, src=self._ctl_src, group=self._ctl)
                flat = flat.tolist()
                ids, pos, slots = flat[:m], flat[m:2 * m], flat[2 * m:3 * m]
                bt = [flat[3 * m + i * width:3 * m + (i + 1) * width] for i in range(m)]
                cm = make_step_input(ids, pos, slots, list(range(m + 1)), [p + 1 for p in pos], bt,
                                     logits_idx=list(range(m)), num_prefill=0, device=dev)
                emb = ops.embedding(cm.input_ids, model.embed, model.cfg.emb_scale)
                h, prev = mtp.forward(emb, prev, cm, cache, return_residual=True)
                model.greedy_tokens(h, cm.logits_idx)

    def _run_probes(self, plan, meta, hidden) -> None:
        for e in plan.entries:
            owner = self.seq_owner.get(e.seq_id)
            if owner is None or owner[0].probe is None:
                continue
            from .forward_probe import run_probe
            b = [x.seq_id for x in plan.entries].index(e.seq_id)
            lo, hi = int(meta.cu_q_host[b]), int(meta.cu_q_host[b + 1])
            prenorm = self.model.last_residual[lo:hi]

            def cutoff_forward(depth, seq_id=e.seq_id, n=hi - lo, toks=owner[0].prompt_tokens):
                # a layer-wise reranker head reads the stack after `depth` layers: one more pass over this request's
                # rows only (its cache pages receive the same values again)
                from .step_input import make_step_input
                table = self.cache.block_table(seq_id)
                bs = self.block_size
                slots = [table[p // bs] * bs + p % bs for p in range(n)]
                m1 = make_step_input(list(toks[:n]), list(range(n)), slots, [0, n], [n], [table],
                                     device=self.runner.device)
                return self.model.forward(m1, self.runner.kv_caches, cutoff_layer=depth)

            owner[0].probe_result = run_probe(self.model, owner[0].probe, hidden[lo:hi], prenorm,
                                              owner[0].prompt_tokens, cutoff_forward)

    # ---- multi-rank plan distribution ---------------------------------------------------------------------
    def attach_control_group(self, group, src: int = 0) -> None:
        """``group``: CPU process group over which the driving rank broadcasts its step plans; ``src``: that rank's
        GLOBAL rank (not 0 for the DP groups after the first)."""
        self._ctl = group
        self._ctl_src = src

    def post_control(self, msg: Dict[str, Any], wait: float = 60.0) -> bool:
        """Queues a control message for the follower ranks; it travels in the same ordered stream as the step plans
        (sent at the start of the next step, before that step is scheduled). Returns once it has been sent."""
        return self.enqueue_control(msg).wait(wait)

    def enqueue_control(self, msg: Dict[str, Any]) -> threading.Event:
        """The non-waiting half of ``post_control``: callers that hold the engine lock (so that no step can be
        scheduled between their change and the message) enqueue here and wait on the event after releasing it."""
        ev = threading.Event()
        if not self._has_followers():
            ev.set()
            return ev
        with self.lock:
            self._ctl_ops.append((msg, ev))
        self._wake.set()
        return ev

    def _flush_control_ops(self) -> None:
        with self.lock:
            ops, self._ctl_ops = self._ctl_ops, []
        for msg, ev in ops:
            data = np.frombuffer(json.dumps(msg).encode(), dtype=np.uint8).copy()
            h = self._hdr
            h[:] = 0
            h[0], h[1] = 4, len(data)
            dist.broadcast(torch.from_numpy(h), src=self._ctl_src, group=self._ctl)
            dist.broadcast(torch.from_numpy(data), src=self._ctl_src, group=self._ctl)
            ev.set()

    def _has_followers(self) -> bool:
        """Other ranks execute this engine's plans: tensor-parallel peers and / or later pipeline stages."""
        return self.tp.size > 1 or (self.pipeline is not None and self.pipeline.topo.num_stages > 1)

    def _broadcast_plan(self, layout, plan, greedy: bool, stop: bool = False, fixup: bool = False, refit=None,
                        mrope=None, noplan: bool = False) -> None:
        keys = ["num_seqs", "num_prefill", "num_decode", "total_tokens", "total_logits", "max_q_len", "max_kv_len",
                "max_blocks", "input_ids", "positions", "slot_mapping", "seq_of_token", "cu_q", "kv_lens", "q_starts",
                "logits_idx", "block_tables", "total_words"]
        h = self._hdr
        h[:] = 0
        h[0] = 2 if stop else (3 if noplan else 1)
        if not stop and not noplan:
            for i, k in enumerate(keys):
                h[1 + i] = layout[k]
            h[30] = 1 if greedy else 0
            h[34] = 1 if fixup else 0
            so, si, bc = plan.swap_out, plan.swap_in, plan.block_copies
            fx = np.asarray(plan.flexible, dtype=np.int32).reshape(-1, 2)  # [n, 4] travels as 2n pairs
            h[31], h[32], h[33], h[35] = len(so), len(si), len(bc), len(fx)
            h[36] = len(refit) if refit else 0
            h[37] = sum(int(e.shape[0]) for _, e in refit) if refit else 0
            h[38] = int(mrope.shape[0]) if mrope is not None else 0
        hdr = torch.from_numpy(h)
        dist.broadcast(hdr, src=self._ctl_src, group=self._ctl)
        if stop or noplan:
            return
        n = int(h[18])
        dist.broadcast(self.runner.staging.host[:n], src=self._ctl_src, group=self._ctl)
        extra = int(h[31] + h[32] + h[33] + h[35])
        if extra:
            arr = np.concatenate([np.asarray(a, dtype=np.int32).reshape(-1, 2) for a in (so, si, bc, fx)], 0)
            dist.broadcast(torch.from_numpy(np.ascontiguousarray(arr)), src=self._ctl_src, group=self._ctl)
        if refit:
            # multimodal: (first row, row count) of every spliced run, then all embedding rows
            runs = torch.tensor([[p, e.shape[0]] for p, e in refit], dtype=torch.int32)
            dist.broadcast(runs, src=self._ctl_src, group=self._ctl)
            dist.broadcast(torch.cat([e.float().cpu() for _, e in refit]).contiguous(), src=self._ctl_src, group=self._ctl)
        if mrope is not None:
            dist.broadcast(mrope, src=self._ctl_src, group=self._ctl)

    def follow(self) -> None:
        """Step loop of a non-driver rank: receive plan, run the shard, join the collectives."""
        keys = ["num_seqs", "num_prefill", "num_decode", "total_tokens", "total_logits", "max_q_len", "max_kv_len",
                "max_blocks", "input_ids", "positions", "slot_mapping", "seq_of_token", "cu_q", "kv_lens", "q_starts",
                "logits_idx", "block_tables", "total_words"]
        hdr = torch.zeros(64, dtype=torch.int32)
        while True:
            dist.broadcast(hdr, src=self._ctl_src, group=self._ctl)
            h = hdr.numpy()
            if h[0] == 2:
                return
            if h[0] == 4:
                data = torch.zeros(int(h[1]), dtype=torch.uint8)
                dist.broadcast(data, src=self._ctl_src, group=self._ctl)
                if self.on_control is not None:
                    self.on_control(json.loads(bytes(data.numpy())))
                continue
            if h[0] == 3:
                # a DP group's step without a plan: still agree with the other groups, run a mock step if they work
                stride, _ = self.dp.sync(0, False)
                if self.tp.ep is not None:
                    self.tp.ep.step_stride = max(stride, 1)
                if stride > 0:
                    self.runner.mock_forward(bool(self.mtp_steps))
                if self.dp.stopping:
                    return
                continue
            layout = {k: int(h[1 + i]) for i, k in enumerate(keys)}
            n = layout["total_words"]
            self.runner.staging.flip()  # the previous step's host-to-device copy may still be pending
            dist.broadcast(self.runner.staging.host[:n], src=self._ctl_src, group=self._ctl)
            nso, nsi, nbc, nfx = int(h[31]), int(h[32]), int(h[33]), int(h[35])
            so = si = bc = fx = np.zeros((0, 2), dtype=np.int32)
            if nso + nsi + nbc + nfx:
                arr = torch.zeros(nso + nsi + nbc + nfx, 2, dtype=torch.int32)
                dist.broadcast(arr, src=self._ctl_src, group=self._ctl)
                a = arr.numpy()
                so, si, bc, fx = a[:nso], a[nso:nso + nsi], a[nso + nsi:nso + nsi + nbc], a[nso + nsi + nbc:]
            refit = None
            if h[36]:
                runs = torch.zeros(int(h[36]), 2, dtype=torch.int32)
                dist.broadcast(runs, src=self._ctl_src, group=self._ctl)
                vals = torch.zeros(int(h[37]), self.cfg.hidden_size, dtype=torch.float32)
                dist.broadcast(vals, src=self._ctl_src, group=self._ctl)
                refit, at = [], 0
                for p, n in runs.tolist():
                    refit.append((p, vals[at:at + n].to(self.runner.device)))
                    at += n
            mrope = None
            if h[38]:
                mrope = torch.zeros(int(h[38]), layout["total_tokens"], dtype=torch.int32)
                dist.broadcast(mrope, src=self._ctl_src, group=self._ctl)
            if self.dp is not None:
                stride, _ = self.dp.sync(layout["total_tokens"], True)
                if self.tp.ep is not None:
                    self.tp.ep.step_stride = max(stride, 1)
            self.runner.apply_flexible(fx.reshape(-1, 4))
            self.runner.apply_block_ops(so, si, bc)
            meta = self.runner.upload(layout)
            if mrope is not None:
                meta.mrope_positions = mrope.to(self.runner.device)
            if h[34]:
                self.runner.fixup_inputs(meta)
            if self.pipeline is not None and self.pipeline.topo.num_stages > 1:
                self._pipeline_step_follower(meta, bool(h[30]))
                continue
            hidden = self.runner.forward(meta, refit)
            self.runner.sample(hidden, meta, None, bool(h[30]))
            if self.mtp_steps:
                self._mtp_follow(meta, hidden)
            if self.dp is not None and self.dp.stopping:
                return

    # ---- attention data parallelism ------------------------------------------------------------------------------
    def attach_dp(self, coordinator, balance_coordinator=None) -> None:
        """This engine is one DP rank: its own requests, scheduler and KV cache; MoE blocks exchange tokens with the
        other ranks, so every rank steps in lock-step (``run_dp``). ``balance_coordinator``: for DP groups with tensor
        parallelism inside, a coordinator over the groups' leaders only (None on followers): the prefill balancer's
        per-step agreement is between the ranks that schedule."""
        self.dp = coordinator
        self.async_mode = False
        self.tp.ep_dp = True
        # Every pass of the draft module goes through the experts' exchange, which needs every DP rank: single-rank DP
        # groups all run the same number of passes per step (a rank without drafts joins with empty passes, see
        # _mtp_idle_passes); with tensor parallelism inside the groups the followers' protocol carries one draft
        self._dp_mtp_lockstep = self.tp.size == 1
        if not self._dp_mtp_lockstep:
            self.mtp_steps = min(self.mtp_steps, 1)
        lb = self.serving.setting.batch_scheduler.attention_dp_lb_config
        bc = coordinator if self.tp.size == 1 else balance_coordinator
        if lb.enable_balance and bc is not None:
            from ..parallel.attn_dp import ADPBalance
            self.adp_balance = ADPBalance(bc, lb.max_waiting_steps, lb.max_waiting_time_in_ms, lb.min_qps_for_waiting)

    def run_dp(self, max_steps: int = 1 << 30) -> int:
        """Steps until NO rank has unfinished work (a rank whose own requests are done keeps running mock steps)."""
        steps = 0
        while steps < max_steps:
            self._step_sync()
            steps += 1
            if not self.dp_any_work:
                break
        return steps

    # ---- pipeline parallelism ---------------------------------------------------------------------------------
    def attach_pipeline(self, stage, micro_batches: int = 1) -> None:
        """``stage``: parallel.pipeline.PipelineStage of this rank. The driver is rank 0 (first stage); the last
        stage computes the tokens and returns them to the driver. With ``micro_batches`` > 1 the driver keeps that
        many disjoint groups of sequences in flight: while a later stage works on one group the first stage already
        runs the next (reference: pp_multibatch + MultiBatchController)."""
        from ..parallel.pipeline import MultiBatchController
        self.pipeline = stage
        self.is_driver = stage.topo.rank == 0
        self.async_mode = False
        self.pp_micro_batches = max(int(micro_batches), 1) if stage.topo.num_stages > 1 else 1
        self.mbc = MultiBatchController(self.pp_micro_batches)
        self._mb_inflight = [None] * self.pp_micro_batches
        self._mb_next = 0

    def _collect_micro_batch(self, mb: int) -> int:
        from .sampler import SampleOutput
        plan, n, rows, greedy = self._mb_inflight[mb]
        self._mb_inflight[mb] = None
        pl = self.pipeline
        last = pl.topo.num_stages * pl.topo.tp_size - pl.topo.tp_size
        out = SampleOutput(tokens=[], logprobs=[], chosen_logprob=[])
        if n and greedy:
            toks = pl.channel.recv_tokens(n, last).to("cpu").tolist()
            self.runner.d2h_bytes += 4 * n
            out = SampleOutput(tokens=toks, logprobs=[None] * n, chosen_logprob=[None] * n)
        elif n:
            out = self.runner.sampler.sample(pl.channel.recv_logits(n, self.cfg.vocab_size, last), rows)
        with self.lock:
            got = self._apply_results(plan, out, None, None)
        self.mbc.collected(mb)
        return got

    def _step_pipelined(self) -> int:
        """One driver step with several pipeline micro-batches: collect the oldest in-flight step of this
        micro-batch (its tokens come back from the last stage), then schedule and launch its next step."""
        mb = self._mb_next
        self._mb_next = (mb + 1) % self.pp_micro_batches
        n_new = 0
        if self._mb_inflight[mb] is not None:
            n_new += self._collect_micro_batch(mb)
        with self.lock:
            self.sched.set_micro_batch(mb, self.pp_micro_batches)
            plan = self.sched.schedule(int(time.time() * 1000))
            self.sched.set_micro_batch(-1)
            for sid, reason in plan.dropped:
                self._finish_seq(sid, reason)
            if plan.empty():
                return n_new
            self.runner.staging.flip()
            layout = self.sched.pack(plan, self.runner.staging.host_np, self.runner.max_blocks_per_seq)
            rows, greedy, refit = self._sample_rows(plan)
        self._broadcast_plan(layout, plan, greedy)
        self.runner.apply_flexible(plan.flexible)
        self.runner.apply_block_ops(plan.swap_out, plan.swap_in, plan.block_copies)
        meta = self.runner.upload(layout)
        self.mbc.ready(mb)
        self.mbc.start(mb)
        self.pipeline.run(meta, self.runner.kv_caches, refit)  # first stage: forward + send, returns None
        self.mbc.done(mb)  # this stage is free for the next micro-batch; the results are still travelling
        self._mb_inflight[mb] = (plan, meta.total_logits, rows, greedy)
        self.step_count += 1
        self.stats["steps"] += 1
        return n_new

    def _pipeline_step_driver(self, meta, refit, rows, greedy):
        from .sampler import SampleOutput
        pl = self.pipeline
        hidden = pl.run(meta, self.runner.kv_caches, refit)
        n = meta.total_logits
        if n == 0:
            return SampleOutput(tokens=[]), hidden
        last = pl.topo.num_stages * pl.topo.tp_size - pl.topo.tp_size
        if not greedy:
            # sampling state lives here, the logits on the last stage: it returns the rows' logits
            logits = self.model.compute_logits(hidden, meta.logits_idx) if pl.topo.is_last else \
                pl.channel.recv_logits(n, self.cfg.vocab_size, last)
            return self.runner.sampler.sample(logits, rows), hidden
        if pl.topo.is_last:
            toks = self.model.greedy_tokens(hidden, meta.logits_idx)
        else:
            toks = pl.channel.recv_tokens(n, last)
        host = toks.to("cpu").tolist()
        self.runner.d2h_bytes += 4 * n
        return SampleOutput(tokens=host, logprobs=[None] * n, chosen_logprob=[None] * n), hidden

    def _pipeline_step_follower(self, meta, greedy: bool = True) -> None:
        pl = self.pipeline
        hidden = pl.run(meta, self.runner.kv_caches)
        if pl.topo.is_last and meta.total_logits:
            if greedy:
                toks = self.model.greedy_tokens(hidden, meta.logits_idx)
                if pl.topo.tp_rank == 0:
                    pl.channel.send_tokens(toks, 0)
            else:
                logits = self.model.compute_logits(hidden, meta.logits_idx)
                if pl.topo.tp_rank == 0:
                    pl.channel.send_logits(logits, 0)

    def shutdown_followers(self) -> None:
        if self._has_followers() and self.is_driver and self._ctl is not None:
            self._broadcast_plan(None, None, True, stop=True)

    # ---- loops ----------------------------------------------------------------------------------------------
    def run_until_done(self, max_steps: Optional[int] = None) -> int:
        steps = 0
        while self.has_unfinished():
            self.step()
            steps += 1
            if max_steps is not None and steps >= max_steps:
                break
        return steps

    def warmup(self, max_len: int = 2048, step: int = 64, new_tokens: int = 2) -> int:
        """Runs throw-away requests of 64, 128, ... tokens (2 new tokens each) so that every lazily initialised piece
        (kernel modules, tensor-map and workspace set-up, allocator pools, collective buffers) is paid for before
        the first user request, then drops the cached blocks they left behind. The driving rank calls this; the
        followers are already in ``follow``. Reference: InferenceEngine::DoWarmupRun
        (src/ksana_llm/service/inference_engine.cpp:447-506)."""
        limit = min(max_len, self.sched_cfg.max_token_len - new_tokens - 1, self.sched_cfg.max_step_tokens)
        lens = list(range(step, limit + 1, step)) or [max(limit, 1)]
        vocab = max(self.cfg.vocab_size, 8)
        done = 0
        for n in lens:
            prompt = [3 + (7 * i + n) % (vocab - 4) for i in range(n)]
            req = self.add_request(prompt, SamplingParams(topk=1, max_new_tokens=new_tokens, ignore_eos=True))
            while not req.finished and self.has_unfinished():
                self.step()
            done += 1
        self._drain_inflight()
        with self.lock:
            self.cache.clear_unreferenced()
        for k in ("generated_tokens", "prompt_tokens", "steps"):
            self.stats[k] = 0
        return done

    def start(self) -> None:
        """Background step loop (serving mode)."""
        if self._loop_thread is not None:
            return
        self._stop.clear()

        def loop():
            if self.dp is not None:
                self.serve_dp()
                return
            while not self._stop.is_set():
                if self._ctl_ops and not self.has_unfinished():
                    self._flush_control_ops()
                if self.has_unfinished():
                    try:
                        self.step()
                    except Exception as ex:  # fail in-flight requests, keep serving
                        self._fail_all(ex)
                else:
                    self._wake.wait(0.05)
                    self._wake.clear()

        self._loop_thread = threading.Thread(target=loop, name="ksana-step-loop", daemon=True)
        self._loop_thread.start()

    def serve_dp(self) -> None:
        """Step loop of a served attention-DP rank: all ranks step together for as long as the instance lives (the
        MoE exchange and the per-step agreement are collectives), idling briefly when nobody has work; a shutdown
        requested on any rank reaches all of them in the same step."""
        while True:
            try:
                self._step_sync()
            except Exception as ex:
                self._fail_all(ex)
            if self.dp_worker is not None:
                self.dp_worker.report()
            if self.dp.stopping:
                return
            if not self.dp_any_work:
                time.sleep(0.002)

    def stop(self) -> None:
        self._stop.set()
        self._wake.set()
        if self.dp is not None:
            self.dp.stop_requested = True
        if self._loop_thread is not None:
            self._loop_thread.join(timeout=10)
            self._loop_thread = None
        if self.dp_router is not None:
            self.dp_router.close()
        if self.dp is None:  # a DP group's followers leave with the agreed stop, nobody listens any more
            self.shutdown_followers()

    def _fail_all(self, ex: Exception) -> None:
        with self.lock:
            for req in list(self.requests.values()):
                req.error = EngineError(_host.FINISH_ERROR, f"engine step failed: {ex}")
                for s in req.seqs:
                    if not s.finished:
                        self.sched.finish(s.seq_id, _host.FINISH_ERROR)
                        self.seq_owner.pop(s.seq_id, None)
                        self.sched.forget(s.seq_id)
                        s.finished, s.finish_reason = True, "error"
                req.finished = True
                req.notify()
            self.requests.clear()

    # ---- convenience ------------------------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[Sequence[SamplingParams]] = None
                 ) -> List[Request]:
        """Synchronous batch generation (offline use, tests, benchmarks)."""
        if params is None:
            params = [SamplingParams() for _ in prompts]
        elif isinstance(params, SamplingParams):
            params = [params for _ in prompts]
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        if self._loop_thread is None:
            self.run_until_done()
        else:
            for r in reqs:
                v = -1
                while not r.finished:
                    v = r.wait(v, 1.0)
        return reqs
