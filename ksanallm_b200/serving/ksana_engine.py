"""Public Python engine API: ``KsanaLLMEngine`` (from_engine_args / initialize / generate / forward).

Same surface as the reference's Python wrapper (src/ksana_llm/python/ksana_llm/ksana_engine.py:91-473 and
arg_utils.py:36-254): a request dictionary with ``prompt`` | ``input_tokens`` | ``messages``, ``sampling_config``,
``stream`` ... goes in, a status plus an output object (or an async iterator of outputs when streaming) comes out.
Underneath it drives :class:`ksanallm_b200.engine.llm_engine.LLMEngine` instead of a pybind module.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import os
from dataclasses import dataclass, field
from typing import Any, AsyncIterator, Dict, List, Optional, Tuple

import torch

from ..config.model_config import ModelConfig, load_model_config, NAMED_CONFIGS
from ..config.schema import ServingConfig, load_serving_config, parse_serving_config
from ..engine.llm_engine import EngineError, LLMEngine, Request
from ..engine.sampling_params import SamplingParams
from ..engine.forward_probe import validate_targets
from .tokenizer import TokenizerProcessor


# ---- status object -------------------------------------------------------------------------------------
class RetCode:
    RET_SUCCESS = 0
    RET_EXCEED_CAPACITY = 1
    RET_INPUT_LENGTH_EXCEEDED = 2
    RET_INVALID_ARGUMENT = 3
    RET_REQUEST_TIMEOUT = 4
    RET_REQUEST_TERMINATED = 5
    RET_OUT_OF_MEMORY = 6
    RET_INTERNAL_ERROR = 7
    RET_STOP_ITERATION = 3011  # a streaming iterator has no further item (the reference's value)


class _Code(int):
    @property
    def value(self) -> int:
        return int(self)


class Status:
    def __init__(self, code: int = 0, message: str = ""):
        self._code, self._msg = code, message

    def OK(self) -> bool:  # noqa: N802  (name kept for API compatibility)
        return self._code == 0

    def GetMessage(self) -> str:  # noqa: N802
        return self._msg

    def GetCode(self):  # noqa: N802
        return _Code(self._code)

    def __repr__(self):
        return f"Status(code={self._code}, message={self._msg!r})"


@dataclass
class KsanaPythonOutput:
    input_tokens: List[int] = field(default_factory=list)
    output_tokens: List[List[int]] = field(default_factory=list)
    logprobs: List[Any] = field(default_factory=list)
    finish_status: Status = field(default_factory=Status)
    finish_reasons: List[Optional[str]] = field(default_factory=list)
    finished: bool = False


@dataclass
class EngineArgs:
    config_file: str = ""
    model_dir: str = ""
    tokenizer_path: str = ""
    model_type: str = ""
    host: str = "0.0.0.0"
    port: int = 8080
    endpoint: str = "python"
    access_log: bool = True
    ssl_keyfile: Optional[str] = None
    ssl_certfile: Optional[str] = None
    root_path: Optional[str] = None
    tool_call_parser: Optional[str] = None
    reasoning_parser: Optional[str] = None
    enable_auto_tool_choice: bool = False
    tool_parser_plugin: str = ""
    chat_template: Optional[str] = None
    chat_template_content_format: str = "auto"
    synthetic_model: Optional[str] = None  # one of NAMED_CONFIGS: random weights, no checkpoint files needed
    device: Optional[str] = None
    serving: Optional[ServingConfig] = None
    max_token_len: int = 0

    @classmethod
    def from_config_file(cls, config_file: str, **overrides) -> "EngineArgs":
        serving = load_serving_config(config_file)
        a = cls(config_file=config_file, serving=serving, model_dir=serving.model_spec.model_dir)
        a.endpoint = serving.setting.endpoint_type or "python"
        a.max_token_len = serving.setting.batch_scheduler.max_token_len
        for k, v in overrides.items():
            if v is not None and hasattr(a, k):
                setattr(a, k, v)
        if not a.tokenizer_path:
            a.tokenizer_path = a.model_dir
        cfg_path = os.path.join(a.model_dir or "", "config.json")
        if os.path.isfile(cfg_path):
            with open(cfg_path, "r", encoding="utf-8") as f:
                a.model_type = str(json.load(f).get("model_type", ""))
        return a

    @classmethod
    def add_cli_args(cls, p: argparse.ArgumentParser) -> argparse.ArgumentParser:
        p.add_argument("--config_file", type=str, default="examples/ksana_llm.yaml", help="serving config file")
        p.add_argument("--tokenizer_path", type=str, default=None)
        p.add_argument("--host", type=str, default="0.0.0.0")
        p.add_argument("--port", type=int, default=8080)
        p.add_argument("--endpoint", type=str, default=None)
        p.add_argument("--access_log", action="store_true", default=False)
        p.add_argument("--ssl_keyfile", type=str, default=None)
        p.add_argument("--ssl_certfile", type=str, default=None)
        p.add_argument("--root_path", type=str, default=None)
        p.add_argument("--tool-call-parser", dest="tool_call_parser", type=str, default=None)
        p.add_argument("--reasoning-parser", dest="reasoning_parser", type=str, default=None)
        p.add_argument("--enable-auto-tool-choice", dest="enable_auto_tool_choice", action="store_true")
        p.add_argument("--tool-parser-plugin", dest="tool_parser_plugin", type=str, default="")
        p.add_argument("--chat-template", dest="chat_template", type=str, default=None)
        p.add_argument("--chat-template-content-format", dest="chat_template_content_format", type=str, default="auto",
                       choices=["auto", "string", "openai"])
        p.add_argument("--synthetic-model", dest="synthetic_model", type=str, default=None,
                       help="serve random-init weights of a named architecture: " + ", ".join(NAMED_CONFIGS))
        p.add_argument("--device", type=str, default=None)
        return p

    @classmethod
    def from_command_line(cls, argv: Optional[List[str]] = None) -> "EngineArgs":
        p = cls.add_cli_args(argparse.ArgumentParser(description="ksanallm_b200 serving server"))
        ns = p.parse_args(argv)
        d = vars(ns)
        cfg_file = d.pop("config_file")
        return cls.from_config_file(cfg_file, **d)


class PyAsyncStreamingIterator:
    """Async iterator over the growing output of one request; each item carries the FULL output so far
    (reference streaming contract). Dropping the iterator aborts the request (client disconnect)."""

    def __init__(self, engine: "KsanaLLMEngine", req: Request):
        self.engine, self.req = engine, req
        self.version = -1
        self.done = False

    def __aiter__(self):
        return self

    async def __anext__(self) -> KsanaPythonOutput:
        if self.done:
            raise StopAsyncIteration
        loop = asyncio.get_running_loop()
        self.version = await loop.run_in_executor(self.engine.pool, self.req.wait, self.version, 1.0)
        out = self.engine._snapshot(self.req)
        if self.req.finished:
            self.done = True
        return out

    def abort(self) -> None:
        if not self.req.finished and not getattr(self, "detached", False):
            self.engine.llm.abort(self.req)

    def __del__(self):
        try:
            self.abort()
        except Exception:
            pass


class _FinishedIterator:
    """Streaming view of a request that is already complete (one item)."""

    def __init__(self, out: KsanaPythonOutput):
        self.out = out

    def __aiter__(self):
        return self

    async def __anext__(self) -> KsanaPythonOutput:
        if self.out is None:
            raise StopAsyncIteration
        out, self.out = self.out, None
        return out


class KsanaLLMEngine:
    def __init__(self, args: EngineArgs):
        self.args = args
        self.serving: ServingConfig = args.serving or parse_serving_config({})
        self.llm: Optional[LLMEngine] = None
        self.tokenizer: Optional[TokenizerProcessor] = None
        self.model_config: Optional[ModelConfig] = None
        self.plugin = None
        self.think_end_token_id: Optional[int] = None
        # every in-flight request parks one thread while it waits for its next tokens; the event loop's default
        # executor (a few dozen threads) would make hundreds of concurrent streams take turns (the reference runs its
        # blocking calls in a 1024-thread executor as well: ksana_engine.py)
        from concurrent.futures import ThreadPoolExecutor
        self.pool = ThreadPoolExecutor(max_workers=int(os.environ.get("KSANA_WAITER_THREADS", "1024")),
                                       thread_name_prefix="ksana-wait")

    @classmethod
    def from_engine_args(cls, args: EngineArgs) -> "KsanaLLMEngine":
        return cls(args)

    # ---- bootstrap ---------------------------------------------------------------------------------------
    def initialize(self, tp=None) -> None:
        """Loads config, weights and the model on this rank and starts the step loop (rank 0 only)."""
        from ..models.loader import load_model_weights
        from ..models.transformer import TransformerModel
        from ..parallel.comm import TPGroup, init_distributed, world_group

        a = self.args
        world = int(os.environ.get("WORLD_SIZE", "1"))
        want_cuda = (a.device or ("cuda" if torch.cuda.is_available() else "cpu")).startswith("cuda")
        if tp is None:
            tp = init_distributed("cuda" if want_cuda else "cpu") if (world > 1 or want_cuda) else TPGroup()
        device = tp.device if tp.device is not None else torch.device(a.device or "cpu")
        if a.synthetic_model:
            cfg = NAMED_CONFIGS[a.synthetic_model]()
        else:
            cfg = load_model_config(a.model_dir)
        self.model_config = cfg
        dtype = torch.float32 if device.type == "cpu" and cfg.torch_dtype == "float32" else \
            (torch.bfloat16 if device.type == "cuda" else getattr(torch, cfg.torch_dtype, torch.float32))
        qmethod = self.serving.setting.quantization_config.weight.quant_method
        quantize = {"fp8_e4m3": "fp8_block", "fp8_block": "fp8_block", "int4": "int4"}.get(qmethod)
        bs = self.serving.setting.batch_scheduler
        g = self.serving.setting.global_
        world_tp = tp
        topo = layer_range = None
        if g.pipeline_para_size > 1:
            # pipeline stages: world = stages x tensor_para_size, stage-major rank order; every stage gets its own
            # tensor-parallel group and a contiguous layer range (reference: PipelineConfig + layer allocation in
            # distributed/control_channel.cpp, here parallel/pipeline.py)
            import torch.distributed as dist
            from ..parallel.pipeline import StageTopology, split_layers
            if world_tp.size != g.pipeline_para_size * g.tensor_para_size:
                raise ValueError(f"pipeline_para_size x tensor_para_size = {g.pipeline_para_size * g.tensor_para_size}"
                                 f" but {world_tp.size} ranks were started")
            topo = StageTopology(world_tp.size, g.tensor_para_size, world_tp.rank)
            layer_range = split_layers(cfg.num_layers, topo.num_stages)[topo.stage]
            stage_group = None
            for st in range(topo.num_stages):  # every rank creates every group, in the same order
                ranks = list(range(st * topo.tp_size, (st + 1) * topo.tp_size))
                grp = dist.new_group(ranks) if topo.tp_size > 1 else None
                if st == topo.stage:
                    stage_group = grp
            tp = TPGroup(topo.tp_rank, topo.tp_size, stage_group, device, use_fused=False) if topo.tp_size > 1 \
                else TPGroup(0, 1, None, device, use_fused=False)
        dp_world = None
        ep_rank = ep_size = None
        if g.attn_data_para_size > 1:
            # attention data parallelism: every rank is a DP group of its own (attention / dense weights replicated,
            # own scheduler and KV cache), the routed experts are sharded over all ranks (reference: attn_data_para_size
            # + expert_para_size, service/inference_engine.cpp:201-260)
            if topo is not None or world_tp.size % g.attn_data_para_size:
                raise ValueError("the number of ranks must be a multiple of attn_data_para_size, and attention DP "
                                 "cannot be combined with pipeline stages")
            import torch.distributed as dist
            dp_world = world_tp
            attn_tp = world_tp.size // g.attn_data_para_size  # ranks per DP group (tensor-parallel inside)
            dp_group_id, dp_tp_rank = world_tp.rank // attn_tp, world_tp.rank % attn_tp
            tp = TPGroup(0, 1, None, device, use_fused=False)
            dp_ctl = None
            if attn_tp > 1:
                for gi in range(g.attn_data_para_size):  # every rank creates every group, in the same order
                    ranks = list(range(gi * attn_tp, (gi + 1) * attn_tp))
                    grp, ctl = dist.new_group(ranks), dist.new_group(ranks, backend="gloo")
                    if gi == dp_group_id:
                        tp, dp_ctl = TPGroup(dp_tp_rank, attn_tp, grp, device, use_fused=False), ctl
            if cfg.is_moe:
                ep_rank, ep_size = dp_world.rank, dp_world.size
                tp.ep_rank, tp.ep_size = ep_rank, ep_size
                plain_experts = cfg.quant.method in ("none", "", None) and not quantize
                # the grouped expert GEMM behind the peer-memory exchange takes hidden and 2 x expert widths that are
                # multiples of 128; other shapes (and quantised experts) go through the collective exchange
                inter = cfg.moe_intermediate_size or cfg.intermediate_size
                grouped_ok = cfg.hidden_size % 128 == 0 and (2 * inter) % 128 == 0 and inter % 8 == 0
                if device.type == "cuda" and 2 <= dp_world.size <= 8 and cfg.num_experts % dp_world.size == 0 \
                        and plain_experts and grouped_ok:
                    from ..parallel.ep import EPExchange
                    tp.ep = EPExchange(dp_world.group, dp_world.rank, dp_world.size, device, cfg.hidden_size,
                                       cfg.num_experts_per_tok, cfg.num_experts, bs.max_step_tokens)
                else:
                    from ..parallel.attn_dp import GatherEPExchange
                    tp.ep = GatherEPExchange(dp_world.group, dp_world.rank, dp_world.size, cfg.num_experts_per_tok,
                                             cfg.num_experts)
        weights = load_model_weights(cfg, "" if a.synthetic_model else a.model_dir, tp.rank, tp.size, device, dtype,
                                     quantize, synthetic_seed=0 if a.synthetic_model else None,
                                     layer_range=layer_range, ep_rank=ep_rank, ep_size=ep_size)
        if tp.size > 1 and device.type == "cuda" and topo is None and dp_world is None:
            tp.init_fused(cfg.hidden_size, bs.max_step_tokens)
        model = TransformerModel(cfg, weights, tp, max_positions=max(bs.max_token_len, 2048), layer_range=layer_range)
        if topo is not None and not topo.is_last:
            model.norm_w = None  # the next stage continues from the un-normalised residual stream
        self.tokenizer = TokenizerProcessor(a.tokenizer_path or a.model_dir, cfg.vocab_size,
                                            self.serving.setting.tokenization.add_special_tokens,
                                            self.serving.setting.tokenization.skip_special_tokens, a.chat_template)
        kvd = self.serving.setting.quantization_config.kv_cache.dtype
        kv_dtype = torch.float8_e4m3fn if kvd == "fp8_e4m3" else (torch.float8_e5m2 if kvd == "fp8_e5m2" else None)
        if kv_dtype is not None and not a.synthetic_model:
            from ..models.kv_scales import apply_kv_scales, find_kv_scales_file, load_kv_cache_scales
            scales_file = find_kv_scales_file(a.model_dir)
            if scales_file:
                apply_kv_scales(model, load_kv_cache_scales(scales_file, tp.rank, cfg.num_layers))
        self.llm = LLMEngine(model, self.serving, tp, detokenize=lambda ids: self.tokenizer.decode(ids),
                             kv_dtype=kv_dtype, block_sync_group=world_tp.group if topo is not None else None)
        if dp_world is not None:
            import torch.distributed as dist
            from ..parallel.attn_dp import DPCoordinator, DPRequestRouter, DPRequestWorker
            balance = None
            if attn_tp > 1 and self.serving.setting.batch_scheduler.attention_dp_lb_config.enable_balance:
                # the prefill balancer's agreement runs between the DP groups' leaders (the ranks that schedule);
                # every rank creates the group, only leaders use it
                leaders = dist.new_group(ranks=[gi * attn_tp for gi in range(g.attn_data_para_size)], backend="gloo")
                if dp_tp_rank == 0:
                    balance = DPCoordinator(leaders)
            self.llm.attach_dp(DPCoordinator(dp_world.group, device if device.type == "cuda" else None), balance)
            if dp_ctl is not None:
                self.llm.attach_control_group(dp_ctl, src=dp_group_id * attn_tp)
                self.llm.is_driver = dp_tp_rank == 0
            host = os.environ.get("MASTER_ADDR", "127.0.0.1")
            port = int(os.environ.get("KSANA_DP_PORT", int(os.environ.get("MASTER_PORT", "29511")) + 17))
            if dp_world.rank == 0:
                self.llm.dp_router = DPRequestRouter(self.llm, host, port, g.attn_data_para_size)
                dist.barrier(group=dp_world.group)  # the listener exists before anybody connects
                self.llm.dp_router.accept_all()
            else:
                dist.barrier(group=dp_world.group)
                if dp_tp_rank == 0:  # the leaders of the other DP groups take requests from rank 0
                    self.llm.dp_worker = DPRequestWorker(self.llm, host, port, dp_group_id)
        elif world_tp.size > 1:
            import torch.distributed as dist
            self.llm.attach_control_group(dist.new_group(backend="gloo"))
        if topo is not None:
            from ..parallel.pipeline import HiddenChannel, PipelineStage
            self.llm.attach_pipeline(PipelineStage(model, topo, HiddenChannel(topo, cfg.hidden_size, dtype, device)),
                                     max(int(bs.max_pp_batch_num), 1))
        self.is_driver = world_tp.rank == 0
        self._start_heartbeat(world_tp)
        self._load_plugin()
        self.connector = None
        cs = self.serving.setting.connector
        if cs.group_role in ("prefill", "decode", "both") and world_tp.rank == 0:
            from .connector import PDConnector
            self.connector = PDConnector(self.llm, cs)
            self.connector.start()
        elif cs.group_role in ("prefill", "decode", "both") and topo is None and dp_world is None:
            from .connector import PDShardWorker
            self.connector = PDShardWorker(self.llm, cs, world_tp.rank)
            self.connector.start()
        from ..ops import gemm_tune
        gemm_tune.maybe_load_from_env()  # KSANA_GEMM_TUNE_FILE written by benchmarks/search_best_gemm.py
        if world_tp.rank == 0:
            if os.environ.get("KSANA_SKIP_WARMUP", "0") != "1" and world_tp.size == 1:
                # multi-rank instances warm up through their first requests: the followers only enter their loop
                # after initialisation returns
                self.llm.warmup(max_len=min(2048, self.serving.setting.batch_scheduler.max_token_len))
            self.llm.start()

    def _start_heartbeat(self, world) -> None:
        """Failure detection between the ranks of one instance: every rank beats to rank 0 over the TCP control
        channel; a rank that falls silent (process gone, host down) is reported, rank 0 fails what is in flight and
        refuses new requests instead of waiting in a collective for ever. KSANA_HEARTBEAT_TIMEOUT_S (default 120, 0 =
        off). Reference: distributed/control_channel.cpp heartbeat -> cluster shutdown."""
        self.control = None
        self.failed_ranks = []
        timeout = float(os.environ.get("KSANA_HEARTBEAT_TIMEOUT_S", "120"))
        if world.size <= 1 or timeout <= 0:
            return
        from ..parallel.control_channel import ControlMaster, ControlWorker
        host = os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = int(os.environ.get("KSANA_CONTROL_PORT", int(os.environ.get("MASTER_PORT", "29511")) + 23))
        interval = max(min(timeout / 4.0, 30.0), 0.05)
        if world.rank == 0:
            def lost(rank: int) -> None:
                self.failed_ranks.append(rank)
                self.llm._fail_all(RuntimeError(f"rank {rank} stopped sending heartbeats"))
            self.control = ControlMaster(host, port, world.size, interval, timeout, on_failure=lost)
        else:
            self.control = ControlWorker(host, port, world.rank, interval, timeout, connect_timeout=120.0)

    def serve_follower(self) -> None:
        """Blocks in the follower loop (ranks > 0): executes rank 0's plans (TP / PP), or - as an attention-DP rank -
        runs its own scheduler on the requests rank 0 places here."""
        if self.llm.dp is not None and self.llm.is_driver:
            self.llm.serve_dp()  # the leader of a DP group
        else:
            self.llm.follow()

    def shutdown(self) -> None:
        if getattr(self, "control", None) is not None:
            (self.control.shutdown if hasattr(self.control, "shutdown") else self.control.close)()
        from ..models.layers import dump_eplb_counts
        dump_eplb_counts(rank=int(os.environ.get("RANK", "0")))  # no-op unless DUMP_EPLB_PATH asked for routing counts
        if getattr(self, "connector", None) is not None:
            self.connector.stop()
        if self.llm is not None:
            self.llm.stop()
        self.pool.shutdown(wait=False)

    def _load_plugin(self) -> None:
        from .plugin import load_plugin
        self.plugin = load_plugin(self.args.model_dir, self.serving.model_spec.plugin_model, self)

    # ---- request construction --------------------------------------------------------------------------------
    def _build_sampling(self, request_dict: Dict[str, Any]) -> SamplingParams:
        sc = dict(request_dict.get("sampling_config") or {})
        for k in ("structured_output_regex",):
            if k in request_dict and k not in sc:
                sc[k] = request_dict[k]
        if "max_new_tokens" not in sc:
            sc["max_new_tokens"] = max(self.serving.setting.batch_scheduler.max_token_len // 2, 1)
        return SamplingParams.from_dict(sc)

    def _build_tokens(self, request_dict: Dict[str, Any]) -> Tuple[List[int], Any]:
        refit = None
        if request_dict.get("input_tokens") is not None:
            tokens = [int(t) for t in request_dict["input_tokens"]]
        elif request_dict.get("messages") is not None:
            msgs = request_dict["messages"]
            kw = {}
            if request_dict.get("sampling_config", {}).get("enable_thinking") is not None:
                kw["enable_thinking"] = bool(request_dict["sampling_config"]["enable_thinking"])
            text = self.tokenizer.apply_chat_template(msgs, True, request_dict.get("tools"), **kw)
            tokens = self.tokenizer.encode(text, add_special_tokens=False)
        else:
            prompt = request_dict.get("prompt")
            if prompt is None:
                raise ValueError("one of prompt, input_tokens, messages is required")
            if request_dict.get("use_chat_template"):
                prompt = self.tokenizer.apply_chat_template([{"role": "user", "content": prompt}])
                tokens = self.tokenizer.encode(prompt, add_special_tokens=False)
            else:
                tokens = self.tokenizer.encode(prompt)
        emb = request_dict.get("input_refit_embedding") or {}
        pos = emb.get("pos", request_dict.get("pos"))
        vals = emb.get("embeddings", request_dict.get("embeddings"))
        if pos and vals:
            refit = []
            for p, e in zip(pos, vals):
                t = torch.as_tensor(e, dtype=torch.float32)
                refit.append((int(p), t.view(-1, self.model_config.hidden_size)))
        self._last_mrope = (request_dict.get("additional_params") or {}).get("mrope_positions")
        if self.plugin is not None:
            extra = self.plugin.preprocess(request_dict, tokens)
            if extra:
                tokens = extra.get("input_tokens", tokens)
                refit = extra.get("refit", refit)
                # vision plugins of M-RoPE models return [3, prompt_len] (temporal, height, width) positions
                self._last_mrope = extra.get("mrope_positions", self._last_mrope)
        return tokens, refit

    def _grammar_for(self, sp: SamplingParams):
        if not (sp.enable_structured_output or sp.json_schema or sp.structured_output_regex):
            return None
        from ..engine.structured import build_grammar
        return build_grammar(sp, self.tokenizer, self.model_config.vocab_size, self.think_end_token_id)

    def _snapshot(self, req: Request) -> KsanaPythonOutput:
        out = KsanaPythonOutput(input_tokens=list(req.prompt_tokens))
        seqs = req.seqs
        if req.beam is not None and req.finished:
            seqs = req.beam.best(req)
        elif req.params.num_return_sequences < len(seqs) and req.finished:
            seqs = seqs[:req.params.num_return_sequences]
        first = list(getattr(req, "pd_first", []) or [])
        out.output_tokens = [first + list(s.output_tokens) for s in seqs]
        if first:
            out.input_tokens = list(req.prompt_tokens[:req.pd_prompt_len])
        out.logprobs = [s.logprobs for s in seqs] if req.params.logprobs else []
        out.finish_reasons = [s.finish_reason for s in seqs]
        out.finished = req.finished
        if req.error is not None:
            out.finish_status = Status(req.error.code, str(req.error))
        return out

    # ---- public calls --------------------------------------------------------------------------------------------
    async def generate(self, request_dict: Dict[str, Any], streamer: Optional[bool] = None,
                       req_ctx: Optional[Dict[str, str]] = None):
        """Returns (Status, KsanaPythonOutput) or (Status, async iterator of KsanaPythonOutput) when streaming."""
        if getattr(self, "failed_ranks", None):
            return Status(RetCode.RET_INTERNAL_ERROR, f"ranks {self.failed_ranks} of this instance are gone"), None
        if self.llm.refusing_requests():
            return Status(RetCode.RET_INTERNAL_ERROR, f"device fault on this instance: {self.llm.device_fault}"), None
        pd_first: List[int] = []
        pd_rid = (req_ctx or {}).get("kv-comm-request-id") if getattr(self, "connector", None) is not None else None
        try:
            sp = self._build_sampling(request_dict)
            tokens, refit = self._build_tokens(request_dict)
            mrope = self._last_mrope  # taken before any await: other requests share the attribute
            grammar = self._grammar_for(sp)
            if pd_rid and self.connector.role == "decode":
                # the prefill instance computes the prompt and pushes its KV blocks + first token here
                loop0 = asyncio.get_running_loop()
                got = await loop0.run_in_executor(self.pool, self.connector.wait_import, pd_rid,
                                                  float(self.serving.setting.connector.connector_waiting_sec))
                if got is None:
                    return Status(RetCode.RET_REQUEST_TIMEOUT,
                                  "timed out waiting for the prefill instance's KV transfer"), None
                _, pd_first, _ = got
                if pd_first:
                    import dataclasses as _dc
                    stops = set(sp.stop_token_ids or [])
                    if not sp.ignore_eos:
                        stops |= set(self.model_config.eos_token_ids)
                    left = sp.max_new_tokens - len(pd_first)
                    if pd_first[-1] in stops or left <= 0:
                        # the prefill instance's token already ended the request
                        out = KsanaPythonOutput(input_tokens=list(tokens), output_tokens=[list(pd_first)],
                                                finish_reasons=["stop" if pd_first[-1] in stops else "length"],
                                                finished=True)
                        return Status(), (_FinishedIterator(out) if streamer else out)
                    tokens = list(tokens) + list(pd_first)
                    sp = _dc.replace(sp, max_new_tokens=left)
                    if mrope is not None:
                        # multi-axis positions cover the prompt; the handed-over tokens continue from max + 1 on
                        # every axis, as generated tokens do
                        mp = torch.as_tensor(mrope, dtype=torch.int32)
                        mp = mp.reshape(-1, len(tokens) - len(pd_first))
                        tail = (int(mp.max()) + 1 + torch.arange(len(pd_first), dtype=torch.int32)).expand(mp.shape[0], -1)
                        mrope = torch.cat((mp, tail), dim=1)
            elif pd_rid and self.connector.role == "prefill":
                import dataclasses as _dc
                sp = _dc.replace(sp, max_new_tokens=1)
            req = self.llm.add_request(tokens, sp, refit=refit, grammar=grammar, mrope_positions=mrope)
            req.ctx = req_ctx or {}
            if pd_rid and self.connector.role == "prefill" and refit is None:
                self.connector.expect_export(req, pd_rid, (req_ctx or {}).get("kv-comm-group-key", ""))
            req.pd_first = pd_first
            req.pd_prompt_len = len(tokens) - len(pd_first)
        except EngineError as ex:
            return Status(ex.code, str(ex)), None
        except (ValueError, KeyError, TypeError) as ex:
            return Status(RetCode.RET_INVALID_ARGUMENT, str(ex)), None
        handing_over = bool(pd_rid) and self.connector.role == "prefill"
        if streamer and not handing_over:
            return Status(), PyAsyncStreamingIterator(self, req)
        loop = asyncio.get_running_loop()
        v = -1
        while not req.finished:
            v = await loop.run_in_executor(self.pool, req.wait, v, 1.0)
        out = self._snapshot(req)
        if pd_rid and self.connector.role == "prefill" and req.error is None:
            # hand the request over: KV of the prompt's full blocks + the first token
            await loop.run_in_executor(self.pool, self.connector.export, pd_rid, (req_ctx or {}).get("kv-comm-group-key", ""),
                                       list(req.prompt_tokens), list(req.seqs[0].output_tokens))
        elif pd_rid and self.connector.role == "prefill":
            self.connector.cancel_export(pd_rid)
        if self.plugin is not None:
            self.plugin.postprocess(request_dict, out)
        if streamer:  # a prefill instance answers a streaming request with its single item
            return out.finish_status, _FinishedIterator(out)
        return out.finish_status, out

    def generate_sync(self, request_dict: Dict[str, Any]) -> Tuple[Status, Optional[KsanaPythonOutput]]:
        return asyncio.run(self.generate(request_dict, streamer=False))

    async def forward(self, request_bytes: bytes, req_ctx: Optional[Dict[str, str]] = None):
        """msgpack (or JSON when Content-Type says so) batch of single-prefill probes -> packed responses."""
        import msgpack
        is_json = bool(req_ctx) and "json" in (req_ctx.get("Content-Type", "") or "").lower()
        try:
            body = json.loads(request_bytes) if is_json else msgpack.unpackb(request_bytes, raw=False)
            reqs = []
            for r in body.get("requests", []):
                tokens, refit = self._build_tokens(r)
                targets = r.get("request_target") or []
                validate_targets(targets, len(tokens))
                sp = SamplingParams(topk=1, max_new_tokens=1, ignore_eos=True)
                reqs.append(self.llm.add_request(tokens, sp, refit=refit, probe=targets))
        except EngineError as ex:
            return Status(ex.code, str(ex)), None
        except Exception as ex:
            return Status(RetCode.RET_INVALID_ARGUMENT, str(ex)), None
        loop = asyncio.get_running_loop()
        for q in reqs:
            v = -1
            while not q.finished:
                v = await loop.run_in_executor(self.pool, q.wait, v, 1.0)
        responses = [{"input_token_ids": list(q.prompt_tokens), "response": q.probe_result or []} for q in reqs]
        payload = {"responses": responses}
        data = json.dumps(payload).encode() if is_json else msgpack.packb(payload, use_bin_type=True)
        return Status(), data
