"""Typed view of the serving YAML.

The YAML schema is the reference's public configuration surface and is kept key-for-key
(`setting.global`, `setting.batch_scheduler`, `setting.block_manager`, `setting.attn_backend`,
`setting.quantization_config`, `setting.profiler`, `setting.connector`, `setting.tokenization`,
`model_spec.base_model.model_dir`; parser in the reference:
src/ksana_llm/utils/config/schedule_config_parser.cpp:90-428, examples/ksana_llm2-7b.yaml).
Unknown keys are preserved in ``extra`` so a reference YAML always loads.
"""
from __future__ import annotations

import dataclasses
import os
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import yaml


def _fill(dc, src: Optional[Dict[str, Any]]):
    """Copies known keys of ``src`` into dataclass ``dc``; the rest goes to ``dc.extra``."""
    if not src:
        return dc
    names = {f.name: f for f in dataclasses.fields(dc)}
    for k, v in src.items():
        if k in names and k != "extra":
            cur = getattr(dc, k)
            if dataclasses.is_dataclass(cur) and isinstance(v, dict):
                _fill(cur, v)
            elif isinstance(cur, bool):
                setattr(dc, k, bool(v))
            elif isinstance(cur, int) and not isinstance(v, bool) and v is not None:
                setattr(dc, k, int(v))
            elif isinstance(cur, float) and v is not None:
                setattr(dc, k, float(v))
            else:
                setattr(dc, k, v)
        else:
            dc.extra[k] = v
    return dc


@dataclass
class GlobalSetting:
    tensor_para_size: int = 1
    pipeline_para_size: int = 1
    attn_data_para_size: int = 1
    expert_para_size: int = 1
    expert_world_size: int = 1
    enable_full_shared_expert: bool = False
    pipeline_para_comm_type: str = "default"
    enable_lora_adapter: bool = False
    embed_tokens_use_cpu: bool = False
    enable_cuda_graph: bool = True
    is_version_report: bool = False
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class AttentionDpLbConfig:
    # reference defaults: utils/config/schedule_config_parser.cpp:268-275
    enable_balance: bool = False
    max_waiting_steps: int = 50
    max_waiting_time_in_ms: int = 1000
    min_qps_for_waiting: float = -1.0
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class BatchSchedulerSetting:
    schedule_strategy: int = 0
    waiting_timeout_in_ms: int = 3600000
    max_waiting_queue_len: int = 1200
    max_step_tokens: int = 4096
    max_batch_size: int = 128
    max_token_len: int = 2048
    max_pp_batch_num: int = 1
    pp_multibatch_wb_strategy: int = 0
    swapout_block_threshold: float = 1.0
    swapin_block_threshold: float = 2.0
    launch_block_threshold: float = 2.0
    enable_auto_prefix_cache: bool = False
    split_fuse_token_num: int = 0
    swap_threadpool_size: int = 8
    preempt_mode: int = 0
    min_flexible_cache_num: int = 0
    enable_speculative_decoding: bool = False
    mtp_step_num: int = 0
    enable_xgrammar: bool = False
    enable_async: bool = False
    max_pretransfer_batch_size: int = 64
    transfer_layer_chunk_size: int = 1
    attention_dp_lb_config: AttentionDpLbConfig = field(default_factory=AttentionDpLbConfig)
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class BlockManagerSetting:
    block_token_num: int = 16
    reserved_device_memory_ratio: float = 0.01
    lora_deivce_memory_ratio: float = 0.0
    lora_host_memory_factor: float = 10.0
    block_device_memory_ratio: float = -1.0
    block_host_memory_factor: float = 1.0
    enable_block_checksum: bool = False
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class AttnBackendSetting:
    enable_blocked_multi_token_forwarding_kv: bool = True
    use_flashinfer_for_decode: bool = False
    flash_attn_impl: str = "auto"
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class KvCacheQuant:
    dtype: str = "auto"  # auto | fp8_e4m3 | fp8_e5m2
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class WeightQuant:
    quant_method: str = "auto"
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class QuantizationSetting:
    gptq_backend: str = "auto"
    kv_cache: KvCacheQuant = field(default_factory=KvCacheQuant)
    weight: WeightQuant = field(default_factory=WeightQuant)
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ProfilerSetting:
    metrics_export_url: str = ""
    trace_export_url: str = ""
    export_interval_millis: int = 60000
    export_timeout_millis: int = 1000
    attributes: Dict[str, Any] = field(default_factory=dict)
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ConnectorSetting:
    group_role: str = "none"  # none | prefill | decode | both
    router_addr: str = ""
    group_name: str = ""
    node_name: str = ""
    heartbeat_interval_ms: int = 5000
    transfer_batch: int = 1048576
    connector_waiting_sec: int = 3600
    communication_type: str = "nccl"
    inference_addr: str = ""
    inference_port: int = 8080
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class TokenizationSetting:
    add_special_tokens: bool = True
    skip_special_tokens: bool = True
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class Setting:
    global_: GlobalSetting = field(default_factory=GlobalSetting)
    batch_scheduler: BatchSchedulerSetting = field(default_factory=BatchSchedulerSetting)
    block_manager: BlockManagerSetting = field(default_factory=BlockManagerSetting)
    attn_backend: AttnBackendSetting = field(default_factory=AttnBackendSetting)
    quantization_config: QuantizationSetting = field(default_factory=QuantizationSetting)
    profiler: ProfilerSetting = field(default_factory=ProfilerSetting)
    connector: ConnectorSetting = field(default_factory=ConnectorSetting)
    tokenization: TokenizationSetting = field(default_factory=TokenizationSetting)
    endpoint_type: str = "python"
    kernel_config: Dict[str, Any] = field(default_factory=dict)
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ModelSpec:
    model_dir: str = ""
    plugin_model: Dict[str, Any] = field(default_factory=dict)
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ServingConfig:
    setting: Setting = field(default_factory=Setting)
    model_spec: ModelSpec = field(default_factory=ModelSpec)
    config_file: str = ""
    raw: Dict[str, Any] = field(default_factory=dict)

    # ---- derived views -----------------------------------------------------------------------
    @property
    def tp(self) -> int:
        return self.setting.global_.tensor_para_size

    @property
    def attn_dp(self) -> int:
        return self.setting.global_.attn_data_para_size

    @property
    def ep(self) -> int:
        return self.setting.global_.expert_para_size

    def validate(self) -> None:
        """Cross-field rules (reference: schedule_config_parser.cpp:188-205, 263-266, 423-426)."""
        g, b = self.setting.global_, self.setting.batch_scheduler
        if g.tensor_para_size < 1 or g.attn_data_para_size < 1:
            raise ValueError("tensor_para_size and attn_data_para_size must be >= 1")
        if g.tensor_para_size % g.attn_data_para_size != 0:
            raise ValueError("tensor_para_size must be a multiple of attn_data_para_size")
        if b.max_step_tokens < 1 or b.max_batch_size < 1:
            raise ValueError("max_step_tokens and max_batch_size must be >= 1")
        if b.split_fuse_token_num > 0:
            # chunked prefill re-reads earlier chunks from the cache: prefix caching is implied
            b.enable_auto_prefix_cache = True
            if b.enable_async:
                raise ValueError("split_fuse_token_num cannot be combined with enable_async")
        if self.setting.block_manager.block_token_num < 1:
            raise ValueError("block_token_num must be >= 1")
        if b.preempt_mode not in (0, 1):
            raise ValueError("preempt_mode must be 0 (swap) or 1 (recompute)")
        kvd = self.setting.quantization_config.kv_cache.dtype
        if kvd not in ("auto", "fp8_e4m3", "fp8_e5m2"):
            raise ValueError(f"unsupported kv_cache.dtype {kvd}")


def parse_serving_config(raw: Dict[str, Any], config_file: str = "") -> ServingConfig:
    cfg = ServingConfig(config_file=config_file, raw=raw or {})
    setting = dict((raw or {}).get("setting") or {})
    st = cfg.setting
    _fill(st.global_, setting.pop("global", None))
    for key in ("batch_scheduler", "block_manager", "attn_backend", "quantization_config", "profiler",
                "connector", "tokenization"):
        _fill(getattr(st, key), setting.pop(key, None))
    if "endpoint_type" in setting:
        st.endpoint_type = str(setting.pop("endpoint_type"))
    if "kernel_config" in setting:
        st.kernel_config = setting.pop("kernel_config") or {}
    st.extra.update(setting)
    ms = dict((raw or {}).get("model_spec") or {})
    base = dict(ms.pop("base_model", None) or {})
    cfg.model_spec.model_dir = str(base.pop("model_dir", "") or "")
    cfg.model_spec.extra.update(base)
    cfg.model_spec.plugin_model = ms.pop("plugin_model", None) or {}
    cfg.model_spec.extra.update(ms)
    if cfg.model_spec.model_dir and config_file and not os.path.isabs(cfg.model_spec.model_dir):
        cand = os.path.join(os.path.dirname(os.path.abspath(config_file)), cfg.model_spec.model_dir)
        if os.path.isdir(cand):
            cfg.model_spec.model_dir = cand
    cfg.validate()
    return cfg


def load_serving_config(path: str) -> ServingConfig:
    with open(path, "r", encoding="utf-8") as f:
        raw = yaml.safe_load(f) or {}
    return parse_serving_config(raw, config_file=path)
