"""HF ``config.json`` -> ModelConfig.

One normalised description for every supported architecture family (dense Llama-like, Qwen
variants, MoE variants, DeepSeek MLA+MoE, GPT-style post-norm, ChatGLM, Baichuan, InternLM2 ...).
Reference: src/ksana_llm/utils/config/model_config_parser.cpp (field extraction and
``quantization_config`` parsing, :75-113), model_config.h:222-327 (fields), and the
model-type dispatch of src/ksana_llm/runtime/model_instance.cpp:50-145.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class RopeScaling:
    type: str = "default"  # default | linear | dynamic | llama3 | yarn | mrope | internlm2_dynamic
    factor: float = 1.0
    original_max_position_embeddings: int = 0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0
    mrope_section: List[int] = field(default_factory=list)
    alpha: float = 0.0  # dynamic-NTK "alpha" flavour


@dataclass
class QuantConfig:
    method: str = "none"  # none | fp8 | fp8_block | gptq | awq | w4a8_awq
    bits: int = 16
    group_size: int = 128
    desc_act: bool = False
    weight_block_size: List[int] = field(default_factory=list)  # [128, 128] for block-scaled fp8
    zero_point: bool = False
    modules_to_not_convert: List[str] = field(default_factory=list)


@dataclass
class ModelConfig:
    model_type: str = "llama"
    architectures: List[str] = field(default_factory=list)
    vocab_size: int = 32000
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 32
    head_dim: int = 128
    intermediate_size: int = 11008
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    rope_interleaved: bool = False  # GPT-J style pairs instead of neox halves
    rotary_dim: int = 0  # 0 = full head_dim
    position_encoding: str = "rope"  # rope | alibi | learned | none
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    norm_type: str = "rmsnorm"  # rmsnorm | layernorm
    post_norm: bool = False  # GPT-style
    qkv_bias: bool = False
    o_bias: bool = False
    mlp_bias: bool = False
    gated_mlp: bool = True
    qk_norm: bool = False  # per-head RMSNorm on q and k before RoPE (Qwen3)
    cla_share_factor: int = 0  # cross-layer attention: K/V projections shared by groups of this many layers (Hunyuan)
    qk_norm_after_rope: bool = False  # ... applied after RoPE instead (Hunyuan)
    sliding_window: int = 0  # attention window in tokens (0: full causal); per layer via sliding_layers
    sliding_layers: List[int] = field(default_factory=list)  # 1 = windowed layer; empty with a window: every layer
    qk_l2_norm: bool = False  # weightless RMS normalisation of q and k after RoPE on the RoPE layers (Llama 4)
    rope_layers: List[int] = field(default_factory=list)  # per layer: 1 = RoPE, 0 = no position encoding (Llama 4)
    moe_layers: List[int] = field(default_factory=list)   # explicit MoE layer indices (Llama 4); empty: by frequency
    moe_router: str = "standard"  # standard | llama4 (top-k on logits, sigmoid score scales the expert INPUT)
    attn_temperature_tuning: bool = False  # Llama 4: query scaling on the no-RoPE layers
    attention_chunk_size: int = 0  # Llama 4: RoPE layers attend inside blocks of this many positions (0 = off)
    attn_floor_scale: float = 8192.0
    attn_scale_coef: float = 0.1
    bos_token_id: Optional[int] = None
    eos_token_ids: List[int] = field(default_factory=list)
    pad_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    emb_scale: float = 1.0
    logit_scale: float = 1.0
    residual_scale: float = 1.0
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    num_shared_experts: int = 0
    shared_expert_intermediate_size: int = 0
    shared_expert_gate: bool = False
    first_k_dense_replace: int = 0
    moe_layer_freq: int = 1
    norm_topk_prob: bool = False
    scoring_func: str = "softmax"  # softmax | sigmoid
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    topk_method: str = "greedy"  # greedy | group_limited_greedy | noaux_tc
    # MLA
    use_mla: bool = False
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # MTP
    # sparse attention indexer (DeepSeek-V3.2, GLM DSA): every query keeps the index_topk best-scoring keys
    mla_norm_eps: float = 0.0  # epsilon of the low-rank q / kv norms when it differs from rms_norm_eps (0: same)
    index_topk: int = 0
    index_n_heads: int = 0
    index_head_dim: int = 0
    num_nextn_predict_layers: int = 0
    reranker_start_layer: int = 0  # layer-wise reranker: depth of the first scoring head lm_head.0.linear_head
    num_register_token: int = 0  # parallel token prediction: register tokens appended per step (0 = off)
    reg_token_id: int = 0
    # quantisation
    quant: QuantConfig = field(default_factory=QuantConfig)
    raw: Dict[str, Any] = field(default_factory=dict)

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def is_moe_layer(self, layer_idx: int) -> bool:
        if not self.is_moe:
            return False
        if self.moe_layers:
            return layer_idx in self.moe_layers
        return layer_idx >= self.first_k_dense_replace and (layer_idx % max(self.moe_layer_freq, 1) == 0)

    @property
    def q_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim if self.use_mla else self.head_dim


def _rope_scaling(d: Optional[Dict[str, Any]], cfg: Dict[str, Any]) -> RopeScaling:
    rs = RopeScaling()
    if not d:
        return rs
    t = d.get("rope_type", d.get("type", "default")) or "default"
    rs.type = {"ntk": "dynamic", "dynamic_ntk": "dynamic", "deepseek_yarn": "yarn", "mrope": "default"}.get(t, t)
    rs.factor = float(d.get("factor", 1.0) or 1.0)
    rs.original_max_position_embeddings = int(
        d.get("original_max_position_embeddings", cfg.get("max_position_embeddings", 0)) or 0)
    rs.low_freq_factor = float(d.get("low_freq_factor", 1.0))
    rs.high_freq_factor = float(d.get("high_freq_factor", 4.0))
    rs.beta_fast = float(d.get("beta_fast", 32.0))
    rs.beta_slow = float(d.get("beta_slow", 1.0))
    rs.mscale = float(d.get("mscale", 1.0))
    rs.mscale_all_dim = float(d.get("mscale_all_dim", 0.0))
    rs.mrope_section = list(d.get("mrope_section", []) or [])
    rs.alpha = float(d.get("alpha", 0.0) or 0.0)
    return rs


def _quant(d: Optional[Dict[str, Any]]) -> QuantConfig:
    q = QuantConfig()
    if not d:
        return q
    method = str(d.get("quant_method", d.get("quant_algo", "none"))).lower()
    if method == "fp8":
        wbs = d.get("weight_block_size")
        if wbs:
            q.method, q.weight_block_size, q.bits = "fp8_block", [int(x) for x in wbs], 8
        else:
            q.method, q.bits = "fp8", 8
    elif method in ("gptq", "awq"):
        q.method = method
        q.bits = int(d.get("bits", d.get("w_bit", 4)))
        q.group_size = int(d.get("group_size", d.get("q_group_size", 128)))
        q.desc_act = bool(d.get("desc_act", False))
        q.zero_point = bool(d.get("zero_point", method == "awq"))
    elif method in ("w4a8_awq", "mixed", "modelopt", "rtn"):
        q.method = method
        q.bits = int(d.get("bits", 4))
        q.group_size = int(d.get("group_size", 128))
    else:
        q.method = method
    q.modules_to_not_convert = list(d.get("modules_to_not_convert", []) or [])
    return q


def model_config_from_dict(c: Dict[str, Any]) -> ModelConfig:
    if isinstance(c.get("text_config"), dict) and str(c.get("model_type", "")).lower() in ("llama4",):
        # multimodal wrapper configs keep the language model under "text_config"
        inner = dict(c["text_config"])
        inner.setdefault("model_type", "llama4_text")
        for k in ("torch_dtype", "dtype", "quantization_config"):
            if k in c and k not in inner:
                inner[k] = c[k]
        c = inner
    if isinstance(c.get("text_config"), dict) and str(c.get("model_type", "")).lower() in ("qwen2_vl", "qwen2_5_vl",
                                                                                              "internvl"):
        inner = dict(c["text_config"])
        if str(c["model_type"]).lower() != "internvl":  # InternVL's tower keeps its own type (qwen2, llama, ...)
            inner["model_type"] = str(c["model_type"]).lower()
        for k in ("torch_dtype", "dtype", "quantization_config", "tie_word_embeddings", "architectures"):
            if k in c and k not in inner:
                inner[k] = c[k]
        c = inner
    mt = str(c.get("model_type", "llama")).lower()
    m = ModelConfig(model_type=mt, architectures=list(c.get("architectures", []) or []), raw=c)
    g = c.get
    m.vocab_size = int(g("vocab_size", g("padded_vocab_size", 32000)))
    m.hidden_size = int(g("hidden_size", g("n_embd", g("d_model", 4096))))
    m.num_layers = int(g("num_hidden_layers", g("n_layer", g("num_layers", 32))))
    m.num_heads = int(g("num_attention_heads", g("n_head", 32)))
    kv = g("num_key_value_heads", None)
    if kv is None:
        if g("multi_query_attention", False):
            kv = g("multi_query_group_num", 1)
        else:
            kv = g("num_kv_heads", m.num_heads)
    m.num_kv_heads = int(kv)
    m.head_dim = int(g("head_dim", None) or g("kv_channels", None) or (m.hidden_size // m.num_heads))
    m.intermediate_size = int(g("intermediate_size", g("ffn_hidden_size", g("n_inner", None) or 4 * m.hidden_size)))
    m.max_position_embeddings = int(g("max_position_embeddings", g("n_positions", g("seq_length", 4096))))
    m.rms_norm_eps = float(g("rms_norm_eps", g("layer_norm_epsilon", g("layernorm_epsilon", g("layer_norm_eps", 1e-6)))))
    # transformers >= 5 folds rope_theta and the scaling block into one "rope_parameters" dict
    rp = g("rope_parameters", None) or {}
    m.rope_theta = float(g("rope_theta", None) or rp.get("rope_theta", None) or g("rotary_emb_base", 10000.0))
    rs_dict = g("rope_scaling", None)
    if rs_dict is None and rp and (str(rp.get("rope_type", rp.get("type", "default"))) != "default" or
                                   rp.get("mrope_section")):
        rs_dict = rp
    m.rope_scaling = _rope_scaling(rs_dict, c)
    xd = g("xdrope_section", None)
    if xd and g("position_embedding_xdrope", True):
        # XD-RoPE (Arc-Hunyuan-Video): four position axes, sections given as fractions of half the head size; the
        # table itself is the alpha-scaled NTK one (reference: arc_hunyuan_video_config_parser.cpp:72-93,
        # rotary_embedding.cu:361-372)
        half = (m.head_dim or m.hidden_size // m.num_heads) // 2
        m.rope_scaling.mrope_section = [int(float(f) * half) for f in xd]
        if m.rope_scaling.type in ("default", "xdrope"):
            m.rope_scaling.type = "dynamic"
            m.rope_scaling.alpha = float((rs_dict or {}).get("alpha", 1000.0))
    m.tie_word_embeddings = bool(g("tie_word_embeddings", False))
    m.hidden_act = str(g("hidden_act", g("activation_function", "silu")))
    m.torch_dtype = str(g("torch_dtype", g("dtype", "bfloat16")))
    m.bos_token_id = g("bos_token_id", None)
    eos = g("eos_token_id", None)
    m.eos_token_ids = [int(e) for e in eos] if isinstance(eos, (list, tuple)) else ([int(eos)] if eos is not None else [])
    m.pad_token_id = g("pad_token_id", None)
    m.qkv_bias = bool(g("attention_bias", g("qkv_bias", g("add_qkv_bias", False))))
    m.mlp_bias = bool(g("mlp_bias", False))
    sw = g("sliding_window", None)
    if sw and g("use_sliding_window", True):
        m.sliding_window = int(sw)
        lt = g("layer_types", None)
        if lt:
            m.sliding_layers = [1 if str(t) == "sliding_attention" else 0 for t in lt]

    if mt in ("qwen2", "qwen2_moe", "qwen", "qwen2_vl", "qwen2_5_vl"):
        m.qkv_bias = True if g("attention_bias", None) is None else bool(g("attention_bias"))
    if mt in ("qwen3", "qwen3_moe"):
        m.qk_norm = True
        m.qkv_bias = bool(g("attention_bias", False))
    if mt.startswith("hunyuan"):
        m.qk_norm = bool(g("use_qk_norm", True))
        m.qk_norm_after_rope = m.qk_norm
        if g("use_cla", False):
            m.cla_share_factor = int(g("cla_share_factor", 0) or 0)
    if mt.startswith("llama4"):
        m.rope_interleaved = True
        m.qk_l2_norm = bool(g("use_qk_norm", True))
        m.rope_layers = [int(x) for x in (g("no_rope_layers", None) or [])]
        m.attn_temperature_tuning = bool(g("attn_temperature_tuning", False))
        m.attn_floor_scale = float(g("floor_scale", 8192))
        m.attention_chunk_size = int(g("attention_chunk_size", 0) or 0)
        m.attn_scale_coef = float(g("attn_scale", 0.1))
    if mt in ("gpt2", "fairseq_transformer", "gpt"):
        m.norm_type, m.post_norm, m.gated_mlp, m.position_encoding = "layernorm", False, False, "learned"
        m.qkv_bias = m.o_bias = m.mlp_bias = True
        m.hidden_act = str(g("activation_function", "gelu_new"))
        m.tie_word_embeddings = bool(g("tie_word_embeddings", True))
    if mt == "baichuan":
        # Baichuan-13B (hidden 5120) uses ALiBi, 7B uses RoPE
        if m.hidden_size >= 5120:
            m.position_encoding = "alibi"
    if mt == "chatglm":
        m.rope_interleaved = True
        m.rotary_dim = m.head_dim // 2
        m.qkv_bias = bool(g("add_qkv_bias", True))
        m.rope_theta = 10000.0 * float(g("rope_ratio", 1.0))
    if mt in ("glm", "glm4"):
        # the HF port of GLM-4: interleaved rotary pairs on a fraction of the head, fused gate_up_proj
        m.rope_interleaved = True
        prf = float(g("partial_rotary_factor", None) or rp.get("partial_rotary_factor", 0.5) or 0.5)
        m.rotary_dim = int(m.head_dim * prf)
        m.qkv_bias = bool(g("attention_bias", True))
    if mt in ("internlm2", "internvl_chat", "internlmxcomposer2"):
        m.qkv_bias = bool(g("bias", False))
    if mt in ("minicpm", "minicpm3"):
        m.emb_scale = float(g("scale_emb", 1.0))
        depth = float(g("scale_depth", 1.0))
        m.residual_scale = depth / (m.num_layers ** 0.5) if depth != 1.0 else 1.0
        dmb = float(g("dim_model_base", m.hidden_size))
        m.logit_scale = dmb / m.hidden_size

    # ---- MoE ------------------------------------------------------------------------------
    ne = g("num_experts", None) or g("num_local_experts", None) or g("n_routed_experts", None) or 0
    if isinstance(ne, (list, tuple)):
        ne = ne[0] if ne else 0
    m.num_experts = int(ne or 0)
    if m.num_experts:
        m.num_experts_per_tok = int(g("num_experts_per_tok", g("moe_topk", 2)))
        mis = g("moe_intermediate_size", m.intermediate_size)
        m.moe_intermediate_size = int(mis[0] if isinstance(mis, (list, tuple)) else mis)
        m.norm_topk_prob = bool(g("norm_topk_prob", mt == "mixtral"))
        m.num_shared_experts = int(g("n_shared_experts", 0) or 0)
        sei = g("shared_expert_intermediate_size", 0) or 0
        if sei:
            m.num_shared_experts = max(m.num_shared_experts, 1)
            m.shared_expert_intermediate_size = int(sei)
            m.shared_expert_gate = mt == "qwen2_moe"
        elif m.num_shared_experts:
            m.shared_expert_intermediate_size = m.moe_intermediate_size * m.num_shared_experts
        m.first_k_dense_replace = int(g("first_k_dense_replace", 0) or 0)
        m.moe_layer_freq = int(g("moe_layer_freq", g("decoder_sparse_step", 1)) or 1)
        v3_like = mt in ("deepseek_v3", "deepseek_v32", "kimi_k2", "glm_moe_dsa")  # sigmoid routing even when the field is absent
        m.scoring_func = str(g("scoring_func", "sigmoid" if v3_like else "softmax"))
        m.n_group = int(g("n_group", 1) or 1)
        m.topk_group = int(g("topk_group", 1) or 1)
        m.routed_scaling_factor = float(g("routed_scaling_factor", 1.0) or 1.0)
        m.topk_method = str(g("topk_method", "noaux_tc" if v3_like else "greedy"))
        if mt.startswith("llama4"):
            # experts use intermediate_size, the dense layers and nothing else intermediate_size_mlp
            m.moe_intermediate_size = int(g("intermediate_size", m.moe_intermediate_size))
            m.intermediate_size = int(g("intermediate_size_mlp", m.intermediate_size))
            m.num_shared_experts, m.shared_expert_intermediate_size = 1, m.moe_intermediate_size
            m.moe_router = "llama4"
            ml = g("moe_layers", None)
            step = int(g("interleave_moe_layer_step", 1) or 1)
            m.moe_layers = [int(x) for x in ml] if ml is not None else list(range(step - 1, m.num_layers, step))
        mlt = g("mlp_layer_types", None)
        if mlt:  # explicit per-layer list of "dense" / "sparse" (GLM MoE)
            m.moe_layers = [i for i, t in enumerate(mlt) if str(t) == "sparse"]
            m.first_k_dense_replace = 0
        if mt.startswith("hunyuan"):
            tk = g("moe_topk", m.num_experts_per_tok)
            m.num_experts_per_tok = int(tk[0] if isinstance(tk, (list, tuple)) else tk)
            ne_ = g("num_experts", m.num_experts)
            m.num_experts = int(ne_[0] if isinstance(ne_, (list, tuple)) else ne_)
            m.moe_intermediate_size = m.intermediate_size  # the experts are full-width MLPs
            nse = g("num_shared_expert", 1)
            m.num_shared_experts = int(nse[0] if isinstance(nse, (list, tuple)) else nse) or 1
            m.shared_expert_intermediate_size = m.intermediate_size * m.num_shared_experts
            m.norm_topk_prob = True

    # ---- MLA ------------------------------------------------------------------------------
    if g("kv_lora_rank", None):
        m.use_mla = True
        m.q_lora_rank = int(g("q_lora_rank", 0) or 0)
        m.kv_lora_rank = int(g("kv_lora_rank"))
        m.qk_nope_head_dim = int(g("qk_nope_head_dim", 128))
        m.qk_rope_head_dim = int(g("qk_rope_head_dim", 64))
        m.v_head_dim = int(g("v_head_dim", 128))
        m.num_kv_heads = 1
        m.rope_interleaved = bool(g("rope_interleave", mt != "glm_moe_dsa"))
        if mt == "glm_moe_dsa":
            m.mla_norm_eps = 1e-6  # the transformers implementation keeps the default there
        if g("index_topk", None) and (mt in ("deepseek_v32", "glm_moe_dsa") or g("index_n_heads", None)):
            m.index_topk = int(g("index_topk"))
            m.index_n_heads = int(g("index_n_heads", 64))
            m.index_head_dim = int(g("index_head_dim", 128))
    m.num_nextn_predict_layers = int(g("num_nextn_predict_layers", 0) or 0)
    if g("start_layer", None) is not None:  # reference: models/bge_reranker_minicpm/bge_reranker_minicpm_config.h:19
        m.reranker_start_layer = int(g("start_layer"))
    m.num_register_token = int(g("num_register_token", 0) or 0)  # reference: models/common/common_config.h:36-37
    m.reg_token_id = int(g("reg_token_id", 0) or 0)
    m.quant = _quant(g("quantization_config", None))
    return m


def load_model_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    # ModelOpt / TensorRT-LLM exports describe their quantisation in hf_quant_config.json:
    # {"quantization": {"quant_algo": "W4A8_AWQ", "group_size": 128, ...}}
    # (reference: utils/config/quant_config_parser.cpp:52-60)
    hq = os.path.join(model_dir, "hf_quant_config.json")
    if "quantization_config" not in raw and os.path.isfile(hq):
        with open(hq, "r", encoding="utf-8") as f:
            qd = json.load(f).get("quantization") or {}
        if qd.get("quant_algo"):
            raw["quantization_config"] = dict(qd, modules_to_not_convert=qd.get("exclude_modules") or [])
    cfg = model_config_from_dict(raw)
    # generation_config.json may name further end-of-sequence ids (Llama 3: <|eot_id|> next to <|end_of_text|>);
    # the reference adds them to every request's stop ids (python/ksana_llm/processor_op_base.py:74-90)
    gen = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(gen):
        try:
            with open(gen, "r", encoding="utf-8") as f:
                eos = json.load(f).get("eos_token_id")
        except (OSError, ValueError):
            eos = None
        extra = eos if isinstance(eos, (list, tuple)) else ([eos] if eos is not None else [])
        for t in extra:
            if int(t) not in cfg.eos_token_ids:
                cfg.eos_token_ids.append(int(t))
    return cfg


# ---- named synthetic configurations used by benchmarks and tests ---------------------------------

def tiny_llama_config() -> ModelConfig:
    return model_config_from_dict(dict(
        model_type="llama", hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
        intermediate_size=688, rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=32000,
        max_position_embeddings=2048, torch_dtype="float32", eos_token_id=2, bos_token_id=1))


def llama2_7b_config() -> ModelConfig:
    return model_config_from_dict(dict(
        model_type="llama", hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=32,
        intermediate_size=11008, rms_norm_eps=1e-5, rope_theta=10000.0, vocab_size=32000,
        max_position_embeddings=4096, torch_dtype="bfloat16", eos_token_id=2, bos_token_id=1))


def llama3_70b_config() -> ModelConfig:
    return model_config_from_dict(dict(
        model_type="llama", hidden_size=8192, num_hidden_layers=80, num_attention_heads=64, num_key_value_heads=8,
        intermediate_size=28672, rms_norm_eps=1e-5, rope_theta=500000.0, vocab_size=128256,
        max_position_embeddings=8192, torch_dtype="bfloat16", eos_token_id=128001, bos_token_id=128000))


def qwen3_32b_config(fp8_block: bool = True) -> ModelConfig:
    d = dict(model_type="qwen3", hidden_size=5120, num_hidden_layers=64, num_attention_heads=64,
             num_key_value_heads=8, head_dim=128, intermediate_size=25600, rms_norm_eps=1e-6, rope_theta=1000000.0,
             vocab_size=151936, max_position_embeddings=40960, torch_dtype="bfloat16", eos_token_id=151645)
    if fp8_block:
        d["quantization_config"] = dict(quant_method="fp8", weight_block_size=[128, 128], activation_scheme="dynamic")
    return model_config_from_dict(d)


def deepseek_v3_config(num_layers: int = 61, fp8_block: bool = True) -> ModelConfig:
    d = dict(model_type="deepseek_v3", hidden_size=7168, num_hidden_layers=num_layers, num_attention_heads=128,
             num_key_value_heads=128, intermediate_size=18432, moe_intermediate_size=2048, n_routed_experts=256,
             n_shared_experts=1, num_experts_per_tok=8, first_k_dense_replace=3, n_group=8, topk_group=4,
             scoring_func="sigmoid", topk_method="noaux_tc", norm_topk_prob=True, routed_scaling_factor=2.5,
             q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
             rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=129280, max_position_embeddings=163840,
             num_nextn_predict_layers=1, torch_dtype="bfloat16", eos_token_id=1,
             rope_scaling=dict(type="yarn", factor=40, original_max_position_embeddings=4096, beta_fast=32,
                               beta_slow=1, mscale=1.0, mscale_all_dim=1.0))
    if fp8_block:
        d["quantization_config"] = dict(quant_method="fp8", weight_block_size=[128, 128], activation_scheme="dynamic")
    return model_config_from_dict(d)


def tiny_moe_config() -> ModelConfig:
    return model_config_from_dict(dict(
        model_type="mixtral", hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        intermediate_size=96, num_local_experts=4, num_experts_per_tok=2, vocab_size=32000, rms_norm_eps=1e-6,
        max_position_embeddings=2048, torch_dtype="float32", eos_token_id=2, bos_token_id=1))


def tiny_moe_128_config() -> ModelConfig:
    """A small MoE whose shapes the CUDA kernels take (head_dim 128, hidden and expert widths multiples of 128)."""
    return model_config_from_dict(dict(
        model_type="mixtral", hidden_size=256, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=2,
        head_dim=128, intermediate_size=128, num_local_experts=4, num_experts_per_tok=2, vocab_size=32000,
        rms_norm_eps=1e-6, max_position_embeddings=2048, torch_dtype="bfloat16", eos_token_id=2, bos_token_id=1))


NAMED_CONFIGS = {
    "tiny-llama": tiny_llama_config,
    "tiny-moe": tiny_moe_config,
    "tiny-moe-128": tiny_moe_128_config,
    "llama-2-7b": llama2_7b_config,
    "llama-3-70b": llama3_70b_config,
    "qwen3-32b-fp8": qwen3_32b_config,
    "deepseek-v3-fp8": deepseek_v3_config,
}
