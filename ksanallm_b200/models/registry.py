"""model_type -> architecture family.

The reference maps ``model_type`` substrings to one C++ model class per family
(src/ksana_llm/runtime/model_instance.cpp:50-145) and falls back to the Llama classes when the model directory
ships a ``<model_type>_weight_map.json``. Here every family is the generic :class:`TransformerModel`; this table
records which families are recognised, their weight-name conventions (models/loader.py) and the features they
switch on in :class:`ModelConfig` (config/model_config.py).
"""
from __future__ import annotations

import os
from typing import Dict, Optional

FAMILIES: Dict[str, str] = {
    "llama": "dense, RoPE (default / linear / dynamic / llama3 / yarn), GQA, SwiGLU",
    "llama4": "interleaved MoE + shared expert, no-rope layers",
    "qwen": "qkv bias, SwiGLU",
    "qwen2": "qkv bias, GQA",
    "qwen3": "per-head QK RMSNorm before RoPE, GQA",
    "qwen2_moe": "softmax top-k MoE, gated shared expert",
    "qwen3_moe": "softmax top-k MoE (renormalised), QK norm",
    "qwen2_vl": "qwen2 text tower + plugin vision embeddings (input_refit_embedding)",
    "baichuan": "packed W_pack qkv; ALiBi for the 13B size",
    "chatglm": "packed qkv with multi-query groups, interleaved partial rotary",
    "glm": "GLM-4 in its transformers layout: separate q/k/v, fused gate_up_proj, interleaved partial rotary",
    "gpt2": "learned positions, LayerNorm, GELU MLP with biases (also fairseq-transformer / openai-gpt)",
    "internlm2": "packed wqkv per KV group",
    "internvl_chat": "internlm2 / qwen2 language tower + vision plugin",
    "internlmxcomposer2": "internlm2 tower + plugin",
    "hunyuan": "MoE with shared MLP, QK norm, cross-layer attention sharing",
    "mixtral": "softmax top-2 MoE (w1 / w2 / w3 expert names)",
    "deepseek_v2": "MLA + group-limited softmax routing + shared experts",
    "deepseek_v3": "MLA + sigmoid routing with correction bias, 8 groups / top-4, MTP layer, fp8 block weights; "
                   "V3.2 / GLM DSA: sparse attention over the keys picked by the indexer",
    "kimi_k2": "deepseek_v3 architecture with 384 experts",
    "minicpm": "embedding / residual / logit scaling; reranker head",
}

_ALIASES = {"fairseq-transformer": "gpt2", "fairseq_transformer": "gpt2", "openai-gpt": "gpt2", "gpt": "gpt2",
            "deepseek_v32": "deepseek_v3", "glm_moe_dsa": "deepseek_v3", "qwen2_5_vl": "qwen2_vl", "arc_hunyuan_video": "hunyuan",
            "hunyuan_turbo": "hunyuan", "hunyuan_large": "hunyuan", "minicpm3": "minicpm", "mistral": "llama",
            "yi": "llama", "vicuna": "llama", "internlm": "llama"}


def resolve_family(model_type: str, model_dir: str = "") -> Optional[str]:
    mt = (model_type or "").lower()
    if mt in FAMILIES:
        return mt
    if mt in _ALIASES:
        return _ALIASES[mt]
    for name in sorted(FAMILIES, key=len, reverse=True):
        if name in mt:
            return name
    if model_dir and os.path.isfile(os.path.join(model_dir, f"{mt}_weight_map.json")):
        return "llama"  # a weight map renames the checkpoint into Llama names
    return None


def is_supported(model_type: str, model_dir: str = "") -> bool:
    return resolve_family(model_type, model_dir) is not None
