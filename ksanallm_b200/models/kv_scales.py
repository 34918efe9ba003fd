"""Per-layer scaling factors for an fp8 KV cache, read from a ``kv_cache_scales.json`` next to the checkpoint.

Format (the one the reference documents in src/ksana_llm/python/kv_scale_files/README.md, shared with vLLM's
quantisation tooling)::

    {"model_type": "llama",
     "kv_cache": {"dtype": "float8_e4m3fn",
                  "scaling_factor": {"<tp_rank>": {"<layer>": <float>, ...}, ...}}}

A file written for one rank ("0") is accepted for every rank. K and V share the factor, as in the reference
(`k_scale == v_scale`); a missing file or layer means 1.0.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional


def find_kv_scales_file(model_dir: str, explicit: str = "") -> Optional[str]:
    for cand in (explicit, os.path.join(model_dir or "", "kv_cache_scales.json")):
        if cand and os.path.isfile(cand):
            return cand
    return None


def load_kv_cache_scales(path: str, tp_rank: int, num_layers: int, expect_model_type: str = "") -> List[float]:
    with open(path) as f:
        doc = json.load(f)
    kv = doc.get("kv_cache", {})
    dtype = str(kv.get("dtype", "float8_e4m3fn"))
    if "e4m3" not in dtype and "e5m2" not in dtype:
        raise ValueError(f"{path}: unsupported kv_cache dtype {dtype!r}")
    if expect_model_type and doc.get("model_type") and doc["model_type"] != expect_model_type:
        raise ValueError(f"{path}: written for model_type {doc['model_type']!r}, loading {expect_model_type!r}")
    table = kv.get("scaling_factor", {})
    per_rank = table.get(str(tp_rank)) or table.get("0") or {}
    out = []
    for layer in range(num_layers):
        v = per_rank.get(str(layer), 1.0)
        v = float(v)
        if not (v > 0.0):
            raise ValueError(f"{path}: scaling factor of layer {layer} must be positive, got {v}")
        out.append(v)
    return out


def apply_kv_scales(model, scales: List[float]) -> None:
    """Sets k/v scales on the attention modules of ``model`` (layer i of the model <- scales[global layer id])."""
    for layer, gid in zip(model.layers, model.layer_ids):
        if hasattr(layer.attn, "k_scale"):
            layer.attn.k_scale = layer.attn.v_scale = scales[gid]
    model.kv_scales = list(scales)
