"""Per-rank processed-weight cache: ``ENABLE_MODEL_CACHE=1 MODEL_CACHE_PATH=dir`` saves the canonical, already
sliced / fused / quantised tensors of each rank as safetensors and reloads them at the next start instead of
re-running the loader (reference: src/ksana_llm/runtime/weight_instance.cpp:230-240,
utils/safetensors_file_saver.cpp)."""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch


def cache_file(model_dir: str, tp_rank: int, tp_size: int, tag: str = "") -> Optional[str]:
    if os.environ.get("ENABLE_MODEL_CACHE", "0") != "1":
        return None
    root = os.environ.get("MODEL_CACHE_PATH") or os.path.join(model_dir or ".", ".ksana_model_cache")
    os.makedirs(root, exist_ok=True)
    return os.path.join(root, f"rank{tp_rank}of{tp_size}{('_' + tag) if tag else ''}.safetensors")


def save_weights(path: str, weights: Dict[str, torch.Tensor]) -> None:
    from safetensors.torch import save_file
    flat = {}
    for k, v in weights.items():
        t = v.detach().to("cpu").contiguous()
        if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            flat[k + "::" + str(t.dtype).split(".")[-1]] = t.view(torch.uint8)
        else:
            flat[k] = t
    save_file(flat, path)


def load_weights(path: str, device="cpu") -> Dict[str, torch.Tensor]:
    from safetensors import safe_open
    out = {}
    with safe_open(path, framework="pt", device="cpu") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            if "::" in k:
                name, dt = k.split("::")
                out[name] = t.view(getattr(torch, dt)).to(device)
            else:
                out[k] = t.to(device)
    return out
