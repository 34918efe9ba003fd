"""Per-shape GEMM launch parameters found by an offline sweep.

The reference searches cuBLASLt algorithms offline and loads ``gemm_algo_map.yaml`` at start-up
(3rdparty/LLM_kernels/.../search_best_gemm_algo, src/ksana_llm/utils/gemm_algo_map). The tcgen05 GEMM here has two
knobs - tile width (64 / 128 / 256) and split-K factor (positive: cluster split-K, negative: workspace split-K) - with
a built-in heuristic; a map written by ``benchmarks/search_best_gemm.py`` overrides it for the shapes it lists.

File format (YAML)::

    gemm_bf16:
      - {n: 12288, k: 4096, m_max: 64, bn: 128, splits: 4}
      - {n: 12288, k: 4096, m_max: 512, bn: 256, splits: 0}

An entry applies to M <= m_max (first match in ascending m_max order for its (n, k)).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

_MAP: Dict[Tuple[int, int], List[Tuple[int, int, int]]] = {}
_loaded_from: Optional[str] = None


def load_map(path: str) -> int:
    """Loads (replaces) the tuning map; returns the number of entries."""
    import yaml
    global _loaded_from
    with open(path) as f:
        doc = yaml.safe_load(f) or {}
    _MAP.clear()
    n = 0
    for e in doc.get("gemm_bf16", []) or []:
        key = (int(e["n"]), int(e["k"]))
        _MAP.setdefault(key, []).append((int(e["m_max"]), int(e.get("bn", 0)), int(e.get("splits", 0))))
        n += 1
    for v in _MAP.values():
        v.sort()
    _loaded_from = path
    return n


def maybe_load_from_env() -> None:
    path = os.environ.get("KSANA_GEMM_TUNE_FILE", "")
    if path and _loaded_from != path and os.path.isfile(path):
        load_map(path)


def lookup(m: int, n: int, k: int) -> Tuple[int, int]:
    """(bn, splits) for this shape, (0, 0) = use the built-in heuristic."""
    rows = _MAP.get((n, k))
    if not rows:
        return 0, 0
    for m_max, bn, splits in rows:
        if m <= m_max:
            return bn, splits
    return 0, 0


def clear() -> None:
    global _loaded_from
    _MAP.clear()
    _loaded_from = None
