"""`/forward` request targets: read intermediate tensors of ONE prefill step.

Schema (reference: src/ksana_llm/cpp/README.md, src/ksana_llm/utils/request_serial.h, validation in
src/ksana_llm/utils/request.cpp:109-201): each target names ``transformer`` (hidden states before the final norm),
``layernorm`` (after it) or ``logits``; rows are selected with ``slice_pos`` = list of inclusive [l, r] intervals
(negative = from the end) or ``token_id`` positions; ``token_reduce_mode`` is ``GATHER_ALL`` (whole rows / all vocab
logits) or ``GATHER_TOKEN_ID`` (logits target only: softmax probability each row assigns to the NEXT input token).

Layer-wise rerankers (bge-reranker-v2-minicpm-layerwise) add the ``lm_head`` target: ``cutoff_layer`` = [n] stops the
decoder after n layers, the final norm and that depth's one-row scoring head ``lm_head.{n - start_layer}.linear_head``
follow, and the scores of all rows are returned (reference: models/bge_reranker_minicpm/bge_reranker_minicpm_model.cpp
:192-217).
"""
from __future__ import annotations

import base64
from typing import Any, Dict, List, Sequence

import numpy as np
import torch

VALID_TARGETS = ("transformer", "layernorm", "logits", "lm_head")


def validate_targets(targets: Sequence[Dict[str, Any]], num_tokens: int) -> None:
    for t in targets:
        name = t.get("target_name")
        if name not in VALID_TARGETS:
            raise ValueError(f"Invalid target name {name}")
        mode = t.get("token_reduce_mode", "GATHER_ALL")
        if mode not in ("GATHER_ALL", "GATHER_TOKEN_ID"):
            raise ValueError(f"Invalid token_reduce_mode {mode}")
        if name == "lm_head" and mode != "GATHER_ALL":
            raise ValueError("the lm_head target returns every row (GATHER_ALL)")
        if mode == "GATHER_TOKEN_ID" and name != "logits":
            raise ValueError("GATHER_TOKEN_ID is only supported for the logits target")
        if t.get("slice_pos") and t.get("token_id"):
            raise ValueError("slice_pos and token_id cannot both be set")
        for iv in t.get("slice_pos") or []:
            if len(iv) != 2:
                raise ValueError("slice_pos entries must be [l, r]")
            l, r = _norm_interval(iv, num_tokens)
            if l > r or l < 0 or r >= num_tokens:
                raise ValueError(f"slice_pos {iv} out of range for {num_tokens} tokens")


def _norm_interval(iv, n):
    l, r = int(iv[0]), int(iv[1])
    if l < 0:
        l += n
    if r < 0:
        r += n
    return l, r


def _rows(target: Dict[str, Any], n: int) -> List[int]:
    rows: List[int] = []
    if target.get("slice_pos"):
        last = -1
        for iv in target["slice_pos"]:
            l, r = _norm_interval(iv, n)
            if l <= last:
                raise ValueError("slice_pos intervals must be increasing and disjoint")
            rows.extend(range(l, r + 1))
            last = r
    elif target.get("token_id"):
        rows = [int(p) if int(p) >= 0 else int(p) + n for p in target["token_id"]]
    else:
        rows = [n - 1]
    return rows


def _encode(t: torch.Tensor) -> Dict[str, Any]:
    a = t.detach().float().cpu().contiguous().numpy().astype(np.float32)
    return {"data": base64.b64encode(a.tobytes()).decode("ascii"), "shape": list(a.shape), "dtype": "float32"}


def reranker_scores(model, cutoff_hidden: torch.Tensor, cutoff_layer: int) -> torch.Tensor:
    """cutoff_hidden: final-norm output after ``cutoff_layer`` decoder layers [n, H] -> scores [n, 1]."""
    start = int(getattr(model.cfg, "reranker_start_layer", 0) or 0)
    w = model.w.get(f"lm_head.{cutoff_layer - start}.linear_head.weight")
    if w is None or cutoff_layer < start:
        raise ValueError(f"no scoring head for cutoff_layer {cutoff_layer}")
    return cutoff_hidden.float() @ w.float().t()


def run_probe(model, targets, hidden: torch.Tensor, prenorm: torch.Tensor, tokens: Sequence[int],
              cutoff_forward=None) -> List[Dict[str, Any]]:
    """hidden: final-norm output rows of this request [n, H]; prenorm: residual stream rows [n, H];
    ``cutoff_forward(n_layers)`` -> final-norm output of this request after n_layers decoder layers."""
    n = hidden.shape[0]
    out = []
    for t in targets:
        name = t["target_name"]
        if name == "lm_head":
            depth = max(int(c) for c in (t.get("cutoff_layer") or [len(model.layers)]))
            out.append({"target_name": name, "tensor": _encode(reranker_scores(model, cutoff_forward(depth), depth))})
            continue
        rows = _rows(t, n)
        idx = torch.tensor(rows, device=hidden.device, dtype=torch.long)
        if name == "transformer":
            res = prenorm.index_select(0, idx)
        elif name == "layernorm":
            res = hidden.index_select(0, idx)
        else:
            logits = model.compute_logits(hidden.index_select(0, idx))
            if t.get("token_reduce_mode", "GATHER_ALL") == "GATHER_TOKEN_ID":
                probs = torch.softmax(logits, dim=-1)
                nxt = torch.tensor([tokens[min(r + 1, len(tokens) - 1)] for r in rows], device=hidden.device)
                res = probs.gather(1, nxt.unsqueeze(1)).squeeze(1)
            else:
                res = logits
            k = int(t.get("input_top_logprobs_num", 0) or 0)
            if k > 0:
                lp = torch.log_softmax(logits, dim=-1).topk(k, dim=-1)
                out.append({"target_name": name, "tensor": _encode(res),
                            "top_logprobs": {"ids": lp.indices.tolist(), "values": lp.values.tolist()}})
                continue
        out.append({"target_name": name, "tensor": _encode(res)})
    return out
