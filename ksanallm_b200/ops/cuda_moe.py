"""MoE routing and expert computation on the GPU."""
from __future__ import annotations

import torch

from . import reference as ref


def moe_route(logits, top_k, scoring="softmax", norm_topk=False, n_group=1, topk_group=1, routed_scale=1.0,
              correction_bias=None):
    return ref.moe_route(logits, top_k, scoring, norm_topk, n_group, topk_group, routed_scale, correction_bias)


def moe_experts(x, ids, weights, w_gate_up, w_down, expert_offset=0):
    """Tokens are sorted by expert once; each local expert with work runs two tcgen05 GEMMs on its slice."""
    from . import cuda
    T, H = x.shape
    E_local = w_gate_up.shape[0]
    k = ids.shape[1]
    flat = ids.reshape(-1).long() - expert_offset
    local = (flat >= 0) & (flat < E_local)
    order = torch.argsort(torch.where(local, flat, torch.full_like(flat, E_local)), stable=True)
    counts = torch.bincount(flat[local], minlength=E_local).tolist()
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    tok_of = order // k
    wflat = weights.reshape(-1)
    start = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        sel = order[start:start + n]
        tok = tok_of[start:start + n]
        start += n
        h = cuda.gemm_bf16(x.index_select(0, tok), w_gate_up[e])
        a = cuda.silu_and_mul(h)
        y = cuda.gemm_bf16(a, w_down[e]).float()
        out.index_add_(0, tok, y * wflat[sel].unsqueeze(-1))
    return out.to(x.dtype)
