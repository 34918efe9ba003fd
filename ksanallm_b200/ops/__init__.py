"""Operator front door.

CUDA tensors go to the hand-written sm_100a kernels (``ops.cuda``; a missing kernel library on a GPU
box is an error, never a silent fallback). CPU tensors go to the fp32 PyTorch restatements in
``ops.reference`` that also serve as the kernels' test oracle.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import reference as ref


def _cuda():
    from . import cuda as _c
    return _c


def rms_norm(x, weight, eps, residual=None):
    if x.is_cuda:
        return _cuda().rms_norm(x, weight, eps, residual)
    return ref.rms_norm(x, weight, eps, residual)


def layer_norm(x, weight, bias, eps, residual=None):
    return ref.layer_norm(x, weight, bias, eps, residual)


def _library_baseline() -> bool:
    """KSANA_LIBRARY_BASELINE=1 routes dense GEMMs to cuBLAS (torch.matmul): the measured stand-in for the
    reference's cuBLAS + NCCL build, never the default."""
    import os
    return os.environ.get("KSANA_LIBRARY_BASELINE", "0") == "1"


def linear(x, weight, bias=None):
    if x.is_cuda:
        if _library_baseline():
            return torch.nn.functional.linear(x, weight, bias)
        return _cuda().linear(x, weight, bias)
    return ref.linear(x, weight, bias)


def linear_fp8_block(x, wq, w_scale_inv, bias=None, sfb=None, pow2=False):
    """``pow2``: the weight's block scales are powers of two; the activations then get power-of-two group scales
    too and (CUDA, ``sfb`` = the packed scale bytes) large products run on the scaled tensor-core path."""
    if x.is_cuda:
        return _cuda().linear_fp8_block(x, wq, w_scale_inv, bias, sfb, pow2)
    return ref.linear_fp8_block(x, wq, w_scale_inv, bias, ue8m0=pow2)


def linear_int4(x, packed, scales, zeros, bias=None, group=128, sz=None):
    if x.is_cuda:
        return _cuda().linear_int4(x, packed, scales, zeros, bias, group, sz=sz)
    return ref.linear_int4(x, packed, scales, zeros, bias, group)


def silu_and_mul(x):
    if x.is_cuda:
        return _cuda().silu_and_mul(x)
    return ref.silu_and_mul(x)


def activation(x, kind):
    return ref.activation(x, kind)


def embedding(ids, table, scale=1.0):
    if ids.is_cuda:
        return _cuda().embedding(ids, table, scale)
    return ref.embedding(ids, table, scale)


def rope_qknorm_cache(q, k, v, positions, cos_sin, slot_mapping, kv_cache, q_norm_w=None, k_norm_w=None,
                      eps=1e-6, interleaved=False, rotary_dim=0, k_scale=1.0, v_scale=1.0, norm_after_rope=False):
    if norm_after_rope and q_norm_w is not None:
        # the fused kernel normalises before rotating: this order goes through the reference implementation
        return ref.rope_qknorm_cache(q, k, v, positions, cos_sin, slot_mapping, kv_cache, q_norm_w, k_norm_w, eps,
                                     interleaved, rotary_dim, k_scale, v_scale, True)
    if q.is_cuda:
        return _cuda().rope_qknorm_cache(q, k, v, positions, cos_sin, slot_mapping, kv_cache, q_norm_w, k_norm_w,
                                         eps, interleaved, rotary_dim, k_scale, v_scale)
    return ref.rope_qknorm_cache(q, k, v, positions, cos_sin, slot_mapping, kv_cache, q_norm_w, k_norm_w,
                                 eps, interleaved, rotary_dim, k_scale, v_scale)


def paged_attention(q, kv_cache, meta, scale, alibi_slopes=None, k_scale=1.0, v_scale=1.0, window=0):
    """``meta`` is the step's :class:`~ksanallm_b200.engine.step_input.StepInput`."""
    if q.is_cuda:
        return _cuda().paged_attention(q, kv_cache, meta, scale, alibi_slopes, k_scale, v_scale, window)
    return ref.paged_attention(q, kv_cache, meta.block_tables, meta.cu_q, meta.kv_lens, scale, alibi_slopes,
                               k_scale, v_scale, window)


def mla_cache_append(latent, k_rope, slot_mapping, cache):
    if latent.is_cuda:
        return _cuda().mla_cache_append(latent, k_rope, slot_mapping, cache)
    return ref.mla_cache_append(latent, k_rope, slot_mapping, cache)


def mla_paged_attention(q_latent, q_rope, cache, meta, scale):
    if q_latent.is_cuda:
        return _cuda().mla_paged_attention(q_latent, q_rope, cache, meta, scale)
    return ref.mla_paged_attention(q_latent, q_rope, cache, meta.block_tables, meta.cu_q, meta.kv_lens, scale)


def moe_route(logits, top_k, scoring="softmax", norm_topk=False, n_group=1, topk_group=1, routed_scale=1.0,
              correction_bias=None):
    if logits.is_cuda:
        return _cuda().moe_route(logits, top_k, scoring, norm_topk, n_group, topk_group, routed_scale, correction_bias)
    return ref.moe_route(logits, top_k, scoring, norm_topk, n_group, topk_group, routed_scale, correction_bias)


def moe_experts(x, ids, weights, w_gate_up, w_down, expert_offset=0):
    if x.is_cuda:
        return _cuda().moe_experts(x, ids, weights, w_gate_up, w_down, expert_offset)
    return ref.moe_experts(x, ids, weights, w_gate_up, w_down, expert_offset)


def argmax(logits):
    if logits.is_cuda:
        return _cuda().argmax(logits)
    return ref.argmax(logits)


def sample(logits, temperature, top_k, top_p, uniform):
    if logits.is_cuda:
        return _cuda().sample(logits, temperature, top_k, top_p, uniform)
    return ref.sample(logits, temperature, top_k, top_p, uniform)
