"""MLA (latent) cache append and absorbed attention over the latent cache (csrc/cuda/attention_mla.cu)."""
from __future__ import annotations

import torch

from . import reference as ref


def mla_cache_append(latent, k_rope, slot_mapping, cache):
    from . import cuda
    if latent.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        return ref.mla_cache_append(latent, k_rope, slot_mapping, cache)
    T, r = latent.shape
    dr = k_rope.shape[-1]
    k_rope = k_rope.reshape(T, dr)
    code = cuda.lib().ksana_mla_cache_append(cuda._ptr(latent), latent.stride(0), cuda._ptr(k_rope), k_rope.stride(0),
                                             cuda._ptr(slot_mapping), cuda._ptr(cache), T, r, dr, cuda._stream())
    cuda._check(code, "mla_cache_append")


def mla_paged_attention(q_latent, q_rope, cache, meta, scale):
    """q_latent [T, h, 512], q_rope [T, h, 64] -> probability-weighted latent [T, h, 512]."""
    from . import cuda
    T, h, r = q_latent.shape
    nb, bs, width = cache.shape
    if (q_latent.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or r != 512 or q_rope.shape[-1] != 64 or
            bs != 64 or h > 128):
        return ref.mla_paged_attention(q_latent, q_rope, cache, meta.block_tables, meta.cu_q, meta.kv_lens, scale)
    q_cat = torch.cat((q_latent, q_rope), dim=-1).contiguous()
    out = torch.empty(T, h, r, dtype=torch.bfloat16, device=q_latent.device)
    cu = meta.cu_q_host
    max_q = int((cu[1:] - cu[:-1]).max())
    max_kv = int(meta.kv_lens_host.max())
    ws = cuda.workspace(q_latent.device)
    code = cuda.lib().ksana_mla_decode(cuda._ptr(q_cat), T, cuda._ptr(cache), nb, cuda._ptr(meta.block_tables),
                                       meta.max_blocks, cuda._ptr(meta.cu_q), cuda._ptr(meta.kv_lens), 0, meta.num_seqs,
                                       max_q, max_kv, h, float(scale), cuda._ptr(out), cuda._ptr(ws.attn_ws),
                                       ws.attn_ws.numel(), cuda._stream())
    cuda._check(code, "mla_decode")
    return out
