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


def gemm_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, b, :] = a[t, b, :] @ w[b]^T. a: [T, B, K] view (last dim contiguous), w: [B, N, K] contiguous,
    out: [T, B, N] view (last dim contiguous); bf16. Head-batched tcgen05 GEMM (csrc/cuda/gemm_batched.cu)."""
    from . import cuda
    T, B, K = a.shape
    N = w.shape[1]
    code = cuda.lib().ksana_gemm_bf16_batched(cuda._ptr(a), a.stride(0), a.stride(1), cuda._ptr(w), cuda._ptr(out),
                                              out.stride(0), out.stride(1), T, B, N, K, cuda._stream())
    cuda._check(code, "gemm_bf16_batched")
    return out


def fused_supported(q, cache, r, dr, dn, dv, h) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and r == 512 and dr == 64 and
            cache.shape[1] == 64 and cache.shape[2] == r + dr and h <= 128 and dn % 8 == 0 and dv % 128 == 0 and
            q.stride(-1) == 1)


def mla_absorbed_attention(q, w_uk_nk, w_uv_nk, latent, k_rope, positions, cos_sin, interleaved, cache, meta, scale,
                           dn, dr):
    """The MLA attention core without a PyTorch op: head-batched absorb GEMM (q_nope x W_UK^T) straight into the
    [latent | rope] query rows, fused RoPE (query + key) + cache append, absorbed attention over the latent cache,
    head-batched GEMM with W_UV. q: [T, h, dn + dr] bf16; w_uk_nk: [h, r, dn]; w_uv_nk: [h, dv, r]; latent: [T, r];
    k_rope: [T, dr]; cos_sin: the fp32 rope table [max_pos, dr]. Returns [T, h, dv]."""
    from . import cuda
    T, h, _ = q.shape
    r, dv = w_uk_nk.shape[1], w_uv_nk.shape[1]
    dev = q.device
    q_cat = torch.empty(T, h, r + dr, dtype=torch.bfloat16, device=dev)
    gemm_batched(q[..., :dn], w_uk_nk, q_cat[..., :r])
    k_rope = k_rope.reshape(T, dr)
    code = cuda.lib().ksana_mla_rope_append(cuda._ptr(q), q.stride(0), q.stride(1), dn, cuda._ptr(q_cat),
                                            cuda._ptr(k_rope), k_rope.stride(0), cuda._ptr(latent), latent.stride(0),
                                            cuda._ptr(positions), cuda._ptr(cos_sin), cuda._ptr(meta.slot_mapping),
                                            cuda._ptr(cache), cache.shape[2], T, h, r, dr, 1 if interleaved else 0,
                                            cuda._stream())
    cuda._check(code, "mla_rope_append")
    nb = cache.shape[0]
    o_lat = torch.empty(T, h, r, dtype=torch.bfloat16, device=dev)
    cu = meta.cu_q_host
    max_q = int((cu[1:] - cu[:-1]).max())
    max_kv = int(meta.kv_lens_host.max())
    ws = cuda.workspace(dev)
    code = cuda.lib().ksana_mla_decode(cuda._ptr(q_cat), T, cuda._ptr(cache), nb, cuda._ptr(meta.block_tables),
                                       meta.max_blocks, cuda._ptr(meta.cu_q), cuda._ptr(meta.kv_lens), 0, meta.num_seqs,
                                       max_q, max_kv, h, float(scale), cuda._ptr(o_lat), cuda._ptr(ws.attn_ws),
                                       ws.attn_ws.numel(), cuda._stream())
    cuda._check(code, "mla_decode")
    out = torch.empty(T, h, dv, dtype=torch.bfloat16, device=dev)
    return gemm_batched(o_lat, w_uv_nk, out)
