"""MLA (latent) cache append and absorbed attention over the latent cache."""
from __future__ import annotations

from . import reference as ref


def mla_cache_append(latent, k_rope, slot_mapping, cache):
    return ref.mla_cache_append(latent, k_rope, slot_mapping, cache)


def mla_paged_attention(q_latent, q_rope, cache, meta, scale):
    return ref.mla_paged_attention(q_latent, q_rope, cache, meta.block_tables, meta.cu_q, meta.kv_lens, scale)
