"""Plain PyTorch fp32 restatements of every op.

They are the numerical oracle for the sm_100a kernels (each CUDA kernel's test compares against the
function of the same name here) and the execution path on CPU, where no CUDA kernel exists.
KV cache layout per layer: ``[num_blocks, 2, num_kv_heads, block_size, head_dim]`` (index 0 = K, 1 = V).
MLA latent cache layout per layer: ``[num_blocks, block_size, kv_lora_rank + rope_dim]``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# ---- normalisation -------------------------------------------------------------------------------

def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float,
             residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = rmsnorm(x [+ residual]) * weight. With ``residual`` the sum is written back into it."""
    xf = x.float()
    if residual is not None:
        xf = xf + residual.float()
        residual.copy_(xf.to(residual.dtype))
        xf = residual.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps) * weight.float()
    return y.to(x.dtype)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float,
               residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    xf = x.float()
    if residual is not None:
        xf = xf + residual.float()
        residual.copy_(xf.to(residual.dtype))
        xf = residual.float()
    y = F.layer_norm(xf, (xf.shape[-1],), weight.float(), None if bias is None else bias.float(), eps)
    return y.to(x.dtype)


# ---- dense linear algebra -------------------------------------------------------------------------

def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[T, N] = x[T, K] @ weight[N, K]^T (+ bias), fp32 accumulation."""
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    """x = [gate | up] along the last dim -> silu(gate) * up."""
    d = x.shape[-1] // 2
    g, u = x[..., :d].float(), x[..., d:].float()
    return (F.silu(g) * u).to(x.dtype)


def gelu_and_mul(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    g, u = x[..., :d].float(), x[..., d:].float()
    return (F.gelu(g, approximate="tanh") * u).to(x.dtype)


def activation(x: torch.Tensor, kind: str) -> torch.Tensor:
    xf = x.float()
    if kind in ("gelu", "gelu_python"):
        y = F.gelu(xf)
    elif kind in ("gelu_new", "gelu_fast", "gelu_pytorch_tanh"):
        y = F.gelu(xf, approximate="tanh")
    elif kind == "relu":
        y = F.relu(xf)
    elif kind in ("silu", "swish"):
        y = F.silu(xf)
    elif kind == "sigmoid":
        y = torch.sigmoid(xf)
    else:
        raise ValueError(f"unknown activation {kind}")
    return y.to(x.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    y = table[ids.long()]
    return y if scale == 1.0 else (y.float() * scale).to(table.dtype)


# ---- fp8 block-scaled ------------------------------------------------------------------------------

FP8_MAX = 448.0


def pow2_ceil(s: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= s (s > 0, fp32): the UE8M0 scale the tensor core can apply itself."""
    m, e = torch.frexp(s.float())  # s = m * 2^e, m in [0.5, 1)
    return torch.ldexp(torch.ones_like(m), torch.where(m == 0.5, e - 1, e))


def is_pow2(s: torch.Tensor) -> bool:
    m, _ = torch.frexp(s.float())
    return bool(((m == 0.5) & (s > 0)).all())


def quant_fp8_group(x: torch.Tensor, group: int = 128, ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token 1 x ``group`` dynamic e4m3 quantisation: returns (q[T, K] fp8, scale[T, K/group] fp32).
    ``ue8m0``: the scale is rounded up to a power of two."""
    T, K = x.shape
    assert K % group == 0
    xf = x.float().view(T, K // group, group)
    if ue8m0:
        scale = pow2_ceil(xf.abs().amax(-1).clamp_min(1e-30) / FP8_MAX)
    else:
        amax = xf.abs().amax(-1).clamp_min(1e-10)
        scale = amax / FP8_MAX
    q = (xf / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.view(T, K), scale


def quant_fp8_block_weight(w: torch.Tensor, block: int = 128, ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """128x128 block-scaled e4m3 weight: returns (q[N, K] fp8, scale_inv[ceil(N/b), ceil(K/b)] fp32)
    with ``w ~= q * scale_inv`` (the checkpoint convention ``weight_scale_inv``). ``ue8m0``: power-of-two scales."""
    N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    wp = torch.zeros(nb * block, kb * block, dtype=torch.float32, device=w.device)
    wp[:N, :K] = w.float()
    blocks = wp.view(nb, block, kb, block)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-10)
    scale = amax / FP8_MAX
    if ue8m0:
        scale = pow2_ceil(scale)
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.view(nb * block, kb * block)[:N, :K].contiguous(), scale


def requant_fp8_block_ue8m0(q: torch.Tensor, scale_inv: torch.Tensor,
                            block: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """Re-expresses a block-scaled e4m3 weight with power-of-two scales: every block's scale is rounded up to a
    power of two and its values are re-rounded to e4m3 on the coarser grid (ratio in (0.5, 1], at most one extra
    rounding step per element)."""
    N, K = q.shape
    new = pow2_ceil(scale_inv.float())
    ratio = (scale_inv.float() / new).repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return (q.float() * ratio).to(torch.float8_e4m3fn), new


def dequant_fp8_block_weight(q: torch.Tensor, scale_inv: torch.Tensor, block: int = 128) -> torch.Tensor:
    N, K = q.shape
    s = scale_inv.float().repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return q.float() * s


def linear_fp8_block(x: torch.Tensor, wq: torch.Tensor, w_scale_inv: torch.Tensor,
                     bias: Optional[torch.Tensor] = None, block: int = 128, ue8m0: bool = False) -> torch.Tensor:
    """bf16 activations are quantised per token per 128 channels, weights are 128x128 block-scaled e4m3;
    accumulation is fp32 with the scales applied per K-block (same math the tcgen05 kernel performs).
    ``ue8m0``: the activation scales are powers of two (the weights' are whatever ``w_scale_inv`` holds)."""
    T, K = x.shape
    xq, xs = quant_fp8_group(x, block, ue8m0)
    xd = (xq.float().view(T, K // block, block) * xs.unsqueeze(-1)).view(T, K)
    y = xd @ dequant_fp8_block_weight(wq, w_scale_inv, block).t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


# ---- int4 weight-only -------------------------------------------------------------------------------

def pack_int4(w_int: torch.Tensor) -> torch.Tensor:
    """[N, K] ints in [0, 15] -> [N, K/8] int32, element j of a word in bits [4j, 4j+4)."""
    N, K = w_int.shape
    w = w_int.to(torch.int64).view(N, K // 8, 8)
    out = torch.zeros(N, K // 8, dtype=torch.int64, device=w.device)
    for j in range(8):
        out |= (w[..., j] & 0xF) << (4 * j)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out)
    return out.to(torch.int32)


def unpack_int4(packed: torch.Tensor) -> torch.Tensor:
    N, K8 = packed.shape
    p = packed.to(torch.int64) & 0xFFFFFFFF
    cols = [((p >> (4 * j)) & 0xF) for j in range(8)]
    return torch.stack(cols, dim=-1).view(N, K8 * 8).to(torch.int32)


def tile_int4(packed: torch.Tensor) -> torch.Tensor:
    """[N, K/8] packed words -> [K/64, ceil(N/128), 128, 8]: each (128 rows x 64 weights) block contiguous, rows
    past N zero, blocks of one k-step next to each other. This is the layout the CUDA int4 GEMM streams (one 4 KB
    block per pipeline stage; CTAs working on neighbouring row tiles read neighbouring blocks, which keeps their
    concurrent streams spread over all memory channels)."""
    N, K8 = packed.shape
    assert K8 % 8 == 0
    nt = (N + 127) // 128
    p = packed
    if nt * 128 != N:
        p = torch.cat((p, torch.zeros(nt * 128 - N, K8, dtype=p.dtype, device=p.device)), dim=0)
    return p.view(nt, 128, K8 // 8, 8).permute(2, 0, 1, 3).contiguous()


def untile_int4(tiled: torch.Tensor, n_rows: int) -> torch.Tensor:
    kb, nt, _, _ = tiled.shape
    return tiled.permute(1, 2, 0, 3).reshape(nt * 128, kb * 8)[:n_rows].contiguous()


def quant_int4_group(w: torch.Tensor, group: int = 128) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Asymmetric 4-bit group quantisation along K: (packed[N, K/8] i32, scales[N, K/g], zeros[N, K/g])
    with w ~= (q - zero) * scale."""
    N, K = w.shape
    wf = w.float().view(N, K // group, group)
    mx, mn = wf.amax(-1), wf.amin(-1)
    scale = ((mx - mn) / 15.0).clamp_min(1e-8)
    zero = torch.round(-mn / scale).clamp(0, 15)
    q = torch.round(wf / scale.unsqueeze(-1) + zero.unsqueeze(-1)).clamp(0, 15)
    return pack_int4(q.view(N, K).to(torch.int32)), scale, zero


def dequant_int4_group(packed: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, group: int = 128) -> torch.Tensor:
    q = unpack_int4(packed).float()
    N, K = q.shape
    q = q.view(N, K // group, group)
    return ((q - zeros.float().unsqueeze(-1)) * scales.float().unsqueeze(-1)).view(N, K)


def linear_int4(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                bias: Optional[torch.Tensor] = None, group: int = 128) -> torch.Tensor:
    if packed.dim() == 4:
        packed = untile_int4(packed, scales.shape[0])
    w = dequant_int4_group(packed, scales, zeros, group).to(x.dtype)
    return linear(x, w, bias)


# ---- rotary embedding -------------------------------------------------------------------------------

def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool, rotary_dim: int) -> torch.Tensor:
    """x: [T, heads, d]; cos/sin: [T, rotary_dim/2]."""
    xf = x.float()
    rot, rest = xf[..., :rotary_dim], xf[..., rotary_dim:]
    c, s = cos.float().unsqueeze(1), sin.float().unsqueeze(1)
    if interleaved:
        x1, x2 = rot[..., 0::2], rot[..., 1::2]
        o = torch.stack((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).flatten(-2)
    else:
        h = rotary_dim // 2
        x1, x2 = rot[..., :h], rot[..., h:]
        o = torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)
    return torch.cat((o, rest), dim=-1).to(x.dtype)


def rope_qknorm_cache(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor,
                      cos_sin: Optional[torch.Tensor], slot_mapping: torch.Tensor, kv_cache: torch.Tensor,
                      q_norm_w: Optional[torch.Tensor] = None, k_norm_w: Optional[torch.Tensor] = None,
                      eps: float = 1e-6, interleaved: bool = False, rotary_dim: int = 0,
                      k_scale: float = 1.0, v_scale: float = 1.0, norm_after_rope: bool = False) -> None:
    """In place: optional per-head RMSNorm on q,k -> RoPE on q,k -> append k,v to the paged cache
    (``norm_after_rope``: RoPE first, then the norm, as Hunyuan does).

    q: [T, h, d], k/v: [T, hk, d]; cos_sin: [max_pos, rotary_dim] = [cos | sin] or None (no RoPE);
    slot_mapping[t] = block * block_size + offset."""
    T, hk, d = k.shape
    if q_norm_w is not None and not norm_after_rope:
        q.copy_(rms_norm(q, q_norm_w, eps))
        k.copy_(rms_norm(k, k_norm_w, eps))
    if cos_sin is not None:
        rd = rotary_dim or d
        cs = cos_sin[positions.long()]
        cos, sin = cs[:, : rd // 2], cs[:, rd // 2:]
        q.copy_(apply_rope(q, cos, sin, interleaved, rd))
        k.copy_(apply_rope(k, cos, sin, interleaved, rd))
    if q_norm_w is not None and norm_after_rope:
        q.copy_(rms_norm(q, q_norm_w, eps))
        k.copy_(rms_norm(k, k_norm_w, eps))
    bs = kv_cache.shape[3]
    blk = (slot_mapping // bs).long()
    off = (slot_mapping % bs).long()
    if kv_cache.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        kv_cache[blk, 0, :, off] = (k.float() / k_scale).to(kv_cache.dtype)
        kv_cache[blk, 1, :, off] = (v.float() / v_scale).to(kv_cache.dtype)
    else:
        kv_cache[blk, 0, :, off] = k.to(kv_cache.dtype)
        kv_cache[blk, 1, :, off] = v.to(kv_cache.dtype)


# ---- attention over the paged cache -------------------------------------------------------------------

def paged_attention(q: torch.Tensor, kv_cache: torch.Tensor, block_tables: torch.Tensor, cu_q: torch.Tensor,
                    kv_lens: torch.Tensor, scale: float, alibi_slopes: Optional[torch.Tensor] = None,
                    k_scale: float = 1.0, v_scale: float = 1.0, window: int = 0) -> torch.Tensor:
    """Causal attention of each sequence's new tokens over its whole paged context.

    q: [T, h, d]; the new tokens of sequence b are rows cu_q[b]:cu_q[b+1] and occupy context
    positions kv_lens[b]-q_len .. kv_lens[b]-1 (their K/V are already in the cache). ``window`` > 0: sliding window
    of that many keys; ``window`` < 0: chunked attention over blocks of ``-window`` positions (Llama 4)."""
    T, h, d = q.shape
    nb, _, hk, bs, dv = kv_cache.shape
    out = torch.empty(T, h, dv, dtype=q.dtype, device=q.device)
    B = kv_lens.numel()
    cu = cu_q.tolist()
    kl = kv_lens.tolist()
    group = h // hk
    for b in range(B):
        qs, qe = cu[b], cu[b + 1]
        ql, L = qe - qs, kl[b]
        if ql == 0:
            continue
        nblk = (L + bs - 1) // bs
        blocks = block_tables[b, :nblk].long()
        kv = kv_cache[blocks]  # [nblk, 2, hk, bs, d]
        K = kv[:, 0].permute(1, 0, 2, 3).reshape(hk, nblk * bs, d)[:, :L].float() * k_scale
        V = kv[:, 1].permute(1, 0, 2, 3).reshape(hk, nblk * bs, dv)[:, :L].float() * v_scale
        Q = q[qs:qe].float().permute(1, 0, 2)  # [h, ql, d]
        K = K.repeat_interleave(group, 0)
        V = V.repeat_interleave(group, 0)
        s = torch.einsum("hqd,hkd->hqk", Q, K) * scale
        qpos = torch.arange(L - ql, L, device=q.device).unsqueeze(1)
        kpos = torch.arange(L, device=q.device).unsqueeze(0)
        mask = kpos > qpos
        if window > 0:
            mask = mask | (kpos <= qpos - window)
        elif window < 0:  # chunked attention: keys of the query's own block of -window positions
            mask = mask | (kpos < (qpos // -window) * -window)
        if alibi_slopes is not None:
            s = s + alibi_slopes.float().view(h, 1, 1) * (kpos - qpos).float().unsqueeze(0)
        s = s.masked_fill(mask.unsqueeze(0), float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[qs:qe] = torch.einsum("hqk,hkd->hqd", p, V).permute(1, 0, 2).to(q.dtype)
    return out


def mla_cache_append(latent: torch.Tensor, k_rope: torch.Tensor, slot_mapping: torch.Tensor,
                     cache: torch.Tensor) -> None:
    """cache[block, off] = [latent | k_rope]; cache: [num_blocks, block_size, r + dr]."""
    bs = cache.shape[1]
    blk, off = (slot_mapping // bs).long(), (slot_mapping % bs).long()
    cache[blk, off] = torch.cat((latent, k_rope), dim=-1).to(cache.dtype)


def mla_paged_attention(q_latent: torch.Tensor, q_rope: torch.Tensor, cache: torch.Tensor,
                        block_tables: torch.Tensor, cu_q: torch.Tensor, kv_lens: torch.Tensor,
                        scale: float) -> torch.Tensor:
    """Absorbed MLA attention: scores = q_latent . c + q_rope . k_rope over the latent cache, output
    is the probability-weighted latent [T, h, r] (the caller applies W_uv)."""
    T, h, r = q_latent.shape
    bs = cache.shape[1]
    out = torch.empty(T, h, r, dtype=q_latent.dtype, device=q_latent.device)
    cu, kl = cu_q.tolist(), kv_lens.tolist()
    qcat = torch.cat((q_latent, q_rope), dim=-1).float()
    for b in range(len(kl)):
        qs, qe = cu[b], cu[b + 1]
        ql, L = qe - qs, kl[b]
        if ql == 0:
            continue
        nblk = (L + bs - 1) // bs
        c = cache[block_tables[b, :nblk].long()].reshape(nblk * bs, -1)[:L].float()
        s = torch.einsum("qhd,kd->hqk", qcat[qs:qe], c) * scale
        qpos = torch.arange(L - ql, L, device=s.device).unsqueeze(1)
        kpos = torch.arange(L, device=s.device).unsqueeze(0)
        s = s.masked_fill((kpos > qpos).unsqueeze(0), float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[qs:qe] = torch.einsum("hqk,kd->qhd", p, c[:, :r]).to(out.dtype)
    return out


def mla_sparse_paged_attention(q_latent: torch.Tensor, q_rope: torch.Tensor, idx_q: torch.Tensor, idx_w: torch.Tensor,
                               cache: torch.Tensor, block_tables: torch.Tensor, cu_q: torch.Tensor,
                               kv_lens: torch.Tensor, scale: float, main_width: int, topk: int) -> torch.Tensor:
    """Absorbed MLA attention restricted to the keys an indexer selects (DeepSeek sparse attention).

    Cache rows are [latent | k_rope | indexer key]; ``main_width`` = r + dr. idx_q: [T, Hi, Di], idx_w: [T, Hi].
    index score[q, t] = sum_h idx_w[q, h] * relu(idx_q[q, h] . k_idx[t]) over the causally visible keys; each query
    attends to its ``topk`` best keys (all of them while the context is shorter than topk)."""
    T, h, r = q_latent.shape
    bs = cache.shape[1]
    out = torch.empty(T, h, r, dtype=q_latent.dtype, device=q_latent.device)
    cu, kl = cu_q.tolist(), kv_lens.tolist()
    qcat = torch.cat((q_latent, q_rope), dim=-1).float()
    for b in range(len(kl)):
        qs, qe = cu[b], cu[b + 1]
        ql, L = qe - qs, kl[b]
        if ql == 0:
            continue
        nblk = (L + bs - 1) // bs
        rows = cache[block_tables[b, :nblk].long()].reshape(nblk * bs, -1)[:L].float()
        c, kidx = rows[:, :main_width], rows[:, main_width:]
        qpos = torch.arange(L - ql, L, device=rows.device).unsqueeze(1)
        kpos = torch.arange(L, device=rows.device).unsqueeze(0)
        hidden = kpos > qpos
        isc = torch.einsum("qhd,kd->qhk", idx_q[qs:qe].float(), kidx).relu()
        isc = torch.einsum("qhk,qh->qk", isc, idx_w[qs:qe].float()).masked_fill(hidden, float("-inf"))
        if L > topk:
            keep = torch.zeros(ql, L, dtype=torch.bool, device=rows.device)
            keep.scatter_(1, isc.topk(topk, dim=-1).indices, True)
            hidden = hidden | ~keep
        s = torch.einsum("qhd,kd->hqk", qcat[qs:qe], c) * scale
        s = s.masked_fill(hidden.unsqueeze(0), float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[qs:qe] = torch.einsum("hqk,kd->qhd", p, c[:, :r]).to(out.dtype)
    return out


# ---- MoE ------------------------------------------------------------------------------------------

def moe_route(logits: torch.Tensor, top_k: int, scoring: str = "softmax", norm_topk: bool = False,
              n_group: int = 1, topk_group: int = 1, routed_scale: float = 1.0,
              correction_bias: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Router: returns (expert ids [T, k] int32, weights [T, k] fp32).

    softmax: Mixtral / Qwen-MoE (optionally renormalised); sigmoid + correction bias + group-limited
    top-k + scaling: DeepSeek-V3 (group score = sum of the top-2 biased scores in the group)."""
    x = logits.float()
    T, E = x.shape
    if scoring == "sigmoid":
        scores = torch.sigmoid(x)
    else:
        scores = torch.softmax(x, dim=-1)
    choice = scores if correction_bias is None else scores + correction_bias.float().unsqueeze(0)
    if n_group > 1:
        g = choice.view(T, n_group, E // n_group)
        if correction_bias is not None:
            gscore = g.topk(2, dim=-1).values.sum(-1)
        else:
            gscore = g.amax(-1)
        gidx = gscore.topk(topk_group, dim=-1).indices
        gmask = torch.zeros(T, n_group, dtype=torch.bool, device=x.device).scatter_(1, gidx, True)
        choice = g.masked_fill(~gmask.unsqueeze(-1), float("-inf")).view(T, E)
    ids = choice.topk(top_k, dim=-1).indices
    w = scores.gather(1, ids)
    if norm_topk:
        w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
    w = w * routed_scale
    return ids.to(torch.int32), w


def moe_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor,
                w_down: torch.Tensor, expert_offset: int = 0) -> torch.Tensor:
    """Sum over the selected experts that live on this rank.

    w_gate_up: [E_local, 2I, H] ([gate | up] rows), w_down: [E_local, H, I]; ids are global expert ids,
    experts outside [expert_offset, expert_offset + E_local) are skipped (another rank's work)."""
    T, H = x.shape
    E_local = w_gate_up.shape[0]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for e in range(E_local):
        sel = (ids == e + expert_offset)
        tok, slot = sel.nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = linear(x[tok], w_gate_up[e])
        a = silu_and_mul(h)
        y = linear(a, w_down[e]).float()
        out.index_add_(0, tok, y * weights[tok, slot].unsqueeze(-1))
    return out.to(x.dtype)


def moe_experts_fp8(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, wq_gate_up: torch.Tensor,
                    s_gate_up: torch.Tensor, wq_down: torch.Tensor, s_down: torch.Tensor,
                    expert_offset: int = 0) -> torch.Tensor:
    """``moe_experts`` for block-scaled e4m3 expert weights ([E_local, 2I, H] + scales [E_local, 2I/128, H/128],
    [E_local, H, I] + [E_local, H/128, I/128]); activations are quantised per token per 128 channels before each GEMM."""
    T, H = x.shape
    E_local = wq_gate_up.shape[0]
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    for e in range(E_local):
        tok, slot = (ids == e + expert_offset).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        a = silu_and_mul(linear_fp8_block(x[tok], wq_gate_up[e], s_gate_up[e]))
        y = linear_fp8_block(a, wq_down[e], s_down[e]).float()
        out.index_add_(0, tok, y * weights[tok, slot].unsqueeze(-1))
    return out.to(x.dtype)


# ---- sampling ---------------------------------------------------------------------------------------

def argmax(logits: torch.Tensor) -> torch.Tensor:
    return logits.float().argmax(-1).to(torch.int32)


def apply_penalties(logits: torch.Tensor, token_counts: Optional[torch.Tensor], repetition_penalty: torch.Tensor,
                    bitmask: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """logits [B, V] fp32. ``token_counts`` [B, V] > 0 marks tokens seen in prompt or output;
    repetition penalty divides positive logits and multiplies negative ones (HF semantics);
    ``bitmask`` [B, ceil(V/32)] int32 keeps a token only when its bit is set (grammar constraint)."""
    x = logits.float().clone()
    if token_counts is not None:
        pen = repetition_penalty.float().unsqueeze(1)
        seen = token_counts > 0
        x = torch.where(seen, torch.where(x > 0, x / pen, x * pen), x)
    if bias is not None:
        x = x + bias.float()
    if bitmask is not None:
        V = x.shape[1]
        idx = torch.arange(V, device=x.device)
        bits = (bitmask[:, (idx // 32)].to(torch.int64) >> (idx % 32).unsqueeze(0)) & 1
        x = x.masked_fill(bits == 0, float("-inf"))
    return x


def sample_probs(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor) -> torch.Tensor:
    """Distribution the sampler draws from: softmax(logits / T), keep the top-k (1..1024) tokens, then the
    smallest descending prefix of those whose mass reaches top_p * (mass of the top-k set); renormalise.
    top-p is applied inside the top-k set (reference semantics, sampling_topk_kernels.cu:150-215)."""
    B, V = logits.shape
    t = temperature.float().clamp_min(1e-6).unsqueeze(1)
    p = torch.softmax(logits.float() / t, dim=-1)
    sp, si = p.sort(dim=-1, descending=True)
    ranks = torch.arange(V, device=logits.device).unsqueeze(0)
    k = top_k.clamp(1, min(V, 1024)).unsqueeze(1)
    sp = sp.masked_fill(ranks >= k, 0.0)
    mass = sp.sum(-1, keepdim=True)
    cum = sp.cumsum(-1)
    keep = (cum - sp) < top_p.float().unsqueeze(1) * mass
    keep[:, 0] = True
    sp = sp * keep
    sp = sp / sp.sum(-1, keepdim=True)
    return torch.zeros_like(p).scatter_(1, si, sp)


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor) -> torch.Tensor:
    """Inverse-CDF draw in descending-probability order with one uniform number per row."""
    probs = sample_probs(logits, temperature, top_k, top_p)
    sp, si = probs.sort(dim=-1, descending=True)
    cum = sp.cumsum(-1)
    u = uniform.float().clamp(0, 1 - 1e-7).unsqueeze(1) * cum[:, -1:]
    pick = (cum <= u).sum(-1).clamp_max(probs.shape[1] - 1)
    return si.gather(1, pick.unsqueeze(1)).squeeze(1).to(torch.int32)


def logprobs_topn(logits: torch.Tensor, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
    lp = torch.log_softmax(logits.float(), dim=-1)
    v, i = lp.topk(n, dim=-1)
    return v, i.to(torch.int32)


# ---- rope tables ------------------------------------------------------------------------------------

def _yarn_find_dim(num_rot: float, dim: int, base: float, max_pos: int) -> float:
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def yarn_mscale(scale: float, mscale: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


def build_rope_cache(rotary_dim: int, max_pos: int, theta: float, scaling=None, device="cpu") -> torch.Tensor:
    """[max_pos, rotary_dim] = [cos | sin] in fp32. Supports default, linear, dynamic-NTK (factor or alpha),
    llama3 multi-frequency and YaRN scaling (reference: rotary_embedding.cu:237-431 cache builders)."""
    half = rotary_dim // 2
    idx = torch.arange(0, half, dtype=torch.float64)
    base = float(theta)
    typ = getattr(scaling, "type", "default") if scaling is not None else "default"
    factor = float(getattr(scaling, "factor", 1.0)) if scaling is not None else 1.0
    mscale = 1.0
    pos = torch.arange(max_pos, dtype=torch.float64)
    if typ == "dynamic":
        alpha = float(getattr(scaling, "alpha", 0.0))
        if alpha > 0:
            base = base * alpha ** (rotary_dim / (rotary_dim - 2))
        else:
            orig = scaling.original_max_position_embeddings or max_pos
            if max_pos > orig:
                base = base * ((factor * max_pos / orig) - (factor - 1)) ** (rotary_dim / (rotary_dim - 2))
    inv = 1.0 / (base ** (idx * 2 / rotary_dim))
    if typ == "linear":
        pos = pos / factor
    elif typ == "llama3":
        orig = scaling.original_max_position_embeddings or 8192
        lo, hi = scaling.low_freq_factor, scaling.high_freq_factor
        wavelen = 2 * math.pi / inv
        smooth = ((orig / wavelen) - lo) / (hi - lo)
        scaled = torch.where(wavelen > orig / lo, inv / factor,
                             torch.where(wavelen < orig / hi, inv, (1 - smooth) * inv / factor + smooth * inv))
        inv = scaled
    elif typ == "yarn":
        orig = scaling.original_max_position_embeddings or max_pos
        low = max(math.floor(_yarn_find_dim(scaling.beta_fast, rotary_dim, base, orig)), 0)
        high = min(math.ceil(_yarn_find_dim(scaling.beta_slow, rotary_dim, base, orig)), rotary_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(half, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
        inv_mask = 1.0 - ramp
        inv = inv / factor * (1 - inv_mask) + inv * inv_mask
        mscale = yarn_mscale(factor, scaling.mscale) / yarn_mscale(factor, scaling.mscale_all_dim) \
            if scaling.mscale_all_dim else yarn_mscale(factor, 1.0)
    freqs = torch.outer(pos, inv)
    out = torch.cat((freqs.cos() * mscale, freqs.sin() * mscale), dim=-1).float()
    return out.to(device)


def mrope_rows(cos_sin: torch.Tensor, positions3: torch.Tensor, sections) -> torch.Tensor:
    """Multi-axis RoPE. Qwen2-VL (M-RoPE, 3 axes): frequency indices [0, s0) rotate by the temporal position,
    [s0, s0 + s1) by the height position, the rest by the width position. Arc-Hunyuan-Video (XD-RoPE, 4 axes): the
    same with one more axis in front. cos_sin: [max_pos, rd] = [cos | sin]; positions3: [axes, T]. Returns a
    per-token table [T, rd] to be indexed with positions 0..T-1 by the ordinary RoPE code. Reference:
    rotary_embedding.cu:150-235 (section lookup per rotary offset)."""
    rd = cos_sin.shape[1]
    half = rd // 2
    assert sum(sections) == half, "the rope sections must cover half of the rotary dimension"
    p = positions3.long()
    axes = p.shape[0]
    rows = [cos_sin[p[i]] for i in range(axes)]  # each [T, rd]
    cos_parts, sin_parts, lo = [], [], 0
    for i, sec in enumerate(sections):
        src = rows[i % axes]
        cos_parts.append(src[:, lo:lo + sec])
        sin_parts.append(src[:, half + lo:half + lo + sec])
        lo += sec
    return torch.cat(cos_parts + sin_parts, dim=-1).contiguous()


def alibi_slopes(num_heads: int) -> torch.Tensor:
    def pow2(n):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]
    if math.log2(num_heads).is_integer():
        s = pow2(num_heads)
    else:
        c = 2 ** math.floor(math.log2(num_heads))
        s = pow2(c) + pow2(2 * c)[0::2][: num_heads - c]
    return torch.tensor(s, dtype=torch.float32)
