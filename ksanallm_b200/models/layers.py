"""Building blocks shared by every architecture: (quantised) linear holders, attention flavours
(MHA/GQA with RoPE / ALiBi / learned positions, MLA with weight absorption), FFN flavours (gated,
plain, MoE with shared experts) over the paged KV cache.

Reference counterparts: src/ksana_llm/modules/basic/linear.cpp:44, modules/attention/
common_attention.cpp:33-75, multihead_latent_attention.cpp:155-456, modules/ffn/two_layered_ffn.cpp:22-118,
layers/nvidia/moe_layer.cpp:208-377.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional

import torch

from .. import ops
from ..config.model_config import ModelConfig
from ..ops import reference as ref
from ..parallel.comm import TPGroup


_EPLB_LAYERS: Dict[str, "MoEFFN"] = {}


def dump_eplb_counts(path: Optional[str] = None, rank: int = 0) -> Optional[str]:
    """Writes {layer prefix: times each expert was chosen} gathered since start-up (enabled by DUMP_EPLB_PATH) for
    ``python -m ksanallm_b200.tools.eplb``. Reference: moe_layer.cpp:412-415, 465-471 (per-step top-k id dumps)."""
    import json
    path = path or os.environ.get("DUMP_EPLB_PATH")
    if not path or not _EPLB_LAYERS:
        return None
    os.makedirs(path, exist_ok=True)
    out = os.path.join(path, f"expert_counts_rank{rank}.json")
    with open(out, "w", encoding="utf-8") as f:
        json.dump({k.replace(".mlp", "").replace("model.layers.", "layer_"): v._eplb_counts.tolist()
                   for k, v in _EPLB_LAYERS.items()}, f)
    return out


class LinearW:
    """y = x @ W^T (+ b). W is stored [N, K] (K contiguous), which is exactly the K-major B operand the
    tcgen05 kernels want. Quantised variants keep the checkpoint's format:
    fp8 block-scaled (``weight`` e4m3 + ``weight_scale_inv`` fp32 per 128x128) and int4 group-quantised
    (``qweight`` packed + ``scales`` + ``zeros``)."""

    def __init__(self, weights: Dict[str, torch.Tensor], prefix: str):
        self.prefix = prefix
        self.weight = weights.get(prefix + ".weight")
        self.bias = weights.get(prefix + ".bias")
        self.scale_inv = weights.get(prefix + ".weight_scale_inv")
        self.qweight = weights.get(prefix + ".qweight")
        self.scales = weights.get(prefix + ".scales")
        self.zeros = weights.get(prefix + ".zeros")
        self.group = 128
        self.sz = None
        # act-order GPTQ: the 4-bit columns are stored group by group; the input is gathered the same way
        self.perm = weights.get(prefix + ".perm")
        # AWQ smoothing factor of W4A8 checkpoints: y = (x * pre) @ W^T. Folded into a dense weight once; a weight
        # that kept its 4-bit grid gets its input scaled at run time.
        self.pre = weights.get(prefix + ".pre_quant_scale")
        if self.pre is not None and self.qweight is None and self.weight is not None and self.scale_inv is None:
            self.weight = (self.weight.float() * self.pre.float().unsqueeze(0)).to(self.weight.dtype)
            weights[prefix + ".weight"] = self.weight
            weights.pop(prefix + ".pre_quant_scale")
            self.pre = None
        if self.qweight is not None:
            self.kind = "int4"
            self.group = self.qweight.shape[1] * 8 // self.scales.shape[1]
            self._n, self._k = self.qweight.shape[0], self.qweight.shape[1] * 8
            from ..ops import cuda_int4
            if self.qweight.is_cuda and cuda_int4.supports(self._k, self._n, self.group):
                # the CUDA GEMM streams 4 KB (128 rows x 64 weights) blocks: re-tile once, drop the row-major copy
                self.qweight = ref.tile_int4(self.qweight)
                weights[prefix + ".qweight"] = self.qweight
                self.sz = cuda_int4.pack_scale_zero(self.scales, self.zeros)
        elif self.scale_inv is not None:
            self.kind = "fp8_block"
            # power-of-two block scales: the activations get power-of-two group scales as well, and prefill-sized
            # products run with the scales applied by the tensor core (packed scale bytes built on first CUDA use)
            self.pow2 = self.weight.dim() == 2 and ref.is_pow2(self.scale_inv)
            self._sfb = None
        elif self.weight is not None:
            self.kind = "dense"
        else:
            raise KeyError(f"missing weight for {prefix}")

    @property
    def out_features(self) -> int:
        return self._n if self.kind == "int4" else self.weight.shape[0]

    @property
    def in_features(self) -> int:
        return self._k if self.kind == "int4" else self.weight.shape[1]

    def sfb(self) -> Optional[torch.Tensor]:
        """Packed power-of-two scale bytes of an fp8 block-scaled weight for the scaled tensor-core GEMM, or None."""
        if self.kind != "fp8_block" or not self.pow2 or not self.weight.is_cuda:
            return None
        if self._sfb is None:
            n, k = self.weight.shape
            if k % 128 or n % 8 or not self.weight.is_contiguous():
                return None
            from ..ops import cuda_fp8
            self._sfb = cuda_fp8.pack_sfb(self.scale_inv, n, k)
        return self._sfb

    def __call__(self, x: torch.Tensor, add_bias: bool = True) -> torch.Tensor:
        b = self.bias if add_bias else None
        if self.pre is not None:
            x = x * self.pre.to(x.dtype)
        if self.perm is not None and self.kind == "int4":
            x = x.index_select(-1, self.perm.to(x.device))
        if self.kind == "dense":
            return ops.linear(x, self.weight, b)
        if self.kind == "fp8_block":
            return ops.linear_fp8_block(x, self.weight, self.scale_inv, b, self.sfb() if x.is_cuda else None, self.pow2)
        return ops.linear_int4(x, self.qweight, self.scales, self.zeros, b, self.group, self.sz)


class Attention:
    """MHA / GQA over the paged cache. Heads are sharded over the TP group; o_proj is row-parallel."""

    def __init__(self, cfg: ModelConfig, w: Dict[str, torch.Tensor], prefix: str, layer_idx: int, tp: TPGroup,
                 rope_cache: Optional[torch.Tensor]):
        self.cfg = cfg
        self.tp = tp
        self.layer_idx = layer_idx
        self.h = cfg.num_heads // tp.size
        self.hk = max(cfg.num_kv_heads // tp.size, 1)
        self.d = cfg.head_dim
        self.qkv = LinearW(w, prefix + ".query_key_value")
        self.o_proj = LinearW(w, prefix + ".o_proj")
        self.q_norm = w.get(prefix + ".query_layernorm.weight")
        self.k_norm = w.get(prefix + ".key_layernorm.weight")
        self.rope_cache = rope_cache
        self.window = 0
        if cfg.sliding_window and (not cfg.sliding_layers or
                                   (layer_idx < len(cfg.sliding_layers) and cfg.sliding_layers[layer_idx])):
            self.window = cfg.sliding_window
        self.use_rope = True
        if cfg.rope_layers and layer_idx < len(cfg.rope_layers) and not cfg.rope_layers[layer_idx]:
            self.rope_cache, self.use_rope = None, False  # a layer without position encoding (Llama 4)
        if cfg.attention_chunk_size and self.use_rope and not self.window:
            # Llama 4 chunked attention on the RoPE layers: a query sees the keys of its own block of
            # `attention_chunk_size` positions only; passed down as a negative window
            self.window = -cfg.attention_chunk_size
        self.norm_after_rope = cfg.qk_norm_after_rope
        if cfg.qk_l2_norm and self.use_rope:
            # weightless RMS normalisation after RoPE: the ordinary path with unit weights
            ones = torch.ones(self.d, dtype=self.qkv.weight.dtype if self.qkv.weight is not None else torch.float32,
                              device=self.o_proj.weight.device)
            self.q_norm = self.k_norm = ones
            self.norm_after_rope = True
        self.scale = 1.0 / math.sqrt(self.d)
        # cross-layer attention (Hunyuan-Large): of every `cla_share_factor` layers only the first projects K and V,
        # the others project queries and attend over that layer's K / V projections (their own norm weights and
        # their own cache pages still apply). Reference: modules/attention/cross_layer_attention.cpp:51-90.
        f = cfg.cla_share_factor
        self.cla_owner = bool(f) and layer_idx % f == 0
        self.cla_follower = bool(f) and layer_idx % f != 0
        self.k_scale = self.v_scale = 1.0  # fp8 KV cache scaling factors (models/kv_scales.py)
        self.alibi = None
        if cfg.position_encoding == "alibi":
            full = ref.alibi_slopes(cfg.num_heads)
            self.alibi = full[tp.rank * self.h:(tp.rank + 1) * self.h].to(self.o_proj.weight.device)

    def core(self, h: torch.Tensor, meta, kv_cache: torch.Tensor) -> torch.Tensor:
        T = h.shape[0]
        qkv = self.qkv(h)
        nq, nk = self.h * self.d, self.hk * self.d
        q = qkv[:, :nq].view(T, self.h, self.d)
        if self.cla_follower:
            k, v = meta._cla_kv
            k = k.clone()  # RoPE / QK-norm below work in place and every follower applies its own
        else:
            k = qkv[:, nq:nq + nk].view(T, self.hk, self.d)
            v = qkv[:, nq + nk:].view(T, self.hk, self.d)
            if self.cla_owner:
                meta._cla_kv = (k.clone(), v)
        positions, table = meta.positions, self.rope_cache
        sections = self.cfg.rope_scaling.mrope_section
        if sections and table is not None and getattr(meta, "mrope_positions", None) is not None:
            # multimodal RoPE: a per-token cos/sin table built once per step, indexed by the token's row
            if meta._mrope_table is None:
                meta._mrope_table = ref.mrope_rows(table, meta.mrope_positions, sections)
                meta._arange = torch.arange(T, dtype=torch.int32, device=q.device)
            positions, table = meta._arange, meta._mrope_table
        ops.rope_qknorm_cache(q, k, v, positions, table, meta.slot_mapping, kv_cache,
                              self.q_norm, self.k_norm, self.cfg.rms_norm_eps, self.cfg.rope_interleaved,
                              self.cfg.rotary_dim, self.k_scale, self.v_scale, self.norm_after_rope)
        if self.cfg.attn_temperature_tuning and not self.use_rope:
            # Llama 4 temperature tuning of the position-free layers: q *= log1p(floor((pos + 1) / floor)) * c + 1
            t = torch.log1p(torch.floor((meta.positions.float() + 1.0) / self.cfg.attn_floor_scale))
            q.mul_((t * self.cfg.attn_scale_coef + 1.0).to(q.dtype).view(T, 1, 1))
        o = ops.paged_attention(q, kv_cache, meta, self.scale, self.alibi, self.k_scale, self.v_scale, self.window)
        return o.reshape(T, nq)


class MLAttention:
    """Multi-head latent attention with absorbed up-projections: the cache holds one
    ``kv_lora_rank + rope`` vector per token, scores and outputs are computed in latent space."""

    def __init__(self, cfg: ModelConfig, w: Dict[str, torch.Tensor], prefix: str, layer_idx: int, tp: TPGroup,
                 rope_cache: torch.Tensor):
        self.cfg = cfg
        self.tp = tp
        self.h = cfg.num_heads // tp.size
        self.r, self.dr, self.dn, self.dv = cfg.kv_lora_rank, cfg.qk_rope_head_dim, cfg.qk_nope_head_dim, cfg.v_head_dim
        self.q_lora = cfg.q_lora_rank
        self.fused_a = LinearW(w, prefix + ".fused_lora_a_proj")  # [q_lora + r + dr, H] (or [r + dr, H])
        self.q_a_norm = w.get(prefix + ".q_a_layernorm.weight")
        self.kv_a_norm = w[prefix + ".kv_a_layernorm.weight"]
        self.q_b = LinearW(w, prefix + (".q_b_nope_rope_proj" if self.q_lora else ".q_proj"))
        self.w_uk = w[prefix + ".w_uk_t"]  # [h, dn, r]
        self.w_uv = w[prefix + ".w_uv"]    # [h, r, dv]
        self.o_proj = LinearW(w, prefix + ".o_proj")
        self.rope_cache = rope_cache
        self.scale = 1.0 / math.sqrt(self.dn + self.dr)
        rs = cfg.rope_scaling
        if rs.type == "yarn" and rs.mscale_all_dim:
            m = ref.yarn_mscale(rs.factor, rs.mscale_all_dim)
            self.scale *= m * m
        # sparse attention (DeepSeek-V3.2 / GLM DSA): a light multi-head scorer with its own key per token picks the
        # index_topk keys each query attends to. Reference: modules/attention (SparseMlaIndexer), DSA kernels in
        # 3rdparty/LLM_kernels; the scoring rule is score[q, t] = sum_h w[q, h] * relu(q_idx[q, h] . k_idx[t]).
        self.index_topk = cfg.index_topk if (cfg.index_topk and prefix + ".indexer.wq_b.weight" in w) else 0
        if self.index_topk:
            assert self.q_lora, "the sparse-attention indexer reads the low-rank query"
            ip = prefix + ".indexer"
            self.idx_wq, self.idx_wk = w[ip + ".wq_b.weight"], w[ip + ".wk.weight"]
            self.idx_kn_w, self.idx_kn_b = w[ip + ".k_norm.weight"], w[ip + ".k_norm.bias"]
            self.idx_wproj = w[ip + ".weights_proj.weight"]
            self.idx_h, self.idx_d = cfg.index_n_heads, cfg.index_head_dim

    def _fused_core_ok(self, q: torch.Tensor, cache: torch.Tensor) -> bool:
        ok = getattr(self, "_fused_ok", None)
        if ok is None:
            from ..ops import cuda_mla
            ok = bool(cuda_mla.fused_supported(q, cache, self.r, self.dr, self.dn, self.dv, self.h) and
                      self.w_uk.dtype == torch.bfloat16 and self.rope_cache is not None and
                      self.rope_cache.dtype == torch.float32)
            if ok:
                # [h, N, K] operands of the head-batched GEMMs: W_UK^T as [h, r, dn], W_UV as [h, dv, r]
                self.w_uk_nk = self.w_uk.transpose(1, 2).contiguous()
                self.w_uv_nk = self.w_uv.transpose(1, 2).contiguous()
            self._fused_ok = ok
        return ok and q.dtype == torch.bfloat16

    def _indexer(self, h: torch.Tensor, q_a: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
        """Indexer queries [T, Hi, Di], per-head weights [T, Hi] (scales folded in) and keys [T, Di]. The first
        qk_rope_head_dim entries of every indexer head are rotated (half-split layout)."""
        T = h.shape[0]
        q = (q_a @ self.idx_wq.t().to(q_a.dtype)).view(T, self.idx_h, self.idx_d)
        q = ref.apply_rope(q, cos, sin, False, self.dr)
        k = torch.nn.functional.layer_norm((h @ self.idx_wk.t().to(h.dtype)).float(), (self.idx_d,),
                                           self.idx_kn_w.float(), self.idx_kn_b.float(), 1e-6).to(h.dtype)
        k = ref.apply_rope(k.view(T, 1, self.idx_d), cos, sin, False, self.dr).view(T, self.idx_d)
        wts = (h @ self.idx_wproj.t().to(h.dtype)).float() * (self.idx_h ** -0.5) * (self.idx_d ** -0.5)
        return q, wts, k

    def core(self, h: torch.Tensor, meta, cache: torch.Tensor) -> torch.Tensor:
        T = h.shape[0]
        eps = self.cfg.mla_norm_eps or self.cfg.rms_norm_eps
        a = self.fused_a(h)
        if self.q_lora:
            q_a = ops.rms_norm(a[:, :self.q_lora].contiguous(), self.q_a_norm, eps)
            q = self.q_b(q_a)
            rest = a[:, self.q_lora:]
        else:
            q = self.q_b(h)
            rest = a
        latent = ops.rms_norm(rest[:, :self.r].contiguous(), self.kv_a_norm, eps)
        k_rope = rest[:, self.r:].contiguous()
        q = q.view(T, self.h, self.dn + self.dr)
        if not self.index_topk and h.is_cuda and self._fused_core_ok(q, cache):
            # absorb GEMMs, RoPE, cache append and attention as four kernels, no PyTorch op in between
            from ..ops import cuda_mla
            o = cuda_mla.mla_absorbed_attention(q, self.w_uk_nk, self.w_uv_nk, latent, k_rope, meta.positions,
                                                self.rope_cache, self.cfg.rope_interleaved, cache, meta, self.scale,
                                                self.dn, self.dr)
            return o.reshape(T, self.h * self.dv)
        q_nope, q_rope = q[..., :self.dn], q[..., self.dn:].contiguous()
        cs = self.rope_cache[meta.positions.long()]
        cos, sin = cs[:, :self.dr // 2], cs[:, self.dr // 2:]
        q_rope = ref.apply_rope(q_rope, cos, sin, self.cfg.rope_interleaved, self.dr)
        k_rope = ref.apply_rope(k_rope.view(T, 1, self.dr), cos, sin, self.cfg.rope_interleaved, self.dr).view(T, self.dr)
        q_lat = torch.einsum("thd,hdr->thr", q_nope.to(self.w_uk.dtype), self.w_uk)
        if self.index_topk:
            iq, iw, ik = self._indexer(h, q_a, cos, sin)
            flat = cache.view(-1, cache.shape[-1])
            flat[meta.slot_mapping.long()] = torch.cat((latent, k_rope, ik), -1).to(cache.dtype)
            o_lat = ref.mla_sparse_paged_attention(q_lat, q_rope, iq, iw, cache, meta.block_tables, meta.cu_q,
                                                   meta.kv_lens, self.scale, self.r + self.dr, self.index_topk)
        else:
            ops.mla_cache_append(latent, k_rope, meta.slot_mapping, cache)
            o_lat = ops.mla_paged_attention(q_lat.contiguous(), q_rope, cache, meta, self.scale)
        o = torch.einsum("thr,hrd->thd", o_lat.to(self.w_uv.dtype), self.w_uv)
        return o.reshape(T, self.h * self.dv)


class DenseFFN:
    """Gated (SwiGLU / GeGLU) or plain two-layer FFN; up projections column-parallel, down row-parallel."""

    def __init__(self, cfg: ModelConfig, w: Dict[str, torch.Tensor], prefix: str, tp: TPGroup):
        self.cfg = cfg
        self.tp = tp
        self.gated = cfg.gated_mlp
        self.up = LinearW(w, prefix + (".gate_up_proj" if self.gated else ".up_proj"))
        self.down = LinearW(w, prefix + ".down_proj")
        self.act = cfg.hidden_act

    def core(self, h: torch.Tensor) -> torch.Tensor:
        u = self.up(h)
        if self.gated:
            if self.act in ("silu", "swish"):
                return ops.silu_and_mul(u)
            return ref.gelu_and_mul(u)
        return ops.activation(u, self.act)


class MoEFFN:
    """Routed experts (+ optional shared expert). Experts are sharded over the expert-parallel group
    (here: the TP group); every rank sees all tokens, computes its local experts and the partial sums are
    combined by the all-reduce that follows (or by the fused dispatch/combine kernel when attached)."""

    def __init__(self, cfg: ModelConfig, w: Dict[str, torch.Tensor], prefix: str, tp: TPGroup):
        self.cfg = cfg
        self.tp = tp
        self.gate_w = w[prefix + ".gate.weight"]
        self.bias = w.get(prefix + ".gate.e_score_correction_bias")
        self.w_gate_up = w.get(prefix + ".experts.up_gate_proj.weight")  # [E_local, 2I, H]
        self.w_down = w.get(prefix + ".experts.down_proj.weight")        # [E_local, H, I]
        # 4-bit group-quantised experts (GPTQ / AWQ checkpoints): packed words [E_local, N, K / 8] + scales / zeros
        self.q4 = None
        if self.w_gate_up is None:
            e = prefix + ".experts."
            self.q4 = tuple((w[e + n + ".qweight"], w[e + n + ".scales"], w[e + n + ".zeros"])
                            for n in ("up_gate_proj", "down_proj"))
            self.w_gate_up, self.w_down = self.q4[0][0], self.q4[1][0]  # (shape carriers: E_local = dim 0)
        # block-scaled fp8 experts (DeepSeek-V3 checkpoints, or quant_method fp8): e4m3 weights + one fp32 scale per
        # 128 x 128 block; they stay in fp8 and every expert's two GEMMs run through the block-scaled fp8 GEMM
        self.pqs = (w.get(prefix + ".experts.up_gate_proj.pre_quant_scale"),   # [E_local, H] / [E_local, I]: AWQ
                    w.get(prefix + ".experts.down_proj.pre_quant_scale"))      # smoothing of W4A8 experts' inputs
        if self.q4 is None and w.get(prefix + ".experts.up_gate_proj.weight_scale_inv") is None:
            for i, n in enumerate(("up_gate_proj", "down_proj")):  # dense experts: folded into the weights once
                if self.pqs[i] is not None:
                    k = prefix + ".experts." + n
                    w[k + ".weight"] = (w[k + ".weight"].float() * self.pqs[i].float().unsqueeze(1)).to(w[k + ".weight"].dtype)
                    w.pop(k + ".pre_quant_scale")
            if any(p_ is not None for p_ in self.pqs):
                self.w_gate_up, self.w_down = (w[prefix + ".experts.up_gate_proj.weight"],
                                               w[prefix + ".experts.down_proj.weight"])
                self.pqs = (None, None)
        self.perm = w.get(prefix + ".expert_perm")  # logical -> physical expert ids (load-balanced placement)
        self._eplb_counts = None
        if os.environ.get("DUMP_EPLB_PATH"):
            self._eplb_counts = torch.zeros(cfg.num_experts, dtype=torch.int64)
            _EPLB_LAYERS[prefix] = self
        self.s_gate_up = w.get(prefix + ".experts.up_gate_proj.weight_scale_inv")
        self.s_down = w.get(prefix + ".experts.down_proj.weight_scale_inv")
        self.e_local = self.w_gate_up.shape[0]
        self.expert_offset = tp.ep_rank * self.e_local if self.e_local < cfg.num_experts else 0
        self.shared = None
        if cfg.num_shared_experts:
            self.shared = DenseFFN(cfg, w, prefix + ".shared_expert", tp)
            self.shared_gate = w.get(prefix + ".shared_expert_gate.weight")

    def partial(self, h: torch.Tensor) -> torch.Tensor:
        """Per-rank partial sum of the block output (needs a cross-rank sum when size > 1)."""
        c = self.cfg
        ep = self.tp.ep
        quantised = self.s_gate_up is not None or self.q4 is not None
        # block-scaled fp8 experts go through the peer-memory exchange with rows quantised before they leave
        fp8_ep = (quantised and ep is not None and hasattr(ep, "_moe_fp8") and self._grouped_fp8(h) and
                  h.shape[1] % 512 == 0)
        self._ep_kw = {"fp8_scales": (self.s_gate_up, self.s_down)} if fp8_ep else {}
        if quantised and not fp8_ep:
            if self.tp.ep_dp and self.e_local < c.num_experts:
                if not getattr(ep, "custom_experts", False):
                    raise NotImplementedError("the peer-memory expert exchange runs bf16 and block-scaled fp8 experts; "
                                              "other quantised experts under attention DP use the collective exchange")
            else:
                ep = None  # (int4 experts: local loop over the replicated tokens)
        if ep is not None and self.tp.ep_dp and self.e_local < c.num_experts:
            return self._dp_exchange(h, ep)
        if (ep is not None and h.is_cuda and h.dtype == torch.bfloat16 and self.e_local < c.num_experts and
                h.shape[0] <= ep.t_cap * ep.size):
            return self._partial_dispatch(h, ep)
        logits = ops.linear(h.float() if self.gate_w.dtype == torch.float32 else h, self.gate_w)
        if c.moe_router == "llama4":
            y = self._llama4_experts(h, logits)
        else:
            ids, wts = ops.moe_route(logits, c.num_experts_per_tok, c.scoring_func, c.norm_topk_prob, c.n_group,
                                     c.topk_group, c.routed_scaling_factor, self.bias)
            ids = self._place(ids)
            if self.s_gate_up is not None and self._grouped_fp8(h):
                # block-scaled fp8 experts: device-side sort + grouped fp8 tcgen05 GEMMs, no host round trip
                from ..ops import cuda_moe
                y = cuda_moe.moe_experts_fp8(h, ids, wts, self.w_gate_up, self.s_gate_up, self.w_down, self.s_down,
                                             self.expert_offset)
            elif self.s_gate_up is not None or self.q4 is not None:
                y = self._fp8_experts(h, ids, wts)
            else:
                y = ops.moe_experts(h, ids, wts, self.w_gate_up, self.w_down, self.expert_offset)
        if self.shared is not None:
            s = self.shared.down(self.shared.core(h), add_bias=self.tp.rank == 0)
            if self.shared_gate is not None:
                g = torch.sigmoid(ops.linear(h, self.shared_gate).float()).to(s.dtype)
                s = s * g
            y = y + s
        return y

    def _grouped_fp8(self, h: torch.Tensor) -> bool:
        ok = getattr(self, "_grouped_fp8_ok", None)
        if ok is None:
            from ..ops import cuda_moe
            ok = self._grouped_fp8_ok = bool(h.is_cuda and self.q4 is None and cuda_moe.supports_fp8(
                h, self.w_gate_up, self.s_gate_up, self.w_down, self.s_down))
        return ok and h.is_cuda and h.dtype == torch.bfloat16

    def _place(self, ids: torch.Tensor) -> torch.Tensor:
        """Router output (logical expert ids) -> the ids the expert kernels and the exchange work with. Counts the
        choices when a routing dump was asked for (DUMP_EPLB_PATH)."""
        if self._eplb_counts is not None and ids.numel():
            self._eplb_counts += torch.bincount(ids.reshape(-1).long().cpu(), minlength=self.cfg.num_experts)
        if self.perm is not None:
            return self.perm[ids.long()].to(ids.dtype)
        return ids

    def _fp8_experts(self, h: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor) -> torch.Tensor:
        """Local experts with quantised weights - block-scaled fp8 (activations quantised per token per 128 channels)
        or 4-bit group-quantised: tokens are grouped by expert on the host and each group goes through that
        format's two GEMMs. One launch pair per active expert, not a grouped kernel."""
        T, H = h.shape
        out = torch.zeros(T, H, dtype=torch.float32, device=h.device)
        local = (ids >= self.expert_offset) & (ids < self.expert_offset + self.e_local)
        tok, slot = local.nonzero(as_tuple=True)
        if tok.numel() == 0:
            return out.to(h.dtype)
        eid = (ids[tok, slot] - self.expert_offset).long()
        order = torch.argsort(eid, stable=True)
        tok, slot, eid = tok[order], slot[order], eid[order]
        counts = torch.bincount(eid, minlength=self.e_local).tolist()
        at = 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            t = tok[at:at + n]
            if self.q4 is not None:
                (q1, s1, z1), (q2, s2, z2) = self.q4
                g1, g2 = q1.shape[2] * 8 // s1.shape[2], q2.shape[2] * 8 // s2.shape[2]
                x = h[t] if self.pqs[0] is None else h[t] * self.pqs[0][e].to(h.dtype)
                a = ops.silu_and_mul(ops.linear_int4(x, q1[e], s1[e], z1[e], None, g1))
                if self.pqs[1] is not None:
                    a = a * self.pqs[1][e].to(a.dtype)
                y = ops.linear_int4(a, q2[e], s2[e], z2[e], None, g2).float()
            else:
                a = ops.silu_and_mul(ops.linear_fp8_block(h[t], self.w_gate_up[e], self.s_gate_up[e]))
                y = ops.linear_fp8_block(a, self.w_down[e], self.s_down[e]).float()
            out.index_add_(0, t, y * wts[t, slot[at:at + n]].unsqueeze(-1).float())
            at += n
        return out.to(h.dtype)

    def _llama4_experts(self, h: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        """Llama 4 routing: top-k on the raw logits, score = sigmoid(logit), and the score scales the expert's
        INPUT (the expert MLP is non-linear, so this is not the usual output weighting)."""
        k = self.cfg.num_experts_per_tok
        top, ids = torch.topk(logits.float(), k, dim=-1)
        score = torch.sigmoid(top)
        ones = torch.ones_like(score[:, :1])
        y = None
        for j in range(k):
            xj = (h.float() * score[:, j:j + 1]).to(h.dtype)
            yj = ops.moe_experts(xj, ids[:, j:j + 1].to(torch.int32).contiguous(), ones, self.w_gate_up, self.w_down,
                                 self.expert_offset)
            y = yj if y is None else y + yj
        return y

    def _dp_exchange(self, h: torch.Tensor, ep) -> torch.Tensor:
        """Attention data parallelism: ``h`` holds only this rank's tokens (possibly none); the routed experts are
        reached through the exchange, whose slot stride for this step was agreed by the DP coordinator."""
        c = self.cfg
        logits = ops.linear(h.float() if self.gate_w.dtype == torch.float32 else h, self.gate_w)
        ids, wts = ops.moe_route(logits, c.num_experts_per_tok, c.scoring_func, c.norm_topk_prob, c.n_group,
                                 c.topk_group, c.routed_scaling_factor, self.bias)
        ids = self._place(ids)
        kw = dict(getattr(self, "_ep_kw", {}))
        if not kw and (self.s_gate_up is not None or self.q4 is not None):
            kw["experts_fn"] = self._fp8_experts  # quantised local experts over the gathered rows
        s = None
        if self.shared is not None and h.shape[0]:
            s = self.shared.down(self.shared.core(h), add_bias=self.tp.rank == 0)
            if self.shared_gate is not None:
                s = s * torch.sigmoid(ops.linear(h, self.shared_gate).float()).to(s.dtype)
        if self.tp.size > 1:
            # a DP group that is tensor-parallel inside: every rank of the group holds the same rows, so one of them
            # sends them through the exchange and the others join it empty-handed; the block's output is a partial
            # sum over the group (the routed part counted once, the sliced shared expert on every rank)
            if self.tp.rank != 0:
                ep.moe(h[:0], ids[:0], wts[:0], self.w_gate_up, self.w_down, ep.step_stride, **kw)
                return s if s is not None else torch.zeros_like(h)
        return ep.moe(h, ids, wts, self.w_gate_up, self.w_down, ep.step_stride, add=s, **kw)

    def _partial_dispatch(self, h: torch.Tensor, ep) -> torch.Tensor:
        """Expert-parallel path: this rank routes only its own slice of the tokens, sends each row to the ranks
        hosting its experts and gets the weighted outputs back. The result keeps the "partial sum" contract of
        ``partial`` (rows owned by other ranks are zero here), so the reduce that follows is unchanged."""
        c = self.cfg
        T = h.shape[0]
        per = (T + ep.size - 1) // ep.size
        lo, hi = min(T, ep.rank * per), min(T, (ep.rank + 1) * per)
        mine = h[lo:hi]
        logits = ops.linear(mine.float() if self.gate_w.dtype == torch.float32 else mine, self.gate_w)
        ids, wts = ops.moe_route(logits, c.num_experts_per_tok, c.scoring_func, c.norm_topk_prob, c.n_group,
                                 c.topk_group, c.routed_scaling_factor, self.bias)
        ids = self._place(ids)
        y = torch.zeros_like(h)
        if self.shared is not None:
            s = self.shared.down(self.shared.core(h), add_bias=self.tp.rank == 0)
            if self.shared_gate is not None:
                s = s * torch.sigmoid(ops.linear(h, self.shared_gate).float()).to(s.dtype)
            y = s
        out = ep.moe(mine, ids, wts, self.w_gate_up, self.w_down, per, add=y[lo:hi] if hi > lo else None,
                     **getattr(self, "_ep_kw", {}))
        if hi > lo:
            y[lo:hi] = out
        return y
