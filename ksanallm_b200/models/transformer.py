"""Generic decoder-only transformer over a paged KV cache.

One implementation parameterised by :class:`ModelConfig` expresses every dense / MoE / MLA family
the reference ships as separate C++ model classes (src/ksana_llm/models/**; CommonModel::Forward,
common_model.cpp:424-478; SimpleDecoderLayer, simple_decoder_layer.cpp:22-100; DeepSeek-V3 decoder and
MTP layer, deepseek_v3_model.cpp:84-174, 231-288). The residual add is deferred: each block returns its
un-normalised output and the next normalisation consumes ``(x, residual)`` in one fused kernel - for
TP>1 fused with the row-parallel GEMM's reduction (see parallel.comm.TPGroup.row_linear_add_norm).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.model_config import ModelConfig
from ..ops import reference as ref
from ..parallel.comm import TPGroup
from .layers import Attention, DenseFFN, LinearW, MLAttention, MoEFFN


class DecoderLayer:
    def __init__(self, cfg: ModelConfig, w: Dict[str, torch.Tensor], idx: int, tp: TPGroup, rope_cache,
                 prefix: Optional[str] = None):
        p = prefix or f"model.layers.{idx}"
        self.cfg, self.tp, self.idx = cfg, tp, idx
        self.ln1 = w[p + ".input_layernorm.weight"]
        self.ln1_b = w.get(p + ".input_layernorm.bias")
        self.ln2 = w[p + ".post_attention_layernorm.weight"]
        self.ln2_b = w.get(p + ".post_attention_layernorm.bias")
        if cfg.use_mla:
            self.attn = MLAttention(cfg, w, p + ".self_attn", idx, tp, rope_cache)
        else:
            self.attn = Attention(cfg, w, p + ".self_attn", idx, tp, rope_cache)
        self.is_moe = cfg.is_moe_layer(idx) and (p + ".mlp.gate.weight") in w
        self.ffn = MoEFFN(cfg, w, p + ".mlp", tp) if self.is_moe else DenseFFN(cfg, w, p + ".mlp", tp)

    def _norm(self, x, wgt, bias, residual):
        if self.cfg.norm_type == "layernorm":
            return ops.layer_norm(x, wgt, bias, self.cfg.rms_norm_eps, residual)
        return ops.rms_norm(x, wgt, self.cfg.rms_norm_eps, residual)

    def forward(self, h: torch.Tensor, residual: torch.Tensor, meta, kv_cache, next_norm, next_norm_b=None):
        """h: normalised block input; residual: running residual stream (updated in place).
        Returns the next block's normalised input: both row-parallel GEMMs (o_proj, down_proj) are issued
        through the TP group's fused "GEMM -> reduce -> residual add -> RMSNorm" entry, the second one
        already applying the NEXT block's (or the model's final) norm weight."""
        cfg, tp = self.cfg, self.tp
        fused_ok = cfg.norm_type == "rmsnorm" and cfg.residual_scale == 1.0
        a = self.attn.core(h, meta, kv_cache)
        if fused_ok:
            h = tp.row_linear_add_norm(a, self.attn.o_proj, residual, self.ln2, cfg.rms_norm_eps)
        else:
            o = tp.row_linear(a, self.attn.o_proj)
            if cfg.residual_scale != 1.0:
                o = o * cfg.residual_scale
            h = self._norm(o, self.ln2, self.ln2_b, residual)
        if self.is_moe:
            y = self.ffn.partial(h)
            if fused_ok and next_norm is not None:
                return tp.reduce_add_norm(y, residual, next_norm, cfg.rms_norm_eps)
            y = tp.all_reduce(y)
        else:
            f = self.ffn.core(h)
            if fused_ok and next_norm is not None:
                return tp.row_linear_add_norm(f, self.ffn.down, residual, next_norm, cfg.rms_norm_eps)
            y = tp.row_linear(f, self.ffn.down)
        if cfg.residual_scale != 1.0:
            y = y * cfg.residual_scale
        if next_norm is None:
            residual.add_(y)
            return residual
        if cfg.norm_type == "layernorm":
            return ops.layer_norm(y, next_norm, next_norm_b, cfg.rms_norm_eps, residual)
        return ops.rms_norm(y, next_norm, cfg.rms_norm_eps, residual)


class TransformerModel:
    """Embedding -> layers -> final norm -> (vocab-sharded) lm_head."""

    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], tp: Optional[TPGroup] = None,
                 max_positions: Optional[int] = None, layer_range: Optional[range] = None):
        self.cfg = cfg
        self.tp = tp or TPGroup()
        self.w = weights
        self.embed = weights["model.embed_tokens.weight"]
        self.device = self.embed.device
        self.dtype = self.embed.dtype
        self.pos_embed = weights.get("model.embed_positions.weight")
        maxp = max_positions or cfg.max_position_embeddings
        self.rope_cache = None
        if cfg.position_encoding == "rope":
            rd = cfg.qk_rope_head_dim if cfg.use_mla else (cfg.rotary_dim or cfg.head_dim)
            self.rope_cache = ref.build_rope_cache(rd, maxp, cfg.rope_theta, cfg.rope_scaling, self.device)
        self.progress = None  # optional per-layer completion tracker (prefill/decode disaggregation)
        self.layer_ids = list(layer_range) if layer_range is not None else list(range(cfg.num_layers))
        self.layers: List[DecoderLayer] = [DecoderLayer(cfg, weights, i, self.tp, self.rope_cache)
                                           for i in self.layer_ids]
        self.norm_w = weights.get("model.norm.weight")
        self.norm_b = weights.get("model.norm.bias")
        self.lm_head = weights.get("lm_head.weight")
        if self.lm_head is None:
            self.lm_head = self.embed  # tied
        # MTP (next-n) layers, DeepSeek style
        self.mtp_layers = []
        for j in range(cfg.num_nextn_predict_layers):
            p = f"model.layers.{cfg.num_layers + j}"
            if p + ".eh_proj.weight" in weights:
                self.mtp_layers.append(MTPLayer(cfg, weights, cfg.num_layers + j, self.tp, self.rope_cache))

    # ---- KV cache -------------------------------------------------------------------------------
    @property
    def num_cache_layers(self) -> int:
        return len(self.layers) + len(self.mtp_layers)

    def kv_block_bytes(self, block_size: int, kv_dtype: Optional[torch.dtype] = None) -> int:
        """Bytes of one block across all local layers (used to size the block pool)."""
        cfg = self.cfg
        esz = torch.empty(0, dtype=kv_dtype or self.dtype).element_size()
        if cfg.use_mla:
            per_layer = block_size * (cfg.kv_lora_rank + cfg.qk_rope_head_dim + cfg.index_head_dim * bool(cfg.index_topk)) * esz
        else:
            hk = max(cfg.num_kv_heads // self.tp.size, 1)
            per_layer = 2 * hk * block_size * cfg.head_dim * esz
        return per_layer * self.num_cache_layers

    def allocate_kv_cache(self, num_blocks: int, block_size: int, kv_dtype: Optional[torch.dtype] = None):
        cfg = self.cfg
        dt = kv_dtype or self.dtype
        caches = []
        for _ in range(self.num_cache_layers):
            if cfg.use_mla:
                # with a sparse-attention indexer every cache row also carries the token's indexer key
                width = cfg.kv_lora_rank + cfg.qk_rope_head_dim + (cfg.index_head_dim if cfg.index_topk else 0)
                c = torch.zeros(num_blocks, block_size, width, dtype=dt, device=self.device)
            else:
                hk = max(cfg.num_kv_heads // self.tp.size, 1)
                c = torch.zeros(num_blocks, 2, hk, block_size, cfg.head_dim, dtype=dt, device=self.device)
            caches.append(c)
        return caches

    # ---- forward --------------------------------------------------------------------------------
    def embed_tokens(self, meta, refit=None) -> torch.Tensor:
        x = ops.embedding(meta.input_ids, self.embed, self.cfg.emb_scale)
        if self.pos_embed is not None:
            x = x + self.pos_embed[meta.positions.long()]
        if refit is not None:
            # multimodal: rows of precomputed embeddings replace token embeddings at given positions
            for pos, emb in refit:
                x[pos:pos + emb.shape[0]] = emb.to(x.dtype)
        return x

    def forward(self, meta, kv_caches, refit=None, cutoff_layer: Optional[int] = None,
                hidden_in: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Returns the final normalised hidden states [T, H]. ``self.last_residual`` then holds the
        un-normalised residual stream (the "transformer" probe target).

        Pipeline stages: ``hidden_in`` is the residual stream received from the previous stage (no embedding
        lookup); a stage built without ``model.norm.weight`` (not the last one) returns the un-normalised residual
        stream for the next stage."""
        x = self.embed_tokens(meta, refit) if hidden_in is None else hidden_in
        layers = self.layers if cutoff_layer is None else self.layers[:cutoff_layer]
        residual = x
        if not layers:
            self.last_residual = residual
            return self._final_norm_only(residual)
        first = layers[0]
        h = first._norm(x, first.ln1, first.ln1_b, None)
        if h.data_ptr() == residual.data_ptr():
            residual = x.clone()
        native = self._native_executor()
        if native is not None and cutoff_layer is None and native.can_run(meta, kv_caches, len(layers)):
            if not residual.is_contiguous():
                residual = residual.contiguous()
            h = native.forward(meta, kv_caches, h.contiguous(), residual, len(layers))
            self.last_residual = residual
            if self.progress is not None:
                self.progress.record(len(layers) - 1)  # one launch covers the stack: every layer reports together
            return h
        for li, layer in enumerate(layers):
            nxt = layers[li + 1] if li + 1 < len(layers) else None
            nw, nb = (nxt.ln1, nxt.ln1_b) if nxt is not None else (self.norm_w, self.norm_b)
            h = layer.forward(h, residual, meta, kv_caches[li], nw, nb)
            if self.progress is not None:
                self.progress.record(li)  # parallel.transfer.LayerProgressTracker: KV of layer li may leave now
        self.last_residual = residual
        return h

    def _native_executor(self):
        """The one-call-per-step C++ executor for eligible dense models (models/native_executor.py), created on
        first use; None when the model or the environment rules it out."""
        ex = getattr(self, "_native", False)
        if ex is False:
            from .native_executor import DenseExecutor
            ex = self._native = DenseExecutor(self) if DenseExecutor.eligible(self) else None
        return ex

    def _final_norm_only(self, x):
        if self.norm_w is None:
            return x
        if self.cfg.norm_type == "layernorm":
            return ops.layer_norm(x, self.norm_w, self.norm_b, self.cfg.rms_norm_eps)
        return ops.rms_norm(x, self.norm_w, self.cfg.rms_norm_eps)

    def compute_logits(self, hidden: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """fp32 logits for the selected rows; vocab shards are gathered across the TP group."""
        h = hidden if rows is None else hidden.index_select(0, rows.long())
        logits = ops.linear(h, self.lm_head)
        if self.tp.size > 1 and self.lm_head.shape[0] < self.cfg.vocab_size:
            logits = self.tp.all_gather(logits, dim=-1)
        logits = logits.float()
        if self.cfg.logit_scale != 1.0:
            logits = logits * self.cfg.logit_scale
        return logits[:, :self.cfg.vocab_size]

    def greedy_tokens(self, hidden: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """argmax over the full vocabulary without materialising gathered logits on every rank:
        local (max, index) pairs are exchanged instead (reference: greedy.cu:240-424 +
        common_model.cpp:591-617)."""
        h = hidden.index_select(0, rows.long())
        logits = ops.linear(h, self.lm_head).float()
        if self.tp.size == 1 or self.lm_head.shape[0] >= self.cfg.vocab_size:
            return ops.argmax(logits[:, :self.cfg.vocab_size])
        shard = self.lm_head.shape[0]
        v, i = logits.max(dim=-1)
        pair = torch.stack((v, (i + self.tp.rank * shard).float()), dim=-1)
        allp = self.tp.all_gather(pair.unsqueeze(0), dim=0)  # [tp, B, 2]
        best = allp[..., 0].argmax(dim=0)
        return allp[..., 1].gather(0, best.unsqueeze(0)).squeeze(0).to(torch.int32)


class MTPLayer:
    """DeepSeek next-token-prediction module: h' = Layer(eh_proj([RMSNorm(emb(t+1)) | RMSNorm(h)]))."""

    def __init__(self, cfg: ModelConfig, w, idx: int, tp: TPGroup, rope_cache):
        p = f"model.layers.{idx}"
        self.cfg, self.tp = cfg, tp
        self.enorm = w[p + ".enorm.weight"]
        self.hnorm = w[p + ".hnorm.weight"]
        self.eh_proj = LinearW(w, p + ".eh_proj")
        self.layer = DecoderLayer(cfg, w, idx, tp, rope_cache)
        self.final_norm = w[p + ".shared_head.norm.weight"]

    def forward(self, embeds: torch.Tensor, prev_hidden: torch.Tensor, meta, kv_cache,
                return_residual: bool = False):
        """Returns the module's output after its head norm; with ``return_residual`` also the un-normalised output,
        which is the ``prev_hidden`` of the next draft step when the module is applied repeatedly."""
        eps = self.cfg.rms_norm_eps
        e = ops.rms_norm(embeds, self.enorm, eps)
        h = ops.rms_norm(prev_hidden, self.hnorm, eps)
        x = self.eh_proj(torch.cat((e, h), dim=-1))
        residual = x.clone()
        hn = ops.rms_norm(x, self.layer.ln1, eps)
        out = self.layer.forward(hn, residual, meta, kv_cache, self.final_norm)
        return (out, residual) if return_residual else out
