"""Binding of the native dense-layer executor (csrc/cuda/dense_executor.cu): the whole decoder stack of a step is
launched by one C call instead of ~8 Python-level kernel wrappers per layer.

Eligible models: dense (no MoE / MLA) RMSNorm + RoPE decoders with a gated SiLU FFN, bf16 weights or 128 x 128
block-scaled e4m3 weights (all four linears of every layer alike), head_dim 128 and the 16-token KV block, on one GPU or tensor-parallel with the single-kernel fused GEMM + reduce-scatter path. Anything
else keeps the Python layer code in models/transformer.py (same kernels, launched one by one).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import numpy as np
import torch

from ..ops import cuda as kcuda

P, I, F, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


class _Layer(ctypes.Structure):
    _fields_ = [(n, P) for n in ("wqkv", "bqkv", "wo", "ln2", "wgu", "wdown", "next_ln", "q_norm", "k_norm",
                                 "kv_cache", "sqkv", "so", "sgu", "sdown", "fqkv", "fo", "fgu", "fdown", "wgu_il")]


class _Model(ctypes.Structure):
    _fields_ = [("hidden", I), ("heads", I), ("kv_heads", I), ("head_dim", I), ("inter", I), ("n_layers", I),
                ("eps", F), ("rotary_dim", I), ("rope_interleaved", I), ("block_size", I), ("num_blocks", I),
                ("kv_kind", I), ("attn_scale", F), ("k_scale", F), ("v_scale", F), ("rope_cache", P),
                ("rank", I), ("ws", I), ("rows_cap", I), ("comm_ctas", I), ("recv", P), ("hbuf", P), ("sig", P),
                ("hbuf_mc", P), ("partial", P), ("partial_mc", P), ("two_kernel_max_tokens", I), ("ll_recv", P), ("ll_recv2", P),
                ("ll_recv2_mc", P), ("ll_half_words", LL), ("ll_rows_cap", I), ("ll_max_tokens", I),
                ("ll_one_shot", I), ("qkv_buf", P), ("attn_buf", P), ("gu_buf", P), ("act_buf", P), ("proj_buf", P),
                ("h_buf", P * 2), ("gemm_ws", P), ("gemm_ws_floats", LL), ("gemm_counters", P), ("n_counters", I),
                ("attn_ws", P), ("attn_ws_floats", LL), ("sig_words", I), ("a8_buf", P), ("sa_buf", P), ("a8_cols", I),
                ("fp8_pow2", I), ("mx_min_rows", I), ("layers", P)]


class _Step(ctypes.Structure):
    _fields_ = [("positions", P), ("slot_mapping", P), ("block_tables", P), ("cu_q", P), ("kv_lens", P),
                ("total_tokens", I), ("num_prefill", I), ("num_decode", I), ("max_blocks", I), ("max_q_prefill", I),
                ("max_q_decode", I), ("max_kv_decode", I), ("split_seq", I), ("split_row", I), ("num_prefill_b", I),
                ("num_decode_b", I), ("max_q_prefill_b", I), ("max_q_decode_b", I), ("max_kv_decode_b", I)]


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class DenseExecutor:
    @staticmethod
    def eligible(model) -> bool:
        cfg, tp = model.cfg, model.tp
        if os.environ.get("KSANA_DISABLE_NATIVE_EXECUTOR", "0") == "1" or os.environ.get("KSANA_LIBRARY_BASELINE") == "1":
            return False
        if model.device.type != "cuda" or model.dtype != torch.bfloat16 or not model.layers or model.norm_w is None:
            return False
        if getattr(model, "num_cache_layers", len(model.layers)) != len(model.layers):
            return False  # cross-layer KV sharing
        if (cfg.use_mla or cfg.norm_type != "rmsnorm" or cfg.residual_scale != 1.0 or cfg.head_dim != 128 or
                cfg.position_encoding not in ("rope", "none") or not cfg.gated_mlp or
                cfg.hidden_act not in ("silu", "swish") or cfg.sliding_window or
                cfg.qk_norm_after_rope or cfg.qk_l2_norm or cfg.cla_share_factor or cfg.rope_layers or cfg.attn_temperature_tuning):
            return False
        for layer in model.layers:
            if layer.is_moe or not hasattr(layer.attn, "qkv"):
                return False
            lins = (layer.attn.qkv, layer.attn.o_proj, layer.ffn.up, layer.ffn.down)
            kind = model.layers[0].attn.qkv.kind
            if kind not in ("dense", "fp8_block") or any(l.kind != kind for l in lins):
                return False
            if layer.attn.o_proj.bias is not None:
                return False
            if kind == "fp8_block":
                if tp.size > 1 and (tp.fused is None or tp.fused.partial is None):
                    return False
                for l in lins:
                    w, sc = l.weight, l.scale_inv
                    if (w.shape[1] % 128 or w.shape[0] % 8 or not w.is_contiguous() or sc.dtype != torch.float32 or
                            not sc.is_contiguous() or tuple(sc.shape) != ((w.shape[0] + 127) // 128, w.shape[1] // 128)):
                        return False
            if layer.ffn.up.bias is not None or layer.ffn.down.bias is not None or layer.attn.alibi is not None:
                return False
            if layer.ln2 is None or getattr(layer, "ln2_b", None) is not None:
                return False
            if layer.attn.k_scale != 1.0 or layer.attn.v_scale != 1.0:
                return False  # per-layer fp8 KV scales: Python layer path
        if tp.size > 1:
            fc = tp.fused
            if fc is None or not fc.single_kernel or fc.hidden % 256 or fc.hidden > 9216 or fc.hidden != cfg.hidden_size:
                return False
        return True

    def __init__(self, model):
        self.model = model
        cfg, tp = model.cfg, model.tp
        self.tp = tp
        self.H = cfg.hidden_size
        a0 = model.layers[0].attn
        self.h, self.hk, self.d = a0.h, a0.hk, a0.d
        self.inter = model.layers[0].ffn.down.weight.shape[1]
        n = len(model.layers)
        self._layers = (_Layer * n)()
        # power-of-two scales only if every fp8 weight has them: the activation quantiser is chosen per model
        pow2 = all(getattr(l, "pow2", False) for layer in model.layers
                   for l in (layer.attn.qkv, layer.attn.o_proj, layer.ffn.up, layer.ffn.down))
        for i, layer in enumerate(model.layers):
            L = self._layers[i]
            nxt = model.layers[i + 1].ln1 if i + 1 < n else model.norm_w
            L.wqkv, L.bqkv = _p(layer.attn.qkv.weight), _p(layer.attn.qkv.bias)
            L.wo, L.ln2 = _p(layer.attn.o_proj.weight), _p(layer.ln2)
            L.wgu, L.wdown = _p(layer.ffn.up.weight), _p(layer.ffn.down.weight)
            L.next_ln = _p(nxt)
            L.q_norm, L.k_norm = _p(layer.attn.q_norm), _p(layer.attn.k_norm)
            L.kv_cache = None
            if layer.attn.qkv.kind == "fp8_block":
                L.sqkv, L.so = _p(layer.attn.qkv.scale_inv), _p(layer.attn.o_proj.scale_inv)
                L.sgu, L.sdown = _p(layer.ffn.up.scale_inv), _p(layer.ffn.down.scale_inv)
                if pow2:
                    L.fqkv, L.fo = _p(layer.attn.qkv.sfb()), _p(layer.attn.o_proj.sfb())
                    L.fgu, L.fdown = _p(layer.ffn.up.sfb()), _p(layer.ffn.down.sfb())
        self.fp8 = model.layers[0].attn.qkv.kind == "fp8_block"
        # KSANA_FUSED_SWIGLU=1: keep a second copy of every gate_up weight with gate / up rows interleaved in groups of
        # 16, so prefill-sized steps run SiLU-mul as the GEMM's epilogue (costs the memory of the gate_up weights again)
        self._wgu_il = []
        if os.environ.get("KSANA_FUSED_SWIGLU", "0") == "1" and not self.fp8 and self.inter % 16 == 0:
            for i, layer in enumerate(model.layers):
                w = layer.ffn.up.weight
                I_ = w.shape[0] // 2
                il = torch.stack((w[:I_].view(I_ // 16, 16, -1), w[I_:].view(I_ // 16, 16, -1)), 1).reshape(w.shape)
                self._wgu_il.append(il.contiguous())
                self._layers[i].wgu_il = self._wgu_il[-1].data_ptr()
        m = self._m = _Model()
        m.hidden, m.heads, m.kv_heads, m.head_dim, m.inter, m.n_layers = self.H, self.h, self.hk, self.d, self.inter, n
        m.eps = float(cfg.rms_norm_eps)
        m.rotary_dim = int(cfg.rotary_dim or cfg.head_dim)
        m.rope_interleaved = 1 if cfg.rope_interleaved else 0
        m.attn_scale = float(a0.scale)
        m.k_scale = m.v_scale = 1.0
        m.rope_cache = _p(model.rope_cache)
        m.rank, m.ws = tp.rank, tp.size
        if tp.size > 1:
            fc = tp.fused
            m.rows_cap, m.comm_ctas = fc.rows_cap, fc.comm_ctas
            m.recv = ctypes.cast(fc._recv_ptrs, P)
            m.hbuf = ctypes.cast(fc._hbuf_ptrs, P)
            m.sig = ctypes.cast(fc._sig_ptrs, P)
            m.hbuf_mc = fc.hbuf_mc or None
            m.partial = ctypes.cast(fc._partial_ptrs, P)
            m.partial_mc = fc.partial_mc or None
            m.two_kernel_max_tokens = fc.two_kernel_max_tokens
            m.sig_words = fc.sig_words
            m.ll_recv = ctypes.cast(fc._ll_recv_ptrs, P)
            m.ll_recv2 = ctypes.cast(fc._ll_recv2_ptrs, P)
            m.ll_recv2_mc = fc.ll_recv2_mc or None
            m.ll_half_words = fc.ll_half_words
            m.ll_rows_cap, m.ll_max_tokens, m.ll_one_shot = fc.ll_rows_cap, fc.ll_max_tokens, int(fc.ll_one_shot)
        ws = kcuda.workspace(model.device)
        self._ws = ws
        m.gemm_ws, m.gemm_ws_floats = _p(ws.gemm_ws), ws.gemm_ws.numel()
        m.gemm_counters, m.n_counters = _p(ws.gemm_counters), ws.gemm_counters.numel()
        m.attn_ws, m.attn_ws_floats = _p(ws.attn_ws), ws.attn_ws.numel()
        m.layers = ctypes.cast(self._layers, P)
        if self.fp8:
            from ..ops import cuda_fp8
            m.fp8_pow2, m.mx_min_rows = int(pow2), cuda_fp8.MXF8_MIN_ROWS
        self.cap = 0
        self.overlap_min_tokens = int(os.environ.get("KSANA_OVERLAP_MIN_TOKENS", "1024"))
        self._bufs: List[torch.Tensor] = []
        self._kv_key = None
        self._step = _Step()
        lib = kcuda.lib()
        lib.ksana_dense_forward.argtypes = [P, P, P, P, I, I, P, P, P, P, P]
        lib.ksana_dense_forward.restype = I
        self._fn = lib.ksana_dense_forward
        self._out = P()
        self._fail = I()
        self._launches = I()

    def _ensure(self, T: int) -> None:
        if T <= self.cap:
            return
        cap = (max(T, 1024) + 1023) // 1024 * 1024
        dev, bf = self.model.device, torch.bfloat16
        nqkv = (self.h + 2 * self.hk) * self.d
        mk = lambda cols: torch.empty(cap, cols, dtype=bf, device=dev)  # noqa: E731
        qkv, attn, gu, act = mk(nqkv), mk(self.h * self.d), mk(2 * self.inter), mk(self.inter)
        self._bufs = [qkv, attn, gu, act]
        m = self._m
        if self.fp8:
            cols = max(self.H, self.h * self.d, self.inter)
            a8 = torch.empty(cap, cols, dtype=torch.uint8, device=dev)
            sa = torch.empty(cap + 256, cols // 128, dtype=torch.float32, device=dev)
            self._bufs += [a8, sa]
            m.a8_buf, m.sa_buf, m.a8_cols = _p(a8), _p(sa), cols
        m.qkv_buf, m.attn_buf, m.gu_buf, m.act_buf = _p(qkv), _p(attn), _p(gu), _p(act)
        if self.tp.size == 1:
            proj, h0, h1 = mk(self.H), mk(self.H), mk(self.H)
            self._bufs += [proj, h0, h1]
            m.proj_buf = _p(proj)
            m.h_buf[0], m.h_buf[1] = _p(h0), _p(h1)
            self._h = (h0, h1)
        self.cap = cap

    def _bind_kv(self, kv_caches) -> None:
        # every layer's pointer is part of the key: a new cache (a second engine on the same model) may start at the
        # address the old one had while its other layers, or its block count, differ
        key = tuple(c.data_ptr() for c in kv_caches) + tuple(kv_caches[0].shape)
        if key == self._kv_key:
            return
        for i in range(len(self.model.layers)):
            self._layers[i].kv_cache = kv_caches[i].data_ptr()
        c = kv_caches[0]
        m = self._m
        m.num_blocks, m.block_size = c.shape[0], c.shape[3]
        m.kv_kind = 0 if c.dtype == torch.bfloat16 else 1
        self._kv_key = key

    def can_run(self, meta, kv_caches, n_layers: int) -> bool:
        T = meta.total_tokens
        if T == 0 or n_layers == 0 or kv_caches[0].dim() != 5 or kv_caches[0].shape[3] != 16:
            return False
        if getattr(meta, "mrope_positions", None) is not None:
            return False
        if kv_caches[0].dtype != torch.bfloat16 and meta.num_prefill:
            return False  # fp8 cache prefill chunks take the dequantising path
        if self.tp.size > 1:
            fc = self.tp.fused
            return T <= min(8192, fc.max_tokens)
        return True

    def _overlap_split(self, cu, n_seq: int, T: int) -> int:
        """Sequence index at which a prefill-sized tensor-parallel step is cut into two half-batches that run on two
        streams (the collectives of one half overlap the compute of the other); 0: run the step as one batch."""
        fc = self.tp.fused if self.tp.size > 1 else None
        if fc is None or n_seq < 2 or T < self.overlap_min_tokens or fc.partial is None:
            return 0
        split = int(np.abs(cu[1:n_seq] - T // 2).argmin()) + 1
        rows_a = int(cu[split])
        if min(rows_a, T - rows_a) < max(256, T // 4):
            return 0
        return split

    def forward(self, meta, kv_caches, h: torch.Tensor, residual: torch.Tensor, n_layers: int) -> torch.Tensor:
        """h: normalised input of layer 0, residual: the residual stream (both [T, H], contiguous); returns the
        normalised output of layer ``n_layers - 1`` (a view of an internal buffer, valid until the next call)."""
        T = meta.total_tokens
        self._ensure(T)
        self._bind_kv(kv_caches)
        s = self._step
        s.positions, s.slot_mapping = meta.positions.data_ptr(), meta.slot_mapping.data_ptr()
        s.block_tables, s.cu_q, s.kv_lens = meta.block_tables.data_ptr(), meta.cu_q.data_ptr(), meta.kv_lens.data_ptr()
        n_pre, n_dec = meta.num_prefill, meta.num_decode
        s.total_tokens, s.num_prefill, s.num_decode, s.max_blocks = T, n_pre, n_dec, meta.max_blocks
        cu, kl = meta.cu_q_host, meta.kv_lens_host

        def maxima(lo, hi):
            """(prefill count, decode count, max q prefill, max q decode, max kv decode) of sequences [lo, hi)."""
            p_hi = min(hi, n_pre)
            q = cu[lo + 1:hi + 1] - cu[lo:hi]
            n_p, n_d = max(p_hi - lo, 0), hi - max(lo, n_pre)
            mq_p = int(q[:n_p].max()) if n_p > 0 else 0
            mq_d = int(q[n_p:].max()) if n_d > 0 else 0
            mkv = int(kl[max(lo, n_pre):hi].max()) if n_d > 0 else 0
            return n_p, max(n_d, 0), mq_p, mq_d, mkv

        n_seq = n_pre + n_dec
        split = self._overlap_split(cu, n_seq, T)
        s.split_seq, s.split_row = split, int(cu[split]) if split else 0
        s.num_prefill, s.num_decode, s.max_q_prefill, s.max_q_decode, s.max_kv_decode = maxima(0, split or n_seq)
        if split:
            (s.num_prefill_b, s.num_decode_b, s.max_q_prefill_b, s.max_q_decode_b,
             s.max_kv_decode_b) = maxima(split, n_seq)
        fc = self.tp.fused if self.tp.size > 1 else None
        epoch = (ctypes.c_uint * 2)(0, 0)
        if fc is not None:
            epoch[0], epoch[1] = fc.epoch & 0xFFFFFFFF, fc.ll_seq & 0xFFFFFFFF
            self._m.two_kernel_max_tokens = fc.two_kernel_max_tokens
            self._m.ll_max_tokens = fc.ll_max_tokens
        rc = self._fn(ctypes.byref(self._m), ctypes.byref(s), h.data_ptr(), residual.data_ptr(), 0, n_layers,
                      epoch, ctypes.byref(self._out), ctypes.byref(self._fail),
                      ctypes.byref(self._launches), torch.cuda.current_stream().cuda_stream)
        kcuda.launch_count += self._launches.value
        if fc is not None:
            # every collective of the stack took its epoch (and buffer half) from the shared counters
            fc.epoch, fc.ll_seq = epoch[0], epoch[1]
        if rc != 0:
            raise RuntimeError(f"native dense forward failed at layer {rc // 100 - 1}, step {rc % 100}, "
                               f"code {self._fail.value}")
        if fc is not None:
            return fc.hbuf[:T]
        out = self._out.value
        return (self._h[0] if out == self._h[0].data_ptr() else self._h[1])[:T]
