"""ctypes bindings of the sm_100a kernel library (``_lib/libksana_kernels.so``).

Every function takes torch CUDA tensors, launches on the current torch stream and returns torch tensors.
There is no fallback here: if the library is missing or a launcher rejects a shape the call raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Dict, Optional, Tuple

import torch

from .. import _build
from . import gemm_tune
from . import reference as ref

_lib = None
launch_count = 0  # number of kernel-library launches issued (each is at least one CUDA kernel)


def lib():
    global _lib
    if _lib is None:
        path = _build.LIB / "libksana_kernels.so"
        if not path.exists():
            _build.build_cuda()
        if not path.exists():
            raise RuntimeError("libksana_kernels.so is missing: run `python -m ksanallm_b200._build`")
        _lib = ctypes.CDLL(str(path))
        for name in dir(_Sig):
            if name.startswith("ksana_"):
                fn = getattr(_lib, name)
                fn.argtypes, fn.restype = getattr(_Sig, name)
    return _lib


P, I, F, LL = c_void_p, c_int, c_float, c_longlong


class _Sig:
    ksana_read_error = ([I], ctypes.c_uint)
    ksana_sm_count = ([], I)
    ksana_gemm_bf16 = ([P, P, P, P, I, I, I, I, I, I, I, I, I, P, LL, P, I, P], I)
    ksana_gemm_bf16_swiglu = ([P, P, P, I, I, I, I, I, I, P], I)
    ksana_gemm_fp8_block = ([P, P, P, P, P, P, I, I, I, I, I, I, I, I, P, LL, P, I, P], I)
    ksana_moe_route = ([P, I, P, I, I, I, I, I, I, I, F, P, P, P], I)
    ksana_moe_permute = ([P, I, P, I, I, I, I, I, P, P, P, P, P], I)
    ksana_moe_grouped_gemm = ([P, P, P, P, I, I, I, I, P], I)
    ksana_moe_combine = ([P, P, P, I, I, I, P, P], I)
    ksana_moe_grouped_gemm_fp8 = ([P, I, P, I, P, P, P, P, I, I, I, I, P], I)
    ksana_silu_mul_quant_fp8 = ([P, I, P, I, P, I, I, P], I)
    ksana_gemm_int4_small = ([P, P, P, P, P, I, I, I, I, I, I, P, LL, P, I, I, P], I)
    ksana_gemm_int4 = ([P, P, P, P, P, I, I, I, I, I, I, P, LL, P, I, P], I)
    ksana_mla_decode = ([P, I, P, I, P, I, P, P, I, I, I, I, I, F, P, P, LL, P], I)
    ksana_mla_cache_append = ([P, I, P, I, P, P, I, I, I, P], I)
    ksana_rms_norm = ([P, I, P, I, P, P, I, I, I, F, P], I)
    ksana_silu_mul = ([P, I, P, I, I, I, P], I)
    ksana_embedding = ([P, P, P, I, I, I, F, P], I)
    ksana_rope_cache = ([P, I, P, I, P, I, P, P, P, P, P, P, F, I, I, I, I, I, I, I, I, F, F, P], I)
    ksana_quant_fp8_group = ([P, I, P, I, P, I, I, P], I)
    ksana_mxf8_sfa_bytes = ([I, I], LL)
    ksana_mxf8_sfb_bytes = ([I, I], LL)
    ksana_mxf8_pack_sfb = ([P, P, I, I, P, P], I)
    ksana_quant_fp8_ue8m0 = ([P, I, P, I, P, P, I, I, P], I)
    ksana_silu_mul_quant_ue8m0 = ([P, I, P, I, P, P, I, I, P], I)
    ksana_gemm_mxf8 = ([P, P, P, P, P, P, I, I, I, I, I, I, I, P], I)
    ksana_paged_decode = ([P, I, P, I, P, I, P, P, I, I, I, I, I, I, I, I, F, P, F, F, P, I, P, LL, P], I)
    ksana_paged_prefill = ([P, I, I, P, I, P, I, P, P, I, I, I, I, I, I, I, F, P, P, I, P], I)
    ksana_paged_decode_gqa = ([P, I, I, P, I, P, I, P, P, I, I, I, I, I, I, I, I, F, P, I, P, LL, P], I)
    ksana_paged_decode_gqa_set_variant = ([I], None)
    ksana_argmax = ([P, I, I, I, P, P], I)
    ksana_sample = ([P, I, I, I, P, P, P, P, P, P], I)
    ksana_gemm_bf16_batched = ([P, LL, LL, P, P, LL, LL, I, I, I, I, P], I)
    ksana_mla_rope_append = ([P, LL, I, I, P, P, I, P, I, P, P, P, P, I, I, I, I, I, I, P], I)
    ksana_block_copy = ([P, P, I, P, I, LL, P], I)
    ksana_logits_process = ([P, I, I, I, P, P, P, P, P, P, P, P, P, P, P, I, P], I)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code}")


def read_error(clear: bool = True) -> int:
    """Status word written by kernels whose bounded waits expired (0 = ok)."""
    return int(lib().ksana_read_error(1 if clear else 0))


# ---- per-device workspaces ---------------------------------------------------------------------------
class _Workspace:
    def __init__(self, device: torch.device):
        self.gemm_ws = torch.empty(32 << 20, dtype=torch.float32, device=device)       # 128 MiB split-K partials
        self.gemm_counters = torch.zeros(8192, dtype=torch.int32, device=device)
        self.attn_ws = torch.empty(32 << 20, dtype=torch.float32, device=device)       # split-KV partials


_workspaces: Dict[int, _Workspace] = {}


def workspace(device: torch.device) -> _Workspace:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(idx)
    if ws is None:
        ws = _workspaces[idx] = _Workspace(torch.device("cuda", idx))
    return ws


# ---- GEMM -----------------------------------------------------------------------------------------------
def gemm_bf16(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, out_dtype=None,
              bn: int = 0, splits: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[M, N] = x[M, K] @ w[N, K]^T (+ bias). x may be a row-strided view (last dim contiguous)."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
    M, K = x.shape
    N = w.shape[0]
    if x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    if w.stride(1) != 1 or w.stride(0) % 8 or w.data_ptr() % 16:
        w = w.contiguous()
    out_dtype = out_dtype or torch.bfloat16
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=x.device)
    if M == 0:
        return out
    if bn == 0 and splits == 0 and gemm_tune._MAP:
        bn, splits = gemm_tune.lookup(M, N, K)
    ws = workspace(x.device)
    code = lib().ksana_gemm_bf16(_ptr(x), _ptr(w), _ptr(out), _ptr(bias), M, N, K, x.stride(0), w.stride(0),
                                 out.stride(0), 1 if out.dtype == torch.float32 else 0, bn, splits, _ptr(ws.gemm_ws),
                                 ws.gemm_ws.numel(), _ptr(ws.gemm_counters), ws.gemm_counters.numel(), _stream())
    _check(code, f"gemm_bf16 M={M} N={N} K={K}")
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    if x.dtype == torch.float32 or weight.dtype == torch.float32:
        # fp32 router / probe paths: tiny GEMMs outside the bf16 hot path
        y = x.float() @ weight.float().t()
        return y if bias is None else y + bias.float()
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    N, K = weight.shape
    if N % 8 or K % 8:
        y = ref.linear(x2, weight, bias)
    else:
        y = gemm_bf16(x2, weight, bias)
    return y.view(*lead, N)


def gemm_fp8_block(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws_inv: torch.Tensor,
                   bias: Optional[torch.Tensor] = None, out_dtype=None, splits: int = 0,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Block-scaled fp8 GEMM: xq [M, K] e4m3 + xs [M, K/128]; wq [N, K] e4m3 + ws_inv [ceil(N/128), K/128]."""
    M, K = xq.shape
    N = wq.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or torch.bfloat16, device=xq.device)
    if M == 0:
        return out
    w = workspace(xq.device)
    code = lib().ksana_gemm_fp8_block(_ptr(xq), _ptr(xs), _ptr(wq), _ptr(ws_inv), _ptr(out), _ptr(bias), M, N, K,
                                      xq.stride(0), wq.stride(0), out.stride(0),
                                      1 if out.dtype == torch.float32 else 0, splits, _ptr(w.gemm_ws),
                                      w.gemm_ws.numel(), _ptr(w.gemm_counters), w.gemm_counters.numel(), _stream())
    _check(code, f"gemm_fp8_block M={M} N={N} K={K}")
    return out


def interleave_gate_up(w: torch.Tensor) -> torch.Tensor:
    """[2 I, K] (gate rows, then up rows) -> the same rows interleaved in groups of 16, the layout of gemm_bf16_swiglu."""
    I_ = w.shape[0] // 2
    return torch.stack((w[:I_].view(I_ // 16, 16, -1), w[I_:].view(I_ // 16, 16, -1)), 1).reshape(w.shape).contiguous()


def gemm_bf16_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor) -> torch.Tensor:
    """SiLU(x Wg^T) * (x Wu^T) in one kernel: x [M, K] bf16, w_interleaved [2 I, K] from interleave_gate_up -> [M, I]."""
    M, K = x.shape
    N = w_interleaved.shape[0]
    out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=x.device)
    _check(lib().ksana_gemm_bf16_swiglu(_ptr(x), _ptr(w_interleaved), _ptr(out), M, N, K, x.stride(0),
                                        w_interleaved.stride(0), out.stride(0), _stream()), "gemm_bf16_swiglu")
    return out


def linear_fp8_block(x, wq, w_scale_inv, bias=None, sfb=None, pow2=False):
    from . import cuda_fp8
    return cuda_fp8.linear_fp8_block(x, wq, w_scale_inv, bias, sfb, pow2)


def linear_int4(x, packed, scales, zeros, bias=None, group=128, sz=None):
    from . import cuda_int4
    return cuda_int4.linear_int4(x, packed, scales, zeros, bias, group, sz=sz)


# ---- elementwise -------------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    if x.dtype != torch.bfloat16:
        return ref.rms_norm(x, weight, eps, residual)
    shape = x.shape
    H = shape[-1]
    x2 = x.reshape(-1, H)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    r2 = None
    if residual is not None:
        r2 = residual.view(-1, H)
    out = torch.empty(x2.shape, dtype=x.dtype, device=x.device)
    code = lib().ksana_rms_norm(_ptr(x2), x2.stride(0), _ptr(r2), r2.stride(0) if r2 is not None else 0, _ptr(weight),
                                _ptr(out), out.stride(0), x2.shape[0], H, float(eps), _stream())
    if code == -1:
        return ref.rms_norm(x, weight, eps, residual)
    _check(code, "rms_norm")
    return out.view(shape)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    T, two_i = x.shape
    I_ = two_i // 2
    out = torch.empty(T, I_, dtype=x.dtype, device=x.device)
    code = lib().ksana_silu_mul(_ptr(x), x.stride(0), _ptr(out), out.stride(0), T, I_, _stream())
    if code == -1:
        return ref.silu_and_mul(x)
    _check(code, "silu_and_mul")
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    if table.dtype != torch.bfloat16 or table.shape[1] % 8:
        return ref.embedding(ids, table, scale)
    T, H = ids.numel(), table.shape[1]
    out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    _check(lib().ksana_embedding(_ptr(ids), _ptr(table), _ptr(out), T, H, table.shape[0], float(scale), _stream()),
           "embedding")
    return out


def rope_qknorm_cache(q, k, v, positions, cos_sin, slot_mapping, kv_cache, q_norm_w=None, k_norm_w=None, eps=1e-6,
                      interleaved=False, rotary_dim=0, k_scale=1.0, v_scale=1.0) -> None:
    T, h, d = q.shape
    hk = k.shape[1]
    if q.dtype != torch.bfloat16 or kv_cache.dtype not in (torch.bfloat16, torch.float8_e4m3fn):
        return ref.rope_qknorm_cache(q, k, v, positions, cos_sin, slot_mapping, kv_cache, q_norm_w, k_norm_w, eps,
                                     interleaved, rotary_dim, k_scale, v_scale)
    assert q.stride(2) == 1 and q.stride(1) == d and k.stride(1) == d and v.stride(1) == d
    rd = (rotary_dim or d) if cos_sin is not None else 0
    kind = 0 if kv_cache.dtype == torch.bfloat16 else 1
    code = lib().ksana_rope_cache(_ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(positions),
                                  _ptr(cos_sin), _ptr(slot_mapping), _ptr(kv_cache), _ptr(q_norm_w), _ptr(k_norm_w),
                                  float(eps), T, h, hk, d, rd, 1 if interleaved else 0, kv_cache.shape[3], kind,
                                  float(k_scale), float(v_scale), _stream())
    _check(code, "rope_qknorm_cache")


def quant_fp8_group(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    T, K = x.shape
    q = torch.empty(T, K, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(T, K // 128, dtype=torch.float32, device=x.device)
    _check(lib().ksana_quant_fp8_group(_ptr(x), x.stride(0), _ptr(q), q.stride(0), _ptr(s), T, K, _stream()),
           "quant_fp8_group")
    return q, s


# ---- attention ----------------------------------------------------------------------------------------------
GQA_TENSOR_CORE_MIN_GROUP = int(os.environ.get("KSANA_GQA_TC_MIN_GROUP", "4"))


def paged_attention(q, kv_cache, meta, scale, alibi_slopes=None, k_scale=1.0, v_scale=1.0, window=0) -> torch.Tensor:
    T, h, d = q.shape
    nb, _, hk, bs, _ = kv_cache.shape
    supported = (q.dtype == torch.bfloat16 and d == 128 and bs == 16 and window == 0 and
                 kv_cache.dtype in (torch.bfloat16, torch.float8_e4m3fn))
    if not supported:
        return ref.paged_attention(q, kv_cache, meta.block_tables, meta.cu_q, meta.kv_lens, scale, alibi_slopes,
                                   k_scale, v_scale, window)
    out = torch.empty(T, h, d, dtype=q.dtype, device=q.device)
    ldq, ldo = q.stride(0), out.stride(0)
    kind = 0 if kv_cache.dtype == torch.bfloat16 else 1
    n_pre, n_dec = meta.num_prefill, meta.num_decode
    cu = meta.cu_q_host
    if n_pre and kind == 1:
        # fp8 KV: prefill chunks go through the decode-style kernel row by row is too slow; dequantised path
        return ref.paged_attention(q, kv_cache, meta.block_tables, meta.cu_q, meta.kv_lens, scale, alibi_slopes,
                                   k_scale, v_scale, window)
    if n_pre:
        max_q = int((cu[1:n_pre + 1] - cu[:n_pre]).max())
        code = lib().ksana_paged_prefill(_ptr(q), ldq, T, _ptr(kv_cache), nb, _ptr(meta.block_tables), meta.max_blocks,
                                         _ptr(meta.cu_q), _ptr(meta.kv_lens), 0, n_pre, max_q, h, hk, d, bs,
                                         float(scale), _ptr(alibi_slopes), _ptr(out), ldo, _stream())
        _check(code, "paged_prefill")
    if n_dec:
        max_q = int((cu[n_pre + 1:n_pre + n_dec + 1] - cu[n_pre:n_pre + n_dec]).max())
        max_kv = int(meta.kv_lens_host[n_pre:n_pre + n_dec].max())
        ws = workspace(q.device)
        code = -1
        if kind == 0 and alibi_slopes is None and h // hk >= GQA_TENSOR_CORE_MIN_GROUP and (h // hk) * max_q <= 128:
            # grouped-query decode on the tensor cores: the group's heads are the rows of one MMA operand
            code = lib().ksana_paged_decode_gqa(_ptr(q), ldq, T, _ptr(kv_cache), nb, _ptr(meta.block_tables),
                                                meta.max_blocks, _ptr(meta.cu_q), _ptr(meta.kv_lens), n_pre, n_dec, max_q,
                                                max_kv, h, hk, d, bs, float(scale), _ptr(out), ldo, _ptr(ws.attn_ws),
                                                ws.attn_ws.numel(), _stream())
            if code not in (0, -1, -6):
                _check(code, "paged_decode_gqa")
        if code == 0:
            global launch_count
            launch_count += 1
            return out
        code = lib().ksana_paged_decode(_ptr(q), ldq, _ptr(kv_cache), kind, _ptr(meta.block_tables), meta.max_blocks,
                                        _ptr(meta.cu_q), _ptr(meta.kv_lens), n_pre, n_dec, max_q, max_kv, h, hk, d, bs,
                                        float(scale), _ptr(alibi_slopes), float(k_scale), float(v_scale), _ptr(out), ldo,
                                        _ptr(ws.attn_ws), ws.attn_ws.numel(), _stream())
        _check(code, "paged_decode")
    return out


def mla_cache_append(latent, k_rope, slot_mapping, cache):
    from . import cuda_mla
    return cuda_mla.mla_cache_append(latent, k_rope, slot_mapping, cache)


def mla_paged_attention(q_latent, q_rope, cache, meta, scale):
    from . import cuda_mla
    return cuda_mla.mla_paged_attention(q_latent, q_rope, cache, meta, scale)


# ---- MoE ------------------------------------------------------------------------------------------------------
def moe_route(logits, top_k, scoring="softmax", norm_topk=False, n_group=1, topk_group=1, routed_scale=1.0,
              correction_bias=None):
    from . import cuda_moe
    return cuda_moe.moe_route(logits, top_k, scoring, norm_topk, n_group, topk_group, routed_scale, correction_bias)


def moe_experts(x, ids, weights, w_gate_up, w_down, expert_offset=0):
    from . import cuda_moe
    return cuda_moe.moe_experts(x, ids, weights, w_gate_up, w_down, expert_offset)


# ---- sampling ---------------------------------------------------------------------------------------------------
def argmax(logits: torch.Tensor) -> torch.Tensor:
    if logits.dtype != torch.float32:
        logits = logits.float()
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _check(lib().ksana_argmax(_ptr(logits), logits.stride(0), B, V, _ptr(out), _stream()), "argmax")
    return out


def sample(logits, temperature, top_k, top_p, uniform) -> torch.Tensor:
    if logits.dtype != torch.float32:
        logits = logits.float()
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _check(lib().ksana_sample(_ptr(logits), logits.stride(0), B, V, _ptr(temperature.float()), _ptr(top_k.int()),
                              _ptr(top_p.float()), _ptr(uniform.float()), _ptr(out), _stream()), "sample")
    return out


def logits_process(x, hist, row_off, prompt_len, fparams, iparams, edit_off, edit_tok, edit_val, ban_off, ban_tok,
                   bitmask) -> torch.Tensor:
    """In-place penalties / n-gram bans / edits / bans / grammar mask on fp32 logits ``x`` [rows, V] (one kernel for
    the whole step). The other arguments are device tensors laid out as csrc/cuda/sampling.cu describes."""
    assert x.dtype == torch.float32 and x.stride(1) == 1
    L, V = x.shape
    _check(lib().ksana_logits_process(_ptr(x), x.stride(0), L, V, _ptr(hist), _ptr(row_off), _ptr(prompt_len),
                                      _ptr(fparams), _ptr(iparams), _ptr(edit_off), _ptr(edit_tok), _ptr(edit_val),
                                      _ptr(ban_off), _ptr(ban_tok), _ptr(bitmask),
                                      bitmask.shape[1] if bitmask is not None else 0, _stream()), "logits_process")
    return x


def block_copy(src_ptrs: torch.Tensor, dst_ptrs: torch.Tensor, pairs: torch.Tensor, block_bytes: int) -> None:
    """Copies cache blocks ``pairs[i] = (src, dst)`` of every layer in one launch. ``src_ptrs`` / ``dst_ptrs``:
    int64 device tensors with one base address per layer (device memory or mapped pinned host memory)."""
    _check(lib().ksana_block_copy(_ptr(src_ptrs), _ptr(dst_ptrs), src_ptrs.numel(), _ptr(pairs), pairs.shape[0],
                                  int(block_bytes), _stream()), "block_copy")
