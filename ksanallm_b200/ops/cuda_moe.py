"""MoE on the GPU: router kernel, device-side counting sort by expert, grouped tcgen05 expert GEMMs, combine.
No host synchronisation: expert row offsets stay on the device and the grouped GEMM walks them itself."""
from __future__ import annotations

from typing import Dict

import torch

from . import reference as ref

_meta: Dict[tuple, torch.Tensor] = {}


def moe_route(logits, top_k, scoring="softmax", norm_topk=False, n_group=1, topk_group=1, routed_scale=1.0,
              correction_bias=None):
    from . import cuda
    T, E = logits.shape
    if E > 512 or top_k > 16 or n_group > 32 or E % max(n_group, 1):
        return ref.moe_route(logits, top_k, scoring, norm_topk, n_group, topk_group, routed_scale, correction_bias)
    x = logits if logits.dtype == torch.float32 else logits.float()
    if x.stride(1) != 1:
        x = x.contiguous()
    ids = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    b = None if correction_bias is None else correction_bias.float().contiguous()
    code = cuda.lib().ksana_moe_route(cuda._ptr(x), x.stride(0), cuda._ptr(b), T, E, top_k,
                                      1 if scoring == "sigmoid" else 0, 1 if norm_topk else 0, n_group, topk_group,
                                      float(routed_scale), cuda._ptr(ids), cuda._ptr(w), cuda._stream())
    cuda._check(code, "moe_route")
    return ids, w


def expert_pipeline(x, ids, w_gate_up, w_down, expert_offset=0):
    """Sort the (token, slot) pairs by local expert and run gate_up -> SiLU*mul -> down on the sorted rows.
    Returns (y [T*k, H] sorted expert outputs, pos [T*k] sorted row of each pair or -1 for non-local experts)."""
    from . import cuda
    T, H = x.shape
    k = ids.shape[1]
    E_local, two_i, _ = w_gate_up.shape
    I_ = two_i // 2
    dev = x.device
    key = (dev.index, E_local)
    meta = _meta.get(key)
    if meta is None:
        meta = _meta[key] = torch.zeros(3 * E_local + 2, dtype=torch.int32, device=dev)
    n = T * k
    pos = torch.empty(n, dtype=torch.int32, device=dev)
    row_src = torch.empty(n, dtype=torch.int32, device=dev)
    xs = torch.empty(n, H, dtype=torch.bfloat16, device=dev)
    lib = cuda.lib()
    st = cuda._stream()
    idc = ids if ids.is_contiguous() else ids.contiguous()
    cuda._check(lib.ksana_moe_permute(cuda._ptr(x), x.stride(0), cuda._ptr(idc), T, k, H, expert_offset, E_local,
                                      cuda._ptr(meta), cuda._ptr(pos), cuda._ptr(row_src), cuda._ptr(xs), st),
                "moe_permute")
    offsets = meta[E_local:2 * E_local + 1]
    h1 = torch.empty(n, two_i, dtype=torch.bfloat16, device=dev)
    cuda._check(lib.ksana_moe_grouped_gemm(cuda._ptr(xs), cuda._ptr(w_gate_up), cuda._ptr(h1), cuda._ptr(offsets),
                                           E_local, n, two_i, H, st), "moe_grouped_gemm(gate_up)")
    a = cuda.silu_and_mul(h1)
    y = torch.empty(n, H, dtype=torch.bfloat16, device=dev)
    cuda._check(lib.ksana_moe_grouped_gemm(cuda._ptr(a), cuda._ptr(w_down), cuda._ptr(y), cuda._ptr(offsets), E_local,
                                           n, H, I_, st), "moe_grouped_gemm(down)")
    return y, pos


def supports(x, w_gate_up, w_down) -> bool:
    two_i, H = w_gate_up.shape[1], x.shape[1]
    return (x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and two_i % 128 == 0 and H % 128 == 0 and
            (two_i // 2) % 8 == 0 and w_gate_up.is_contiguous() and w_down.is_contiguous())


def moe_experts(x, ids, weights, w_gate_up, w_down, expert_offset=0):
    """x [T, H] bf16; ids/weights [T, k]; w_gate_up [E_local, 2I, H]; w_down [E_local, H, I] (bf16, contiguous)."""
    from . import cuda
    if not supports(x, w_gate_up, w_down):
        return ref.moe_experts(x, ids, weights, w_gate_up, w_down, expert_offset)
    T, H = x.shape
    k = ids.shape[1]
    y, pos = expert_pipeline(x, ids, w_gate_up, w_down, expert_offset)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    wc = weights if weights.dtype == torch.float32 and weights.is_contiguous() else weights.float().contiguous()
    cuda._check(cuda.lib().ksana_moe_combine(cuda._ptr(y), cuda._ptr(pos), cuda._ptr(wc), T, k, H, cuda._ptr(out),
                                             cuda._stream()), "moe_combine")
    return out


def supports_fp8(x, wq_gate_up, s_gate_up, wq_down, s_down) -> bool:
    """Block-scaled fp8 experts the grouped kernel takes: e4m3 weights [E, 2I, H] / [E, H, I] with one scale per
    128 x 128 block, H and I multiples of 128 (gate and up blocks then tile the fused matrix exactly)."""
    if wq_gate_up is None or s_gate_up is None or wq_gate_up.dtype != torch.float8_e4m3fn:
        return False
    E, two_i, H = wq_gate_up.shape
    I_ = two_i // 2
    return (x.dtype == torch.bfloat16 and H % 128 == 0 and I_ % 128 == 0 and wq_gate_up.is_contiguous() and
            wq_down.is_contiguous() and tuple(s_gate_up.shape) == (E, two_i // 128, H // 128) and
            tuple(s_down.shape) == (E, H // 128, I_ // 128))


def pack_fp8_rows(x: torch.Tensor) -> torch.Tensor:
    """[T, H] bf16 -> [T, H + H / 32] bytes: the row's e4m3 values (one scale per 128 channels) followed by its fp32
    scales. This is what travels between ranks under expert parallelism (about half the bytes of the bf16 row) and
    what the grouped fp8 GEMM reads in place."""
    from . import cuda
    T, H = x.shape
    q, s = cuda.quant_fp8_group(x if x.is_contiguous() else x.contiguous())
    packed = torch.empty(T, H + H // 32, dtype=torch.uint8, device=x.device)
    packed[:, :H] = q.view(torch.uint8)
    packed[:, H:] = s.view(torch.uint8).view(T, H // 32)
    return packed


def expert_pipeline_fp8(x, ids, wq_gate_up, s_gate_up, wq_down, s_down, expert_offset=0, packed=False):
    """The expert pipeline for block-scaled fp8 weights, entirely on the device: sort the (token, slot) pairs by
    local expert, quantise the gathered rows per token per 128 channels, grouped fp8 GEMM (gate_up), fused
    SiLU * mul + re-quantisation, grouped fp8 GEMM (down). Returns (y [T*k, H] bf16, pos [T*k]).
    ``packed``: x already holds ``pack_fp8_rows`` rows ([T, (H + H / 32) / 2] viewed as bf16); they are sorted as
    they are and the GEMM reads values and scales out of the sorted rows."""
    from . import cuda
    T = x.shape[0]
    k = ids.shape[1]
    E_local, two_i, H = wq_gate_up.shape
    I_ = two_i // 2
    dev = x.device
    key = (dev.index, E_local)
    meta = _meta.get(key)
    if meta is None:
        meta = _meta[key] = torch.zeros(3 * E_local + 2, dtype=torch.int32, device=dev)
    n = T * k
    W = x.shape[1]  # bf16 elements per row that the sort moves
    pos = torch.empty(n, dtype=torch.int32, device=dev)
    row_src = torch.empty(n, dtype=torch.int32, device=dev)
    xs = torch.empty(n, W, dtype=torch.bfloat16, device=dev)
    lib = cuda.lib()
    st = cuda._stream()
    idc = ids if ids.is_contiguous() else ids.contiguous()
    cuda._check(lib.ksana_moe_permute(cuda._ptr(x), x.stride(0), cuda._ptr(idc), T, k, W, expert_offset, E_local,
                                      cuda._ptr(meta), cuda._ptr(pos), cuda._ptr(row_src), cuda._ptr(xs), st),
                "moe_permute")
    offsets = meta[E_local:2 * E_local + 1]
    if packed:
        assert W * 2 == H + H // 32
        a_ptr, lda, sa_ptr, sa_stride = xs.data_ptr(), W * 2, xs.data_ptr() + H, W // 2
    else:
        xq, xsc = cuda.quant_fp8_group(xs)
        a_ptr, lda, sa_ptr, sa_stride = xq.data_ptr(), H, xsc.data_ptr(), H // 128
    h1 = torch.empty(n, two_i, dtype=torch.bfloat16, device=dev)
    sg = s_gate_up if s_gate_up.is_contiguous() else s_gate_up.contiguous()
    sd = s_down if s_down.is_contiguous() else s_down.contiguous()
    cuda._check(lib.ksana_moe_grouped_gemm_fp8(a_ptr, lda, sa_ptr, sa_stride, cuda._ptr(wq_gate_up), cuda._ptr(sg),
                                               cuda._ptr(h1), cuda._ptr(offsets), E_local, n, two_i, H, st),
                "moe_grouped_gemm_fp8(gate_up)")
    aq = torch.empty(n, I_, dtype=torch.float8_e4m3fn, device=dev)
    asc = torch.empty(n, I_ // 128, dtype=torch.float32, device=dev)
    cuda._check(lib.ksana_silu_mul_quant_fp8(cuda._ptr(h1), two_i, cuda._ptr(aq), I_, cuda._ptr(asc), n, I_, st),
                "silu_mul_quant_fp8")
    y = torch.empty(n, H, dtype=torch.bfloat16, device=dev)
    cuda._check(lib.ksana_moe_grouped_gemm_fp8(cuda._ptr(aq), I_, cuda._ptr(asc), I_ // 128, cuda._ptr(wq_down),
                                               cuda._ptr(sd), cuda._ptr(y), cuda._ptr(offsets), E_local, n, H, I_, st),
                "moe_grouped_gemm_fp8(down)")
    cuda.launch_count += 8
    return y, pos


def moe_experts_fp8(x, ids, weights, wq_gate_up, s_gate_up, wq_down, s_down, expert_offset=0):
    """x [T, H] bf16; ids / weights [T, k]; block-scaled e4m3 expert weights. No host synchronisation."""
    from . import cuda
    T, H = x.shape
    k = ids.shape[1]
    y, pos = expert_pipeline_fp8(x, ids, wq_gate_up, s_gate_up, wq_down, s_down, expert_offset)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device)
    wc = weights if weights.dtype == torch.float32 and weights.is_contiguous() else weights.float().contiguous()
    cuda._check(cuda.lib().ksana_moe_combine(cuda._ptr(y), cuda._ptr(pos), cuda._ptr(wc), T, k, H, cuda._ptr(out),
                                             cuda._stream()), "moe_combine")
    return out
