"""fp8 block-scaled linear: per-token 1 x 128 activation quantisation kernel + block-scaled tcgen05 GEMM.

Two GEMM kernels: csrc/cuda/gemm_fp8_block.cu takes any fp32 scales (per-K-block promotion on the CUDA cores);
csrc/cuda/gemm_mxf8.cu needs power-of-two scales on both operands and lets the tensor core apply them
(kind::mxf8f6f4.block_scale), which is the fast path for prefill-sized products. A weight whose block scales are powers
of two (``pow2``) gets power-of-two activation scales from both kernels, so a layer computes the same function whatever
the batch size. Shapes neither kernel takes (K not a multiple of 128, N not a multiple of 8) are dequantised and sent
through the bf16 GEMM."""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from . import reference as ref

# products with at least this many rows take the scaled tensor-core kernel (measured faster from 128 rows on; below,
# the split-K kernel streams the weight with more CTAs)
MXF8_MIN_ROWS = int(os.environ.get("KSANA_MXF8_MIN_ROWS", "128"))


def _lib():
    from . import cuda
    return cuda.lib()


def pack_sfb(w_scale_inv: torch.Tensor, N: int, K: int) -> torch.Tensor:
    """Power-of-two block scales [ceil(N / 128), K / 128] -> the per-tile byte layout of the scaled GEMM."""
    from . import cuda
    lib = _lib()
    sw = w_scale_inv.float().contiguous()
    out = torch.empty(int(lib.ksana_mxf8_sfb_bytes(N, K)), dtype=torch.uint8, device=sw.device)
    bad = torch.zeros(1, dtype=torch.int32, device=sw.device)
    cuda._check(lib.ksana_mxf8_pack_sfb(cuda._ptr(sw), cuda._ptr(out), N, K, cuda._ptr(bad), cuda._stream()), "pack_sfb")
    if int(bad.item()):
        raise ValueError("pack_sfb: the block scales are not powers of two")
    return out


def quant_fp8_ue8m0(x: torch.Tensor, scales: bool = True,
                    packed: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """x [T, K] bf16 -> (q e4m3, fp32 scales [T, K / 128] or None, packed scale bytes or None)."""
    from . import cuda
    lib = _lib()
    T, K = x.shape
    q = torch.empty(T, K, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(T, K // 128, dtype=torch.float32, device=x.device) if scales else None
    sfa = torch.empty(int(lib.ksana_mxf8_sfa_bytes(T, K)), dtype=torch.uint8, device=x.device) if packed else None
    cuda._check(lib.ksana_quant_fp8_ue8m0(cuda._ptr(x), x.stride(0), cuda._ptr(q), q.stride(0), cuda._ptr(s),
                                          cuda._ptr(sfa), T, K, cuda._stream()), "quant_fp8_ue8m0")
    return q, s, sfa


def silu_mul_quant_ue8m0(x: torch.Tensor, scales: bool = True, packed: bool = False):
    """x [T, 2 I] bf16 (gate | up) -> SiLU(gate) * up quantised like ``quant_fp8_ue8m0``."""
    from . import cuda
    lib = _lib()
    T, two_i = x.shape
    I_ = two_i // 2
    q = torch.empty(T, I_, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(T, I_ // 128, dtype=torch.float32, device=x.device) if scales else None
    sfa = torch.empty(int(lib.ksana_mxf8_sfa_bytes(T, I_)), dtype=torch.uint8, device=x.device) if packed else None
    cuda._check(lib.ksana_silu_mul_quant_ue8m0(cuda._ptr(x), x.stride(0), cuda._ptr(q), q.stride(0), cuda._ptr(s),
                                               cuda._ptr(sfa), T, I_, cuda._stream()), "silu_mul_quant_ue8m0")
    return q, s, sfa


def gemm_mxf8(xq: torch.Tensor, sfa: torch.Tensor, wq: torch.Tensor, sfb: torch.Tensor,
              bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, variant: int = 0) -> torch.Tensor:
    """``variant`` 0 / 1: one CTA per tile; 2: the CTA-pair kernel."""
    from . import cuda
    M, K = xq.shape
    N = wq.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=xq.device)
    if M == 0:
        return out
    cuda._check(_lib().ksana_gemm_mxf8(cuda._ptr(xq), cuda._ptr(sfa), cuda._ptr(wq), cuda._ptr(sfb), cuda._ptr(out),
                                       cuda._ptr(bias), M, N, K, xq.stride(0), wq.stride(0), out.stride(0),
                                       variant, cuda._stream()), f"gemm_mxf8 M={M} N={N} K={K}")
    return out


def linear_fp8_block(x, wq, w_scale_inv, bias=None, sfb=None, pow2=False):
    from . import cuda
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    T, K = x2.shape
    N = wq.shape[0]
    if K % 128 == 0 and N % 8 == 0 and x2.dtype == torch.bfloat16 and wq.stride(1) == 1 and wq.stride(0) % 16 == 0:
        if pow2 and sfb is not None and T >= MXF8_MIN_ROWS:
            xq, _, sfa = quant_fp8_ue8m0(x2, scales=False, packed=True)
            return gemm_mxf8(xq, sfa, wq, sfb, bias).view(*lead, N)
        if pow2:
            xq, xs, _ = quant_fp8_ue8m0(x2)
        else:
            xq, xs = cuda.quant_fp8_group(x2)
        y = cuda.gemm_fp8_block(xq, xs, wq, w_scale_inv.contiguous(), bias)
        return y.view(*lead, N)
    w = ref.dequant_fp8_block_weight(wq, w_scale_inv).to(torch.bfloat16)
    y = cuda.gemm_bf16(x2.contiguous().to(torch.bfloat16), w, bias)
    return y.view(*lead, N)
