"""int4 group-quantised weight-only linear (GPTQ / AWQ formats after repacking): tcgen05 GEMM that dequantises
inside its pipeline (csrc/cuda/gemm_int4.cu)."""
from __future__ import annotations

import torch

from . import reference as ref


def supports(K: int, N: int, group: int) -> bool:
    return K % 64 == 0 and group % 64 == 0 and K % group == 0 and N % 8 == 0


def pack_scale_zero(scales, zeros):
    """[N, G] scales and zeros -> [N, G, 2] fp32 (scale, zero) pairs, the form the kernel loads."""
    return torch.stack((scales.float(), zeros.float()), dim=-1).contiguous()


def linear_int4(x, packed, scales, zeros, bias=None, group=128, force_splits=0, sz=None):
    """``packed`` is either the plain [N, K/8] word matrix (tiled here on every call: tests and one-off use) or the
    4-d pre-tiled form of ``reference.tile_int4`` that the model layers keep after loading."""
    from . import cuda
    lead = x.shape[:-1]
    K = x.shape[-1]
    N = scales.shape[0]
    x2 = x.reshape(-1, K)
    if x.dtype != torch.bfloat16 or not supports(K, N, group) or packed.dtype != torch.int32:
        plain = packed if packed.dim() == 2 else ref.untile_int4(packed, N)
        w = ref.dequant_int4_group(plain, scales, zeros, group).to(torch.bfloat16)
        return cuda.gemm_bf16(x2.contiguous(), w, bias).view(*lead, N)
    if packed.dim() == 2:
        packed = ref.tile_int4(packed)
    if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    if sz is None:
        sz = pack_scale_zero(scales, zeros)
    M = x2.shape[0]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    ws = cuda.workspace(x.device)
    if M <= 64:
        # decode-sized: weights on the M side of the MMA, dequantised straight into TMEM
        code = cuda.lib().ksana_gemm_int4_small(cuda._ptr(x2), cuda._ptr(packed), cuda._ptr(sz), cuda._ptr(bias),
                                                cuda._ptr(out), M, N, K, x2.stride(0), N, group, cuda._ptr(ws.gemm_ws),
                                                ws.gemm_ws.numel(), cuda._ptr(ws.gemm_counters),
                                                ws.gemm_counters.numel(), force_splits, cuda._stream())
        cuda._check(code, "gemm_int4_small")
        return out.view(*lead, N)
    code = cuda.lib().ksana_gemm_int4(cuda._ptr(x2), cuda._ptr(packed), cuda._ptr(sz), cuda._ptr(bias),
                                      cuda._ptr(out), M, N, K, x2.stride(0), N, group, cuda._ptr(ws.gemm_ws),
                                      ws.gemm_ws.numel(), cuda._ptr(ws.gemm_counters), force_splits, cuda._stream())
    cuda._check(code, "gemm_int4")
    return out.view(*lead, N)
