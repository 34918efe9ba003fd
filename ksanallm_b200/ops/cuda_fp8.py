"""fp8 block-scaled linear: per-token 1 x 128 activation quantisation kernel + block-scaled tcgen05 GEMM
(csrc/cuda/gemm_fp8_block.cu). Shapes the kernel does not take (K not a multiple of 128, N not a multiple of 8)
are dequantised and sent through the bf16 GEMM."""
from __future__ import annotations

import torch

from . import reference as ref


def linear_fp8_block(x, wq, w_scale_inv, bias=None):
    from . import cuda
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    T, K = x2.shape
    N = wq.shape[0]
    if K % 128 == 0 and N % 8 == 0 and x2.dtype == torch.bfloat16 and wq.stride(1) == 1 and wq.stride(0) % 16 == 0:
        xq, xs = cuda.quant_fp8_group(x2)
        y = cuda.gemm_fp8_block(xq, xs, wq, w_scale_inv.contiguous(), bias)
        return y.view(*lead, N)
    w = ref.dequant_fp8_block_weight(wq, w_scale_inv).to(torch.bfloat16)
    y = cuda.gemm_bf16(x2.contiguous().to(torch.bfloat16), w, bias)
    return y.view(*lead, N)
