"""fp8 block-scaled linear: per-token 1x128 activation quantisation kernel + GEMM.

The GEMM currently dequantises the 128x128 block-scaled weight to bf16 and runs the bf16 tcgen05 kernel;
activations go through the same quantise/dequantise round trip as the block-scaled kernel would apply, so the
numerics match the fp32 reference of the format.
"""
from __future__ import annotations

import torch

from . import reference as ref


def linear_fp8_block(x, wq, w_scale_inv, bias=None):
    from . import cuda
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    T, K = x2.shape
    if K % 128 == 0 and x2.dtype == torch.bfloat16:
        xq, xs = cuda.quant_fp8_group(x2)
        xd = (xq.float().view(T, K // 128, 128) * xs.unsqueeze(-1)).view(T, K).to(torch.bfloat16)
    else:
        xd = x2
    w = ref.dequant_fp8_block_weight(wq, w_scale_inv).to(torch.bfloat16)
    y = cuda.gemm_bf16(xd, w, bias)
    return y.view(*lead, w.shape[0])
