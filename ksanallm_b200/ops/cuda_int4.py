"""int4 group-quantised weight-only linear (GPTQ / AWQ formats after repacking)."""
from __future__ import annotations

import torch

from . import reference as ref


def linear_int4(x, packed, scales, zeros, bias=None, group=128):
    from . import cuda
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    w = ref.dequant_int4_group(packed, scales, zeros, group).to(torch.bfloat16)
    y = cuda.gemm_bf16(x2.contiguous(), w, bias)
    return y.view(*lead, w.shape[0])
