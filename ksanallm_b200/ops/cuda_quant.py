"""Quantised linear layers on the GPU: fp8 128x128 block-scaled weights and int4 group-quantised weights."""
from __future__ import annotations

from . import reference as ref


def linear_fp8_block(x, wq, w_scale_inv, bias=None):
    from . import cuda
    from . import cuda_fp8
    return cuda_fp8.linear_fp8_block(x, wq, w_scale_inv, bias)


def linear_int4(x, packed, scales, zeros, bias=None, group=128):
    from . import cuda_int4
    return cuda_int4.linear_int4(x, packed, scales, zeros, bias, group)
