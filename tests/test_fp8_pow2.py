"""Power-of-two fp8 scales (what the scaled tensor-core GEMM needs): the reference helpers the loader and the CPU
path use."""
import torch

from ksanallm_b200.ops import reference as ref
import ksanallm_b200.ops as ops


def test_pow2_ceil_and_is_pow2():
    s = torch.tensor([1.0, 0.75, 0.5, 0.5000001, 3.0, 2.0 ** -20, 1e-30])
    p = ref.pow2_ceil(s)
    assert torch.equal(p[:5], torch.tensor([1.0, 1.0, 0.5, 1.0, 4.0]))
    assert ref.is_pow2(p) and not ref.is_pow2(s)
    assert (p >= s).all() and (p < 2 * s).all()


def test_requantisation_keeps_the_weight_within_one_rounding_step():
    torch.manual_seed(0)
    w = torch.randn(256, 384) * 0.05
    q, s = ref.quant_fp8_block_weight(w)
    q2, s2 = ref.requant_fp8_block_ue8m0(q, s)
    assert ref.is_pow2(s2) and (s2 >= s).all() and (s2 < 2 * s).all()
    a, b = ref.dequant_fp8_block_weight(q, s), ref.dequant_fp8_block_weight(q2, s2)
    # e4m3 keeps 3 mantissa bits: one more rounding moves a value by at most half a step of the coarser grid
    assert ((a - b).abs() <= a.abs() * 2 ** -4 + s2.max() * 2 ** -9).all()
    # quantising directly with power-of-two scales: no value is clipped
    q3, s3 = ref.quant_fp8_block_weight(w, ue8m0=True)
    assert ref.is_pow2(s3) and q3.float().abs().max() <= 448
    assert (ref.dequant_fp8_block_weight(q3, s3) - w).abs().max() <= w.abs().max() * 2 ** -3


def test_linear_is_the_same_function_for_any_batch_on_cpu():
    torch.manual_seed(1)
    w = torch.randn(128, 256) * 0.05
    wq, sw = ref.quant_fp8_block_weight(w, ue8m0=True)
    x = torch.randn(9, 256).to(torch.bfloat16)
    whole = ops.linear_fp8_block(x, wq, sw, None, None, True)
    rows = torch.cat([ops.linear_fp8_block(x[i:i + 1], wq, sw, None, None, True) for i in range(9)])
    assert torch.equal(whole, rows)
    xq, xs = ref.quant_fp8_group(x, ue8m0=True)
    assert ref.is_pow2(xs) and xq.float().abs().max() <= 448
