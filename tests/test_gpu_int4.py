"""int4 weight-only tcgen05 GEMM (in-pipeline dequantisation) against the fp32 reference."""
import pytest
import torch

from ksanallm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,group,splits", [(1, 256, 512, 128, 0), (37, 384, 1024, 64, 0), (128, 1024, 4096, 128, 0),
                                                (300, 512, 2048, 128, 1), (16, 4096, 4096, 128, 4),
                                                (5, 264, 256, 128, 2), (2048, 2432, 256, 128, 0)])
def test_int4_gemm(M, N, K, group, splits):
    from ksanallm_b200.ops import cuda, cuda_int4
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.05
    packed, scales, zeros = ref.quant_int4_group(w, group)
    x = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    bias = (torch.randn(N, device="cuda", generator=g) * 0.1).to(torch.bfloat16) if M % 2 else None
    got = cuda_int4.linear_int4(x, packed, scales, zeros, bias, group, force_splits=splits)
    torch.cuda.synchronize()
    assert cuda.read_error() == 0
    wd = ref.dequant_int4_group(packed, scales, zeros, group).to(torch.bfloat16).float()
    want = x.float() @ wd.t()
    if bias is not None:
        want = want + bias.float()
    err = (got.float() - want).abs().max().item()
    assert err < 2e-2 * max(1.0, want.abs().max().item()), err


def test_int4_gemm_deterministic():
    from ksanallm_b200.ops import cuda_int4
    w = torch.randn(1024, 2048, device="cuda") * 0.05
    packed, scales, zeros = ref.quant_int4_group(w, 128)
    x = (torch.randn(8, 2048, device="cuda") * 0.5).to(torch.bfloat16)
    a = cuda_int4.linear_int4(x, packed, scales, zeros)
    b = cuda_int4.linear_int4(x, packed, scales, zeros)
    assert torch.equal(a, b)
