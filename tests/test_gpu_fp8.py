"""Block-scaled fp8 tcgen05 GEMM against the fp32 reference of the same quantised operands."""
import pytest
import torch

from ksanallm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,splits", [(128, 128, 128, 0), (200, 384, 512, 0), (64, 512, 4096, 0), (64, 512, 4096, 4),
                                           (1, 1280, 5120, 0), (300, 1000, 2048, 0), (513, 256, 7168, 0)])
def test_gemm_fp8_block(M, N, K, splits):
    from ksanallm_b200.ops import cuda
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05)
    wq, ws = ref.quant_fp8_block_weight(w)
    xq, xs = cuda.quant_fp8_group(x)
    y = cuda.gemm_fp8_block(xq, xs, wq, ws, splits=splits)
    torch.cuda.synchronize()
    assert cuda.read_error() == 0
    xd = (xq.float().view(M, K // 128, 128) * xs.unsqueeze(-1)).view(M, K)
    want = xd @ ref.dequant_fp8_block_weight(wq, ws).t()
    err = (y.float() - want).abs().max().item()
    assert err <= 2e-2 * max(1.0, want.abs().max().item()), f"max err {err}"


def test_linear_fp8_block_matches_reference_and_bias():
    from ksanallm_b200.ops import cuda
    x = torch.randn(77, 1024, device="cuda").to(torch.bfloat16)
    w = torch.randn(640, 1024, device="cuda") * 0.03
    b = torch.randn(640, device="cuda").to(torch.bfloat16)
    wq, ws = ref.quant_fp8_block_weight(w)
    y = cuda.linear_fp8_block(x, wq, ws, b)
    want = ref.linear_fp8_block(x, wq, ws, b)
    torch.cuda.synchronize()
    assert (y.float() - want.float()).abs().max().item() < 0.05 * max(1.0, want.float().abs().max().item())
