"""tcgen05 bf16 GEMM against an fp32 PyTorch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(M, N, K, bias=False, out_fp32=False, bn=0, splits=0, strided=False):
    from ksanallm_b200.ops import cuda
    torch.manual_seed(M * 131 + N * 7 + K)
    dev = "cuda"
    if strided:
        xbuf = torch.randn(M, K + 64, device=dev, dtype=torch.float32).to(torch.bfloat16)
        x = xbuf[:, 32:32 + K]
    else:
        x = torch.randn(M, K, device=dev, dtype=torch.float32).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev, dtype=torch.float32) * 0.05).to(torch.bfloat16)
    b = torch.randn(N, device=dev).to(torch.bfloat16) if bias else None
    y = cuda.gemm_bf16(x, w, b, out_dtype=torch.float32 if out_fp32 else None, bn=bn, splits=splits)
    torch.cuda.synchronize()
    assert cuda.read_error() == 0
    ref = x.float() @ w.float().t()
    if bias:
        ref = ref + b.float()
    err = (y.float() - ref).abs().max().item()
    tol = 2e-2 * max(1.0, ref.abs().max().item()) if not out_fp32 else 1e-3 * max(1.0, ref.abs().max().item())
    assert err <= tol, f"M={M} N={N} K={K} bn={bn} splits={splits}: max err {err} > {tol}"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 128, 256), (256, 512, 256), (77, 1024, 512),
                                   (300, 1536, 4096), (1, 4096, 4096), (17, 4096, 11008), (1000, 256, 128)])
def test_gemm_shapes(M, N, K):
    _check(M, N, K)


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_tile_widths(bn):
    _check(260, 768, 512, bn=bn)
    _check(260, 776, 520, bn=bn)  # ragged N and K tails


@pytest.mark.parametrize("splits", [2, 3, 4, 8, -2, -4])
def test_gemm_split_k(splits):
    """2 / 4 / 8: thread-block-cluster reduction through distributed shared memory; 3 and negative values: the
    global-workspace reduction."""
    _check(48, 512, 4096, splits=splits)
    _check(48, 512, 4096, splits=splits, bias=True)
    _check(200, 384, 2048, splits=splits, out_fp32=True)


@pytest.mark.parametrize("bn", [1128, 1256])
def test_gemm_cta_pair_kernel(bn):
    """cta_group::2 kernel (256-row tiles over two SMs): full tiles, ragged M / N / K, bias, fp32 output, strided A,
    more tiles than SM pairs (several rounds per pair, both accumulator buffers in use)."""
    _check(256, 256, 64, bn=bn)
    _check(512, 1024, 512, bn=bn)
    _check(300, 776, 520, bn=bn)
    _check(129, 264, 200, bn=bn, bias=True)
    _check(1000, 640, 768, bn=bn, out_fp32=True)
    _check(700, 512, 1024, bn=bn, strided=True)
    _check(4096, 5120, 256, bn=bn)
    # fewer tiles than SM pairs: every tile is cut into k-block ranges of several pairs (partials parked and summed)
    _check(256, 512, 4096, bn=bn)
    _check(64, 1024, 11008, bn=bn)
    _check(200, 384, 2048, bn=bn, out_fp32=True, bias=True)


def test_gemm_auto_dispatch_large_m():
    _check(2048, 4096, 1024)
    _check(8192, 1536, 512, bias=True)


def test_gemm_bias_fp32_out_and_strided_input():
    _check(200, 640, 768, bias=True)
    _check(200, 640, 768, out_fp32=True)
    _check(200, 640, 768, strided=True)


@pytest.mark.parametrize("bn", [0, 1256])
def test_gemm_deterministic(bn):
    from ksanallm_b200.ops import cuda
    x = torch.randn(64, 4096, device="cuda").to(torch.bfloat16)
    w = torch.randn(4096, 4096, device="cuda").to(torch.bfloat16)
    a = cuda.gemm_bf16(x, w, bn=bn)
    b = cuda.gemm_bf16(x, w, bn=bn)
    torch.cuda.synchronize()
    assert torch.equal(a, b)


@pytest.mark.parametrize("M,I,K", [(512, 1408, 1024), (400, 688, 512), (2048, 5504, 4096)])
def test_gemm_with_silu_mul_epilogue(M, I, K):
    """Gated FFN front half in one kernel (gate / up rows interleaved in groups of 16) against fp32 math."""
    from ksanallm_b200.ops import cuda
    torch.manual_seed(M + I)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(2 * I, K, device="cuda") * 0.05).to(torch.bfloat16)
    out = cuda.gemm_bf16_swiglu(x, cuda.interleave_gate_up(w))
    torch.cuda.synchronize()
    assert cuda.read_error() == 0
    y = x.float() @ w.float().t()
    want = torch.nn.functional.silu(y[:, :I]) * y[:, I:]
    assert out.shape == (M, I)
    assert (out.float() - want).abs().max().item() <= 2e-2 * max(1.0, want.abs().max().item())
