"""A chain of this package's kernels (RMSNorm, tcgen05 GEMM, SiLU-mul, GEMM) captured into CUDA graphs keyed by padded
batch size and replayed with fresh inputs must equal the eager result."""
import pytest
import torch

from ksanallm_b200.engine.cuda_graph_runner import CudaGraphBuilder, CudaGraphRunner


@pytest.mark.gpu
def test_runner_captures_own_kernels():
    from ksanallm_b200 import ops
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    H, I_ = 1024, 2048
    nw = (torch.rand(H, device=dev) + 0.5).bfloat16()
    w1 = (torch.randn(2 * I_, H, device=dev) * 0.03).bfloat16()
    w2 = (torch.randn(H, I_, device=dev) * 0.03).bfloat16()

    def ffn(x):
        h = ops.rms_norm(x, nw, 1e-5)
        return ops.linear(ops.silu_and_mul(ops.linear(h, w1)), w2)

    builder = CudaGraphBuilder(max_batch_size=16, step=8)
    runner = CudaGraphRunner(device=dev)
    statics = {}
    for b in builder.capture_list():
        statics[b] = torch.zeros(b, H, dtype=torch.bfloat16, device=dev)
        runner.capture(b, ffn, [statics[b]])
    for n in (1, 3, 8, 13):
        x = torch.randn(n, H, device=dev).bfloat16()
        key = builder.padded(n)
        got = runner.replay(key, [x])[:n].float().clone()
        want = ffn(x).float()
        assert torch.allclose(got, want, atol=2e-2, rtol=2e-2)
        # the same graph again with other values: nothing of the first replay may stick
        x2 = torch.randn(n, H, device=dev).bfloat16()
        got2 = runner.replay(key, [x2])[:n].float()
        assert torch.allclose(got2, ffn(x2).float(), atol=2e-2, rtol=2e-2)
    torch.cuda.synchronize()
    from ksanallm_b200.ops import cuda as kc
    assert kc.read_error() == 0
