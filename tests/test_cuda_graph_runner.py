"""Graph runner: which batch sizes are captured, padding, replay with fresh inputs. Without CUDA the runner calls the
recorded function eagerly, so the bookkeeping is checked here; the GPU test (test_zz_graph_capture.py) captures a chain
of this package's own kernels and replays it."""
import pytest
import torch

from ksanallm_b200.engine.cuda_graph_runner import CudaGraphBuilder, CudaGraphRunner


def test_builder_capture_list_and_padding():
    b = CudaGraphBuilder(max_batch_size=40, step=8)
    assert b.capture_list() == [1, 2, 4, 8, 16, 24, 32, 40]
    assert [b.padded(n) for n in (1, 3, 5, 8, 9, 33, 40, 41)] == [1, 4, 8, 8, 16, 40, 40, None]
    assert CudaGraphBuilder(max_batch_size=3, step=8).capture_list() == [1, 2, 3]
    with pytest.raises(ValueError):
        CudaGraphBuilder(0)


def test_runner_replays_with_fresh_inputs_cpu():
    r = CudaGraphRunner(device="cpu")
    w = torch.randn(16, 16)
    calls = []

    def step(x, y):
        calls.append(1)
        return x @ w + y

    xs, ys = torch.zeros(8, 16), torch.zeros(8, 16)
    r.capture(8, step, [xs, ys])
    assert r.has(8) and not r.has(4) and r.captured_keys == {8}
    with pytest.raises(KeyError):
        r.capture(8, step, [xs, ys])
    x, y = torch.randn(5, 16), torch.randn(5, 16)  # fewer rows than the graph holds
    out = r.replay(8, [x, y])
    assert torch.allclose(out[:5], x @ w + y) and r.launches == 1
    with pytest.raises(ValueError):
        r.replay(8, [torch.randn(9, 16), y])
    with pytest.raises(ValueError):
        r.replay(8, [x])
