"""Latency-optimised fused row-parallel block (GEMM -> word-flagged reduce-scatter -> residual + RMSNorm -> gather)
on ONE GPU with world size 1: every row is owned locally, the "peer" stores land in this GPU's own buffers. The
multi-rank behaviour is covered by test_gpu_multi.py."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bind():
    from ksanallm_b200.ops import cuda
    lib = cuda.lib()
    vp, ci, cu, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_float
    ll = ctypes.c_longlong
    lib.ksana_gemm_ll_reduce_norm.argtypes = [vp, vp, ci, ci, ci, ci, ci, ci, ci, vp, ll, vp, vp, vp, ci, ci, vp, vp,
                                              cf, cu, ci, ci, vp]
    lib.ksana_gemm_ll_reduce_norm.restype = ci
    lib.ksana_ll_reduce_norm.argtypes = [vp, ci, ci, ci, ci, ci, vp, ll, vp, vp, vp, ci, ci, vp, vp, cf, cu, ci, vp]
    lib.ksana_ll_reduce_norm.restype = ci
    return lib, cuda


@pytest.mark.parametrize("one_shot", [0, 1])
@pytest.mark.parametrize("M,N,K,splits", [(64, 4096, 1376, 0), (7, 1024, 512, 0), (200, 2048, 4096, 0),
                                          (128, 8192, 3584, 0), (33, 512, 1024, 4), (256, 5120, 640, 1)])
def test_gemm_ll_reduce_norm_single_rank(M, N, K, splits, one_shot):
    lib, cuda = _bind()
    dev = torch.device("cuda", 0)
    torch.manual_seed(M + N + K)
    x = (torch.randn(M, K, device=dev) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    rows_cap = 256
    half_words = rows_cap * (N // 2)
    recv = torch.zeros(2 * half_words, 2, dtype=torch.int32, device=dev)
    recv2 = torch.zeros(rows_cap * (N // 2), 2, dtype=torch.int32, device=dev)
    hbuf = torch.zeros(rows_cap, N, dtype=torch.bfloat16, device=dev)
    norm_w = (1.0 + 0.1 * torch.randn(N, device=dev)).to(torch.bfloat16)
    arr = ctypes.c_void_p * 1
    st = torch.cuda.current_stream().cuda_stream
    res0 = torch.randn(M, N, device=dev).to(torch.bfloat16)
    for epoch in (1, 2, 3):  # repeated calls reuse the word buffer: older epochs must not be taken for data
        residual = res0.clone()
        code = lib.ksana_gemm_ll_reduce_norm(x.data_ptr(), w.data_ptr(), M, N, K, K, K, 0, 1, arr(recv.data_ptr()),
                                             (epoch & 1) * half_words if one_shot else 0, arr(recv2.data_ptr()), None,
                                             hbuf.data_ptr(), rows_cap, one_shot, residual.data_ptr(),
                                             norm_w.data_ptr(), 1e-6, epoch, 3, splits, st)
        assert code == 0
        torch.cuda.synchronize()
        assert cuda.read_error() == 0
        y = (x.float() @ w.float().t()).to(torch.bfloat16).float()
        new_res = (y + res0.float()).to(torch.bfloat16)
        want = torch.nn.functional.rms_norm(new_res.float(), (N,), norm_w.float(), 1e-6)
        tol = 3e-2 * max(1.0, want.abs().max().item())
        assert (hbuf[:M].float() - want).abs().max().item() < tol
        assert (residual.float() - new_res.float()).abs().max().item() < 6e-2 * max(1.0, new_res.float().abs().max().item())
        x = (x.float() * 0.9).to(torch.bfloat16)  # different data every epoch


def test_ll_reduce_norm_from_memory_single_rank():
    lib, cuda = _bind()
    dev = torch.device("cuda", 0)
    M, H = 50, 2048
    rows_cap = 64
    part = torch.randn(M, H, device=dev).to(torch.bfloat16)
    recv = torch.zeros(rows_cap * (H // 2), 2, dtype=torch.int32, device=dev)
    recv2 = torch.zeros(rows_cap * (H // 2), 2, dtype=torch.int32, device=dev)
    hbuf = torch.zeros(rows_cap, H, dtype=torch.bfloat16, device=dev)
    arr = ctypes.c_void_p * 1
    st = torch.cuda.current_stream().cuda_stream
    # plain sum (all-reduce), no residual, no norm
    code = lib.ksana_ll_reduce_norm(part.data_ptr(), H, M, H, 0, 1, arr(recv.data_ptr()), 0, arr(recv2.data_ptr()), None,
                                    hbuf.data_ptr(), rows_cap, 0, None, None, 0.0, 5, 0, st)
    assert code == 0
    torch.cuda.synchronize()
    assert cuda.read_error() == 0
    assert torch.equal(hbuf[:M], part)
    # with residual and norm
    residual = torch.randn(M, H, device=dev).to(torch.bfloat16)
    r0 = residual.clone()
    nw = torch.ones(H, device=dev, dtype=torch.bfloat16)
    code = lib.ksana_ll_reduce_norm(part.data_ptr(), H, M, H, 0, 1, arr(recv.data_ptr()), 0, arr(recv2.data_ptr()), None,
                                    hbuf.data_ptr(), rows_cap, 1, residual.data_ptr(), nw.data_ptr(), 1e-6, 6, 3, st)
    assert code == 0
    torch.cuda.synchronize()
    assert cuda.read_error() == 0
    new_res = (part.float() + r0.float()).to(torch.bfloat16)
    assert torch.equal(residual, new_res)
    want = torch.nn.functional.rms_norm(new_res.float(), (H,), None, 1e-6)
    assert (hbuf[:M].float() - want).abs().max().item() < 3e-2
