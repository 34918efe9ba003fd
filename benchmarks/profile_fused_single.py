#!/usr/bin/env python
"""Runs the fused GEMM -> reduce-scatter -> norm -> all-gather kernel with world_size 1 on one GPU (every row is
owned locally, so the "peer" stores land in this GPU's own receive buffer). Meant for profiling the kernel under
ncu on a single device; prints the device time per call.

    python benchmarks/profile_fused_single.py [M N K iters]
"""
import ctypes
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ksanallm_b200.ops import cuda  # noqa: E402


def main():
    M, N, K, iters = (int(a) for a in (sys.argv[1:5] + ["2048", "4096", "4096", "5"][len(sys.argv) - 1:]))
    dev = torch.device("cuda", 0)
    lib = cuda.lib()
    fn = lib.ksana_gemm_rs_norm_ag
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, vp, ci, ci, ci, ci, ci, ci, ci, vp, vp, vp, vp, ci, vp, vp, ctypes.c_float, ctypes.c_uint, ci, ci,
                   ci, vp]
    fn.restype = ci
    x = (torch.randn(M, K, device=dev) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    recv = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    hbuf = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    sig = torch.zeros(8192, dtype=torch.int32, device=dev)
    residual = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    norm_w = torch.ones(N, dtype=torch.bfloat16, device=dev)
    arr = vp * 1
    p_recv, p_hbuf, p_sig = arr(recv.data_ptr()), arr(hbuf.data_ptr()), arr(sig.data_ptr())
    st = torch.cuda.current_stream().cuda_stream

    def call(epoch):
        code = fn(x.data_ptr(), w.data_ptr(), M, N, K, K, K, 0, 1, p_recv, p_hbuf, p_sig, None, M, residual.data_ptr(),
                  norm_w.data_ptr(), 1e-6, epoch, 3, 16, 0, st)
        assert code == 0, code

    call(1)
    torch.cuda.synchronize()
    want = torch.nn.functional.rms_norm((x.float() @ w.float().t()).to(torch.bfloat16).float(), (N,), None, 1e-6)
    err = (hbuf.float() - want).abs().max().item()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        call(2 + i)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / iters * 1e3
    flops = 2.0 * M * N * K
    print(f"M={M} N={N} K={K}: {us:.1f} us/call, {flops / us / 1e6:.1f} TFLOP/s, max err vs reference {err:.4f}, "
          f"kernel status {cuda.read_error()}")
    y = cuda.gemm_bf16(x, w)
    torch.cuda.synchronize()
    e0.record()
    for i in range(iters):
        cuda.gemm_bf16(x, w)
    e1.record()
    torch.cuda.synchronize()
    us2 = e0.elapsed_time(e1) / iters * 1e3
    print(f"plain tcgen05 GEMM of the same shape: {us2:.1f} us/call, {flops / us2 / 1e6:.1f} TFLOP/s")


if __name__ == "__main__":
    main()
