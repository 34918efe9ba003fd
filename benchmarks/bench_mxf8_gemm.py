"""Times (CUDA events around a CUDA graph of 8 launches, min of 5 replays, rotating weights larger than L2) the fp8
GEMM with tensor-core-applied scales against the fp32-scale fp8 kernel and the bf16 GEMM.

    python benchmarks/bench_mxf8_gemm.py [MxNxK ...] [--once [--pair]]

``--once`` runs three launches of the scaled GEMM only (the case an ncu capture wraps): the one-CTA-per-tile kernel, or
with ``--pair`` the CTA-pair kernel."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ksanallm_b200.ops import cuda, cuda_fp8, reference as ref  # noqa: E402


def graph_time(fn, n=8, reps=5):
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    best = 1e9
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / n * 1e3)
    return best


def main():
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    once = "--once" in sys.argv
    shapes = [tuple(int(v) for v in a.split("x")) for a in args] or [
        (8192, 7168, 7168), (8192, 5120, 5120), (8192, 12800, 5120), (8192, 5120, 6400), (2048, 5120, 6400),
        (512, 12800, 5120), (256, 5120, 6400), (128, 12800, 5120), (64, 12800, 5120), (64, 5120, 6400),
        (16, 5120, 6400)]
    dev = "cuda"
    for M, N, K in shapes:
        nw = 2 if once else min(8, max(2, int(300e6 // (N * K)) + 1))
        packs = []
        for _ in range(nw):
            wq, sw = ref.quant_fp8_block_weight(torch.randn(N, K, device=dev) * 0.05, ue8m0=True)
            packs.append((wq, sw, cuda_fp8.pack_sfb(sw, N, K)))
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        xq, xs, sfa = cuda_fp8.quant_fp8_ue8m0(x, scales=True, packed=True)
        outs = [torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(2)]
        if once:
            for i in range(3):
                cuda_fp8.gemm_mxf8(xq, sfa, packs[i % nw][0], packs[i % nw][2], out=outs[i % 2],
                                   variant=2 if "--pair" in sys.argv else 1)
            torch.cuda.synchronize()
            print(json.dumps(dict(M=M, N=N, K=K, status=cuda.read_error())))
            continue
        wb = [(torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16) for _ in range(2)]
        row = dict(M=M, N=N, K=K)
        row["mxf8_us"] = round(graph_time(
            lambda i: cuda_fp8.gemm_mxf8(xq, sfa, packs[i % nw][0], packs[i % nw][2], out=outs[i % 2], variant=1)), 1)
        row["mxf8_pair_us"] = round(graph_time(
            lambda i: cuda_fp8.gemm_mxf8(xq, sfa, packs[i % nw][0], packs[i % nw][2], out=outs[i % 2], variant=2)), 1)
        row["fp8_block_us"] = round(graph_time(
            lambda i: cuda.gemm_fp8_block(xq, xs, packs[i % nw][0], packs[i % nw][1], out=outs[i % 2])), 1)
        row["bf16_us"] = round(graph_time(lambda i: cuda.gemm_bf16(x, wb[i % 2], out=outs[i % 2])), 1)
        row["quant_us"] = round(graph_time(lambda i: cuda_fp8.quant_fp8_ue8m0(x, scales=False, packed=True)), 1)
        fl = 2.0 * M * N * K
        for k in ("mxf8", "mxf8_pair", "fp8_block", "bf16"):
            row[k + "_tflops"] = round(fl / row[k + "_us"] / 1e6)
        row["fp8_hbm_floor_us"] = round((N * K + M * K + M * N * 2) / 6.55e6, 1)
        print(json.dumps(row), flush=True)
        del packs, x, wb
    print("status", cuda.read_error())


if __name__ == "__main__":
    main()
