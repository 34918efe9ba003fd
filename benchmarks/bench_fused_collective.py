#!/usr/bin/env python
"""Micro-benchmark of the row-parallel "GEMM -> all-reduce -> residual add -> RMSNorm" block under tensor parallelism.

Implementations of the same math, timed on the device (CUDA events around ONE launch of a CUDA graph that holds
`iters` calls - a Python call costs more host time than these kernels run, so timing eager launches would measure the
host; max over ranks; L2 flushed between iterations by cycling through distinct weight copies larger than L2):
  fused1   one kernel: tcgen05 GEMM whose epilogue pushes tiles to the row owners + communication CTAs
           (csrc/cuda/gemm_fused_rs.cu)
  fused2   tcgen05 GEMM into symmetric memory, then the reduce/add/norm/gather kernel (csrc/cuda/comm_fused.cu)
  ll       one kernel for small M: cluster split-K GEMM whose epilogue sends word-flagged slices to the row owners
           (csrc/cuda/gemm_ll_fused.cu); timed where M <= the kernel's row limit
  nccl     cuBLAS GEMM -> NCCL all-reduce -> add + RMSNorm kernel (the library baseline)
Roofline per call = max(2*M*N*K / measured bf16 GEMM peak, bytes over NVLink / link bandwidth) with bytes =
(ws-1)/ws * M*N*2 out (reduce-scatter) and the same in (all-gather) per GPU, one per direction; `roofline_hbm_us`
additionally counts the time to stream this rank's weight slice once from HBM (the real bound for small M).
Peaks come from MEASURED_PEAKS.json when present (else 1590 TFLOP/s, 6650 GB/s, 770 GB/s per direction).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_fused_collective.py
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ksanallm_b200.ops import cuda  # noqa: E402
from ksanallm_b200.parallel.comm import init_distributed  # noqa: E402


def _time(fn, dev, iters=20, warm=4):
    """Microseconds per call: `iters` calls captured in a CUDA graph that is launched once (every captured call
    carries its own collective epoch, so a graph is never replayed)."""
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(iters):
                fn(warm + i)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()
    del graph
    return float(t.item())


def _time_eager(fn, dev, iters=20, warm=4):
    """Eager launches (for paths that read sizes back to the host and cannot be captured)."""
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()
    return float(t.item())


def bench_allgather_gemm(tp, fc, peaks, Ms, H):
    """Column-parallel GEMM on a row-sharded activation: C[M, N/ws] = all_gather(A_r)[M, H] * W_r^T.
    fused = one kernel reading A tiles from the owners over NVLink; nccl = all_gather + cuBLAS."""
    rank, ws, dev = tp.rank, tp.size, tp.device
    N = int(os.environ.get("BENCH_AG_N", "28672")) // ws
    ncopies = max(2, int(256e6 // (H * N * 2)) + 1)
    wl = [(torch.randn(N, H, device=dev) * 0.02).to(torch.bfloat16) for _ in range(ncopies)]
    out = []
    for M in Ms:
        rows_per = (M + ws - 1) // ws
        if rows_per > fc.rows_cap:
            continue
        mine = (torch.randn(rows_per, H, device=dev) * 0.5).to(torch.bfloat16)
        gathered = torch.empty(ws * rows_per, H, device=dev, dtype=torch.bfloat16)

        def run_fused(i):
            fc.ag_rows(rows_per).copy_(mine)
            fc.gemm_allgather(rows_per, M, wl[i % ncopies])

        def run_nccl(i):
            dist.all_gather_into_tensor(gathered, mine)
            torch.nn.functional.linear(gathered[:M], wl[i % ncopies])

        tf, tn = _time(run_fused, dev), _time(run_nccl, dev)
        t_gemm = 2.0 * M * N * H / (peaks["bf16_tflops"] * 1e12) * 1e6
        t_link = (ws - 1) / ws * M * H * 2 / (peaks["nvlink_gbs"] * 1e9) * 1e6
        roof = max(t_gemm, t_link)
        out.append(dict(M=M, N=N, K=H, ws=ws, roofline_us=round(roof, 2), fused_us=round(tf, 2), nccl_us=round(tn, 2),
                        fused_frac=round(roof / tf, 3), nccl_frac=round(roof / tn, 3)))
    return out


def bench_ep(tp, peaks):
    """MoE block under expert parallelism, each rank owning T/ws tokens: peer-memory dispatch/combine kernels vs
    the replicated-token formulation (all_gather tokens, every rank runs its experts on all of them, reduce_scatter)."""
    from ksanallm_b200.ops import cuda_moe
    from ksanallm_b200.ops import reference as ref
    from ksanallm_b200.parallel.ep import EPExchange
    rank, ws, dev = tp.rank, tp.size, tp.device
    E, k = int(os.environ.get("BENCH_EP_E", "64")), 8
    H, I = int(os.environ.get("BENCH_EP_H", "4096")), int(os.environ.get("BENCH_EP_I", "1024"))
    el = E // ws
    w1 = (torch.randn(el, 2 * I, H, device=dev) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(el, H, I, device=dev) * 0.02).to(torch.bfloat16)
    Ts = [int(x) for x in os.environ.get("BENCH_EP_T", "16,128,1024").split(",")]
    ex = EPExchange(tp.group, rank, ws, dev, H, k, E, max(Ts))
    out = []
    for Tl in Ts:
        x = (torch.randn(Tl, H, device=dev) * 0.5).to(torch.bfloat16)
        ids, w = ref.moe_route(torch.randn(Tl, E, device=dev), k, "softmax", True)
        ids = ids.to(torch.int32)
        xg = torch.empty(ws * Tl, H, device=dev, dtype=torch.bfloat16)
        idg = torch.empty(ws * Tl, k, device=dev, dtype=torch.int32)
        wg = torch.empty(ws * Tl, k, device=dev, dtype=torch.float32)
        ys = torch.empty(Tl, H, device=dev, dtype=torch.bfloat16)

        def run_ep(i):
            ex.moe(x, ids, w, w1, w2, Tl)

        def run_repl(i):
            dist.all_gather_into_tensor(xg, x)
            dist.all_gather_into_tensor(idg, ids)
            dist.all_gather_into_tensor(wg, w)
            y = cuda_moe.moe_experts(xg, idg, wg, w1, w2, rank * el)
            dist.reduce_scatter_tensor(ys, y)

        te, tr = _time_eager(run_ep, dev), _time_eager(run_repl, dev)
        flops = 2.0 * Tl * k * 3 * H * I  # per rank on average
        link = 2.0 * Tl * min(k, ws - 1) * (ws - 1) / ws * H * 2 / 2  # out + back, one per direction (upper bound)
        roof = max(flops / (peaks["bf16_tflops"] * 1e12), link / (peaks["nvlink_gbs"] * 1e9),
                   3 * el * H * I * 2 / (peaks["hbm_gbs"] * 1e9)) * 1e6
        out.append(dict(tokens_per_rank=Tl, E=E, k=k, H=H, I=I, ws=ws, roofline_us=round(roof, 2),
                        ep_dispatch_us=round(te, 2), replicated_nccl_us=round(tr, 2)))
    return out


def main():
    tp = init_distributed("cuda")
    rank, ws, dev = tp.rank, tp.size, tp.device
    H = int(os.environ.get("BENCH_HIDDEN", "8192"))
    Kfull = int(os.environ.get("BENCH_K", "28672"))
    K = Kfull // ws
    Ms = [int(x) for x in os.environ.get("BENCH_M", "16,64,256,2048,8192").split(",")]
    tp.init_fused(H, max(Ms))
    fc = tp.fused
    peaks = {"bf16_tflops": 1590.0, "nvlink_gbs": 770.0, "hbm_gbs": 6650.0}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        mp = json.load(open(pk))
        peaks["bf16_tflops"] = float(mp.get("bf16_tflops", 1590.0))
        peaks["hbm_gbs"] = float(mp.get("hbm_gbs", 6650.0))
    ncopies = max(2, int(256e6 // (H * K * 2)) + 1)  # cycle through > L2 worth of weights
    ws_list = [(torch.randn(H, K, device=dev) * 0.02).to(torch.bfloat16) for _ in range(ncopies)]
    norm_w = torch.ones(H, device=dev, dtype=torch.bfloat16)
    rows = []
    for M in Ms:
        x = (torch.randn(M, K, device=dev) * 0.5).to(torch.bfloat16)
        residual = torch.zeros(M, H, device=dev, dtype=torch.bfloat16)

        def run_fused1(i):
            fc.gemm_reduce_add_norm(x, ws_list[i % ncopies], residual, norm_w, 1e-6)

        def run_fused2(i):
            cuda.gemm_bf16(x, ws_list[i % ncopies], None, out=fc.partial[:M])
            fc._launch(M, residual, norm_w, 1e-6)

        def run_nccl(i):
            y = torch.nn.functional.linear(x, ws_list[i % ncopies])
            dist.all_reduce(y)
            cuda.rms_norm(y, norm_w, 1e-6, residual)

        ybuf = torch.empty(M, H, device=dev, dtype=torch.bfloat16)

        def run_gemm_only(i):
            cuda.gemm_bf16(x, ws_list[i % ncopies], None, out=fc.partial[:M])

        def run_reduce_only(i):
            fc._launch(M, residual, norm_w, 1e-6)

        def run_nccl_ar_only(i):
            dist.all_reduce(ybuf)

        def run_ll(i):
            fc.gemm_ll_reduce_add_norm(x, ws_list[i % ncopies], residual, norm_w, 1e-6)

        res = {}
        parts = (("fused1", run_fused1), ("fused2", run_fused2), ("nccl", run_nccl))
        if 0 < M <= fc.ll_max_tokens:
            parts = (("ll", run_ll),) + parts
        if os.environ.get("BENCH_PARTS", "0") == "1":
            parts += (("gemm_only", run_gemm_only), ("reduce_norm_gather_only", run_reduce_only),
                      ("nccl_allreduce_only", run_nccl_ar_only))
        for name, fn in parts:
            res[name] = _time(fn, dev, iters=30, warm=5)
        flops = 2.0 * M * H * K
        t_gemm = flops / (peaks["bf16_tflops"] * 1e12) * 1e6
        link_bytes = (ws - 1) / ws * M * H * 2
        t_link = link_bytes / (peaks["nvlink_gbs"] * 1e9) * 1e6  # RS out and AG in run in opposite directions
        roof = max(t_gemm, t_link)
        t_hbm = (H * K * 2 + M * K * 2) / (peaks["hbm_gbs"] * 1e9) * 1e6
        rows.append(dict(M=M, N=H, K=K, ws=ws, roofline_us=round(roof, 2), roofline_hbm_us=round(max(roof, t_hbm), 2),
                         gemm_us=round(t_gemm, 2),
                         link_us=round(t_link, 2), **{k: round(v, 2) for k, v in res.items()},
                         fused1_frac=round(roof / res["fused1"], 3), fused2_frac=round(roof / res["fused2"], 3),
                         nccl_frac=round(roof / res["nccl"], 3),
                         ll_frac_of_hbm_roofline=round(max(roof, t_hbm) / res["ll"], 3) if "ll" in res else None))
    ag_rows = bench_allgather_gemm(tp, fc, peaks, Ms, H) if os.environ.get("BENCH_AG", "1") == "1" else []
    ep_rows = bench_ep(tp, peaks) if os.environ.get("BENCH_EP", "1") == "1" else []
    if rank == 0:
        print(json.dumps({"multicast": fc.multicast, "kernel_error": cuda.read_error(), "rows": rows,
                          "allgather_gemm": ag_rows, "ep_moe": ep_rows}, indent=1))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
