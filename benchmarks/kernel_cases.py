#!/usr/bin/env python
"""Stand-alone cases of the hot kernels with achieved bandwidth / FLOP rates (CUDA events, L2 flushed between
iterations by rotating through operand copies larger than L2). Also the entry point used for `ncu` captures:
each case is small (at most a few GB on the device) and launches its kernel a handful of times.

    python benchmarks/kernel_cases.py gemm [M N K]            # tcgen05 bf16 GEMM
    python benchmarks/kernel_cases.py gemm_fp8 [M N K]        # block-scaled fp8 GEMM
    python benchmarks/kernel_cases.py gemm_int4 [M N K]       # int4 weight-only GEMM (in-pipeline dequant)
    python benchmarks/kernel_cases.py decode [B ctx h hk]     # paged split-KV decode attention
    python benchmarks/kernel_cases.py prefill [T h hk]        # tcgen05 paged prefill attention
    python benchmarks/kernel_cases.py mla [B ctx h q_len]     # tcgen05 absorbed-MLA decode over the latent cache
    python benchmarks/kernel_cases.py rmsnorm [T H]
    python benchmarks/kernel_cases.py moe [T E k H I]
    python benchmarks/kernel_cases.py all
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ksanallm_b200.engine.step_input import make_step_input  # noqa: E402
from ksanallm_b200.ops import cuda, cuda_moe  # noqa: E402
from ksanallm_b200.ops import reference as ref  # noqa: E402

DEV = "cuda"


def peaks():
    p = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    f = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(f):
        d = json.load(open(f))
        p["hbm_gbs"], p["bf16_tflops"] = float(d["hbm_gbs"]), float(d["bf16_tflops"])
    return p


def timeit(fn, iters=10, warm=3):
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(warm + i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3  # us


def args_or(default):
    a = [int(x) for x in sys.argv[2:]]
    return a + default[len(a):]


def case_gemm():
    M, N, K = args_or([4096, 4096, 4096])
    nw = max(2, int(300e6 // (N * K * 2)) + 1)
    ws = [(torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16) for _ in range(nw)]
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    us = timeit(lambda i: cuda.gemm_bf16(x, ws[i % nw]))
    us_lib = timeit(lambda i: torch.nn.functional.linear(x, ws[i % nw]))
    fl = 2.0 * M * N * K
    by = (M * K + N * K + M * N) * 2
    p = peaks()
    return dict(kernel="gemm_bf16", M=M, N=N, K=K, us=round(us, 1), tflops=round(fl / us / 1e6, 1),
                frac_of_measured_bf16=round(fl / us / 1e6 / p["bf16_tflops"], 3), gbs=round(by / us / 1e3, 1),
                frac_of_measured_hbm=round(by / us / 1e3 / p["hbm_gbs"], 3), cublas_us=round(us_lib, 1))


def case_gemm_fp8():
    M, N, K = args_or([4096, 4096, 4096])
    nw = max(2, int(300e6 // (N * K)) + 1)
    wq, wsc = [], []
    for _ in range(nw):
        q, s = ref.quant_fp8_block_weight(torch.randn(N, K, device=DEV) * 0.05)
        wq.append(q)
        wsc.append(s)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    xq, xs = cuda.quant_fp8_group(x)
    us = timeit(lambda i: cuda.gemm_fp8_block(xq, xs, wq[i % nw], wsc[i % nw]))
    fl = 2.0 * M * N * K
    by = M * K + N * K + M * N * 2
    p = peaks()
    return dict(kernel="gemm_fp8_block", M=M, N=N, K=K, us=round(us, 1), tflops=round(fl / us / 1e6, 1),
                gbs=round(by / us / 1e3, 1), frac_of_measured_hbm=round(by / us / 1e3 / p["hbm_gbs"], 3),
                frac_of_2x_measured_bf16=round(fl / us / 1e6 / (2 * p["bf16_tflops"]), 3))


def case_gemm_int4():
    from ksanallm_b200.ops import cuda_int4
    M, N, K = args_or([16, 8192, 8192])
    nw = max(2, int(300e6 // (N * K // 2)) + 1)
    qs = [ref.quant_int4_group(torch.randn(N, K, device=DEV) * 0.05, 128) for _ in range(nw)]
    qs = [(ref.tile_int4(p), s, z, cuda_int4.pack_scale_zero(s, z)) for p, s, z in qs]
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    us = timeit(lambda i: cuda_int4.linear_int4(x, *qs[i % nw][:3], None, 128, sz=qs[i % nw][3]))
    by = N * K / 2 + N * (K // 128) * 8 + M * K * 2 + M * N * 2
    fl = 2.0 * M * N * K
    p = peaks()
    return dict(kernel="gemm_int4", M=M, N=N, K=K, us=round(us, 1), gbs=round(by / us / 1e3, 1),
                frac_of_measured_hbm=round(by / us / 1e3 / p["hbm_gbs"], 3), tflops=round(fl / us / 1e6, 1),
                frac_of_measured_bf16=round(fl / us / 1e6 / p["bf16_tflops"], 3))


def _attn_setup(q_lens, kv_lens, h, hk):
    bs, d = 16, 128
    nblk = [(L + bs - 1) // bs for L in kv_lens]
    total = sum(nblk) + 1
    cache = (torch.randn(total, 2, hk, bs, d, device=DEV) * 0.3).to(torch.bfloat16)
    bt = torch.zeros(len(kv_lens), max(nblk), dtype=torch.int32)
    n = 0
    for b, c in enumerate(nblk):
        bt[b, :c] = torch.arange(n, n + c, dtype=torch.int32)
        n += c
    cu = [0]
    for ql in q_lens:
        cu.append(cu[-1] + ql)
    T = cu[-1]
    q = (torch.randn(T, h, d, device=DEV) * 0.3).to(torch.bfloat16)
    return q, cache, bt, cu


def case_decode():
    B, ctx, h, hk = args_or([64, 2048, 32, 32])
    q, cache, bt, cu = _attn_setup([1] * B, [ctx] * B, h, hk)
    meta = make_step_input([0] * B, [0] * B, [0] * B, cu, [ctx] * B, bt, num_prefill=0, device=DEV)
    us = timeit(lambda i: cuda.paged_attention(q, cache, meta, 128 ** -0.5))
    by = B * ctx * 2 * hk * 128 * 2
    p = peaks()
    return dict(kernel="paged_decode", B=B, ctx=ctx, h=h, hk=hk, us=round(us, 1), kv_gb=round(by / 1e9, 3),
                gbs=round(by / us / 1e3, 1), frac_of_measured_hbm=round(by / us / 1e3 / p["hbm_gbs"], 3))


def case_prefill():
    T, h, hk = args_or([4096, 32, 32])
    q, cache, bt, cu = _attn_setup([T], [T], h, hk)
    meta = make_step_input([0] * T, [0] * T, [0] * T, cu, [T], bt, num_prefill=1, device=DEV)
    us = timeit(lambda i: cuda.paged_attention(q, cache, meta, 128 ** -0.5), iters=5)
    fl = 4.0 * h * 128 * T * T / 2  # causal
    p = peaks()
    return dict(kernel="paged_prefill", T=T, h=h, hk=hk, us=round(us, 1), tflops=round(fl / us / 1e6, 1),
                frac_of_measured_bf16=round(fl / us / 1e6 / p["bf16_tflops"], 3))


def case_mla():
    from ksanallm_b200.ops import cuda_mla
    B, ctx, h, ql = args_or([64, 4096, 128, 1])
    bs = 64
    nb = (ctx + bs - 1) // bs
    cache = (torch.randn(B * nb + 1, bs, 576, device=DEV) * 0.3).to(torch.bfloat16)
    bt = torch.arange(B * nb, dtype=torch.int32).reshape(B, nb)
    cu = [i * ql for i in range(B + 1)]
    T = B * ql
    q_lat = (torch.randn(T, h, 512, device=DEV) * 0.3).to(torch.bfloat16)
    q_rope = (torch.randn(T, h, 64, device=DEV) * 0.3).to(torch.bfloat16)
    meta = make_step_input([0] * T, [0] * T, [0] * T, cu, [ctx] * B, bt, num_prefill=0, device=DEV)
    us = timeit(lambda i: cuda_mla.mla_paged_attention(q_lat, q_rope, cache, meta, 0.1147))
    by = B * ctx * 576 * 2
    fl = 2.0 * T * h * ctx * (576 + 512)
    p = peaks()
    return dict(kernel="mla_decode", B=B, ctx=ctx, h=h, q_len=ql, us=round(us, 1), kv_gb=round(by / 1e9, 3),
                gbs=round(by / us / 1e3, 1), frac_of_measured_hbm=round(by / us / 1e3 / p["hbm_gbs"], 3),
                tflops=round(fl / us / 1e6, 1), frac_of_measured_bf16=round(fl / us / 1e6 / p["bf16_tflops"], 3))


def case_rmsnorm():
    T, H = args_or([16384, 8192])
    xs = [torch.randn(T, H, device=DEV).to(torch.bfloat16) for _ in range(2)]
    rs = [torch.randn(T, H, device=DEV).to(torch.bfloat16) for _ in range(2)]
    w = torch.ones(H, device=DEV, dtype=torch.bfloat16)
    us = timeit(lambda i: cuda.rms_norm(xs[i % 2], w, 1e-6, rs[i % 2]))
    by = T * H * 2 * 4  # x, residual in, residual out, y
    p = peaks()
    return dict(kernel="rms_norm+residual", T=T, H=H, us=round(us, 1), gbs=round(by / us / 1e3, 1),
                frac_of_measured_hbm=round(by / us / 1e3 / p["hbm_gbs"], 3))


def case_moe():
    T, E, k, H, I = args_or([2048, 32, 8, 2048, 1024])
    x = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    ids, w = ref.moe_route(torch.randn(T, E, device=DEV), k, "softmax", True)
    w1 = (torch.randn(E, 2 * I, H, device=DEV) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, device=DEV) * 0.05).to(torch.bfloat16)
    us = timeit(lambda i: cuda_moe.moe_experts(x, ids, w, w1, w2, 0), iters=5)
    fl = 2.0 * T * k * (2 * I * H + H * I)
    p = peaks()
    return dict(kernel="moe_experts(pipeline)", T=T, E=E, k=k, H=H, I=I, us=round(us, 1),
                tflops=round(fl / us / 1e6, 1), frac_of_measured_bf16=round(fl / us / 1e6 / p["bf16_tflops"], 3))


CASES = dict(gemm=case_gemm, gemm_fp8=case_gemm_fp8, gemm_int4=case_gemm_int4, decode=case_decode, prefill=case_prefill, mla=case_mla, rmsnorm=case_rmsnorm,
             moe=case_moe)

if __name__ == "__main__":
    which = sys.argv[1] if len(sys.argv) > 1 else "all"
    names = list(CASES) if which == "all" else [which]
    if which == "all":
        sys.argv = sys.argv[:2]
    for n in names:
        print(json.dumps(CASES[n]()))
    print(json.dumps({"kernel_status_word": cuda.read_error()}))
