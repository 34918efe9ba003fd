#!/usr/bin/env python
"""Offline sweep of the tcgen05 GEMM's launch parameters (tile width, split-K factor) for the linear layers of a model
at the batch sizes a server sees; writes the YAML that ``KSANA_GEMM_TUNE_FILE`` / ``ops.gemm_tune.load_map`` read.
Counterpart of the reference's cuBLASLt algorithm search (tools ``search_best_gemm_algo`` -> ``gemm_algo_map.yaml``).

    python benchmarks/search_best_gemm.py --model llama-2-7b --tp 1 --out gemm_map.yaml
"""
import argparse
import os
import sys

import torch
import yaml

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ksanallm_b200.config.model_config import NAMED_CONFIGS  # noqa: E402
from ksanallm_b200.ops import cuda  # noqa: E402


def layer_shapes(cfg, tp):
    h, hk, d, H, I = cfg.num_heads // tp, max(cfg.num_kv_heads // tp, 1), cfg.head_dim, cfg.hidden_size, cfg.intermediate_size // tp
    return {"qkv": ((h + 2 * hk) * d, H), "o_proj": (H, h * d), "gate_up": (2 * I, H), "down": (H, I),
            "lm_head": (-(-cfg.vocab_size // tp) // 8 * 8, H)}


def time_us(fn, iters=20):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-2-7b", choices=sorted(NAMED_CONFIGS))
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--ms", default="1,16,64,128,256,512,1024,2048,4096,8192")
    ap.add_argument("--out", default="gemm_map.yaml")
    args = ap.parse_args()
    cfg = NAMED_CONFIGS[args.model]()
    entries = []
    for name, (N, K) in layer_shapes(cfg, args.tp).items():
        copies = max(2, int(300e6 // (N * K * 2)) + 1)  # rotate through more than L2 worth of weights
        ws = [(torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
        for M in [int(x) for x in args.ms.split(",")]:
            x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
            best = None
            cands = [(0, 0)] + [(bn, sp) for bn in (64, 128, 256) for sp in (1, 2, 4, 8, -2, -4, -8)
                                if not (M > 512 and sp not in (1,))]
            for bn, sp in cands:
                it = [0]

                def run():
                    it[0] += 1
                    cuda.gemm_bf16(x, ws[it[0] % copies], None, bn=bn, splits=sp)
                try:
                    t = time_us(run)
                except RuntimeError:
                    continue
                if best is None or t < best[0]:
                    best = (t, bn, sp)
            print(f"{name:8s} M={M:5d} N={N:6d} K={K:6d}: best bn={best[1]} splits={best[2]} {best[0]:.1f} us")
            if (best[1], best[2]) != (0, 0):
                entries.append(dict(n=N, k=K, m_max=M, bn=best[1], splits=best[2]))
    with open(args.out, "w") as f:
        yaml.safe_dump({"gemm_bf16": entries}, f, sort_keys=False)
    print("wrote", args.out, len(entries), "entries; kernel status word", cuda.read_error())


if __name__ == "__main__":
    main()
