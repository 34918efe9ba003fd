#!/usr/bin/env python
"""Offline forward-pass micro-benchmark: synthetic batches described as lists of
``[new_tokens, cached_tokens, count]`` entries are pushed through the model (no scheduler, no HTTP) and the pure
forward time per step is reported. Counterpart of the reference's ``run_model_performance`` binary
(src/ksana_llm/model_performance/*, config block ``model_performance_runner_config`` in examples/ksana_llm2-7b.yaml).

    python benchmarks/run_model_performance.py --model llama-2-7b --batch "[[1,512,64]]" --rounds 20
    python benchmarks/run_model_performance.py --model llama-2-7b --batch "[[1024,0,4],[1,300,32]]"
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ksanallm_b200.config.model_config import NAMED_CONFIGS  # noqa: E402
from ksanallm_b200.engine.step_input import make_step_input  # noqa: E402
from ksanallm_b200.models.loader import load_model_weights  # noqa: E402
from ksanallm_b200.models.transformer import TransformerModel  # noqa: E402


def build_step(spec, block_size, device):
    ids, pos, slots, cu, kvl, bts = [], [], [], [0], [], []
    nxt = 0
    entries = sorted(([n, c] for n, c, k in spec for _ in range(k)), key=lambda e: (-(e[0] > 1), -e[0]))
    for n_new, cached in entries:
        total = n_new + cached
        nb = (total + block_size - 1) // block_size
        table = list(range(nxt, nxt + nb))
        nxt += nb
        for p in range(cached, total):
            ids.append(3 + (p * 7919) % 30000)
            pos.append(p)
            slots.append(table[p // block_size] * block_size + p % block_size)
        cu.append(cu[-1] + n_new)
        kvl.append(total)
        bts.append(table)
    mb = max(len(t) for t in bts)
    bts = [t + [0] * (mb - len(t)) for t in bts]
    n_pre = sum(1 for n, c in entries if n > 1 or c == 0)
    return make_step_input(ids, pos, slots, cu, kvl, bts, num_prefill=n_pre, device=device), nxt


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-2-7b", choices=sorted(NAMED_CONFIGS))
    ap.add_argument("--batch", default="[[1,512,64]]")
    ap.add_argument("--rounds", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args()
    cfg = NAMED_CONFIGS[a.model]()
    if a.layers:
        cfg.num_layers = a.layers
    dt = torch.bfloat16 if a.device.startswith("cuda") else torch.float32
    w = load_model_weights(cfg, synthetic_seed=0, device=a.device, dtype=dt)
    model = TransformerModel(cfg, w, max_positions=8192)
    meta, nblocks = build_step(json.loads(a.batch), 16, a.device)
    kv = model.allocate_kv_cache(nblocks + 1, 16)
    with torch.inference_mode():
        for _ in range(a.warmup):
            h = model.forward(meta, kv)
            model.greedy_tokens(h, meta.logits_idx)
        if a.device.startswith("cuda"):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        for _ in range(a.rounds):
            h = model.forward(meta, kv)
            model.greedy_tokens(h, meta.logits_idx)
        if a.device.startswith("cuda"):
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / a.rounds
        else:
            ms = (time.perf_counter() - t0) / a.rounds * 1e3
    print(json.dumps({"model": a.model, "layers": cfg.num_layers, "batch": json.loads(a.batch),
                      "tokens": meta.total_tokens, "seqs": meta.num_seqs, "forward_ms": round(ms, 3),
                      "tokens_per_s": round(meta.total_tokens / ms * 1e3, 1)}))


if __name__ == "__main__":
    main()
