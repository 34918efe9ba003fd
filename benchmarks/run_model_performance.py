#!/usr/bin/env python
"""Offline forward-pass and communication micro-benchmarks (no scheduler, no HTTP).

Counterpart of the reference's ``run_model_performance`` and ``run_communication_performance`` binaries
(src/ksana_llm/model_performance/{model_performance_runner,communication_performance_runner,
perf_profile_config_builder_for_json}.cpp, config block ``model_performance_runner_config``).

Forward mode: synthetic batches are pushed through the model and the device time per forward is reported, per batch
and per attention-DP rank. A batch is given inline as ``[new_tokens, cached_tokens, count]`` entries, or with
``--perf-config`` in the reference's JSON form::

    {"layer_forward_round": 6,
     "batch_0": {"dp_0": [{"forwarding_token_num": 128, "sequence_len": 192, "request_num": 2}, ...], "dp_1": [...]},
     "batch_1": {...}}

(``forwarding_token_num`` new tokens of a sequence of ``sequence_len`` tokens in total; ``layer_forward_round`` runs
the chosen layer range that many times per round, to time a few layers with less noise.) Under a multi-process launch
every rank takes the ``dp_<rank>`` entry of each batch (``--same-batch-in-dps``: all take ``dp_0``); a single process
runs the DP entries one after the other.

    python benchmarks/run_model_performance.py --model llama-2-7b --batch "[[1,512,64]]" --profile-round 20
    python benchmarks/run_model_performance.py --model llama-2-7b --perf-config cfg.json --output perf.csv \
        --lower-layer-idx 0 --upper-layer-idx 3

Communication mode (``--comm``, two ranks): rank 0 sends [tokens, hidden] activations to rank 1 over the pipeline data
channel (torch.distributed send / recv: NCCL on GPUs, gloo on CPU) for tokens = 1, 2, 4, ... up to
``--max-step-tokens``, and both print the average time per round::

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/run_model_performance.py \
        --comm --model llama-2-7b
"""
import argparse
import csv
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
    """spec: [[new_tokens, cached_tokens, count], ...] -> (StepInput, blocks used)."""
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


def parse_perf_config(path):
    """The reference's JSON -> (layer_forward_round, {batch id: {dp id: [[new, cached, count], ...]}})."""
    with open(path) as f:
        doc = json.load(f)
    rounds = int(doc.get("layer_forward_round", 1))
    batches = {}
    for key, dps in doc.items():
        if not key.startswith("batch_"):
            continue
        b = int(key.split("_", 1)[1])
        batches[b] = {}
        for dkey, reqs in dps.items():
            if not dkey.startswith("dp_"):
                raise ValueError(f"{key}: unexpected key {dkey!r}")
            spec = []
            for r in reqs:
                new, total, cnt = int(r["forwarding_token_num"]), int(r["sequence_len"]), int(r.get("request_num", 1))
                if new < 1 or total < new or cnt < 1:
                    raise ValueError(f"{key}.{dkey}: need 1 <= forwarding_token_num <= sequence_len and request_num >= 1")
                spec.append([new, total - new, cnt])
            batches[b][int(dkey.split("_", 1)[1])] = spec
    if not batches:
        raise ValueError("no batch_<n> entry in the perf config")
    return rounds, batches


def time_forward(model, meta, kv, warmup, rounds, inner, cutoff, device):
    def one():
        for _ in range(inner):
            h = model.forward(meta, kv, cutoff_layer=cutoff) if cutoff is not None else model.forward(meta, kv)
        if cutoff is None:
            model.greedy_tokens(h, meta.logits_idx)

    with torch.inference_mode():
        for _ in range(warmup):
            one()
        if device.startswith("cuda"):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(rounds):
                one()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / rounds
        t0 = time.perf_counter()
        for _ in range(rounds):
            one()
        return (time.perf_counter() - t0) / rounds * 1e3


def run_comm(a, cfg):
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if world != 2:
        raise SystemExit("--comm needs exactly two ranks (torch.distributed.run --nproc-per-node 2)")
    cuda = a.device.startswith("cuda")
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl" if cuda else "gloo")
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    dt = torch.bfloat16 if cuda else torch.float32
    rows = []
    t = 1
    while t <= a.max_step_tokens:
        x = torch.zeros(t, cfg.hidden_size, dtype=dt, device=dev)
        for phase, n in (("warm", a.warmup_round), ("run", a.profile_round)):
            if phase == "run":
                dist.barrier()
                if cuda:
                    torch.cuda.synchronize()
                t0 = time.perf_counter()
            for _ in range(n):
                if rank == 0:
                    dist.send(x, dst=1)
                else:
                    dist.recv(x, src=0)
            if cuda:
                torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) / max(a.profile_round, 1) * 1e3
        gbs = t * cfg.hidden_size * x.element_size() / ms / 1e6
        rows.append(dict(role="master" if rank == 0 else "worker", tokens=t, hidden=cfg.hidden_size, dtype=str(dt),
                         ms_per_round=round(ms, 4), gb_per_s=round(gbs, 2)))
        print(json.dumps(rows[-1]), flush=True)
        t *= 2
    dist.barrier()
    dist.destroy_process_group()
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-2-7b", choices=sorted(NAMED_CONFIGS))
    ap.add_argument("--batch", default="[[1,512,64]]", help="inline batch: [[new_tokens, cached_tokens, count], ...]")
    ap.add_argument("--perf-config", default="", help="JSON file in the reference's batch_<n> / dp_<m> form")
    ap.add_argument("--warmup-round", "--warmup", dest="warmup_round", type=int, default=2)
    ap.add_argument("--profile-round", "--rounds", dest="profile_round", type=int, default=10)
    ap.add_argument("--output", default="", help="write the results as CSV")
    ap.add_argument("--lower-layer-idx", type=int, default=-1)
    ap.add_argument("--upper-layer-idx", type=int, default=-1)
    ap.add_argument("--same-batch-in-dps", action="store_true")
    ap.add_argument("--layers", type=int, default=0, help="truncate the model to this many layers")
    ap.add_argument("--comm", action="store_true", help="communication benchmark between two ranks")
    ap.add_argument("--max-step-tokens", type=int, default=4096)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args()
    cfg = NAMED_CONFIGS[a.model]()
    if a.layers:
        cfg.num_layers = a.layers
    if a.comm:
        run_comm(a, cfg)
        return
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if a.device.startswith("cuda") and world > 1:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if a.perf_config:
        inner, batches = parse_perf_config(a.perf_config)
    else:
        inner, batches = 1, {0: {0: json.loads(a.batch)}}
    # a layer range [lower, upper]: only those layers are built and run (the reference's partial model execution)
    lo, hi = a.lower_layer_idx, a.upper_layer_idx
    layer_range = None
    if lo >= 0 or hi >= 0:
        lo = max(lo, 0)
        hi = cfg.num_layers - 1 if hi < 0 else min(hi, cfg.num_layers - 1)
        if hi < lo:
            raise SystemExit("--upper-layer-idx is below --lower-layer-idx")
        layer_range = range(lo, hi + 1)
    dt = torch.bfloat16 if a.device.startswith("cuda") else torch.float32
    w = load_model_weights(cfg, synthetic_seed=0, device=a.device, dtype=dt, layer_range=layer_range)
    model = TransformerModel(cfg, w, max_positions=8192, layer_range=layer_range)
    partial = layer_range is not None and (layer_range.start > 0 or layer_range.stop < cfg.num_layers)
    rows = []
    for b in sorted(batches):
        dps = batches[b]
        if world > 1:
            mine = [0] if a.same_batch_in_dps else [rank]
        else:
            mine = [0] if a.same_batch_in_dps else sorted(dps)
        for d in mine:
            if d not in dps:
                continue  # this DP rank idles in this batch
            meta, nblocks = build_step(dps[d], 16, a.device)
            kv = model.allocate_kv_cache(nblocks + 1, 16)
            if partial:
                ms = time_layers(model, meta, kv, a.warmup_round, a.profile_round, inner, a.device)
            else:
                ms = time_forward(model, meta, kv, a.warmup_round, a.profile_round, inner, None, a.device)
            row = {"model": a.model, "layers": len(model.layer_ids), "batch_id": b, "dp": d if world == 1 else rank,
                   "batch": dps[d], "tokens": meta.total_tokens, "seqs": meta.num_seqs,
                   "layer_forward_round": inner, "forward_ms": round(ms / inner, 3),
                   "tokens_per_s": round(meta.total_tokens * inner / ms * 1e3, 1)}
            rows.append(row)
            print(json.dumps(row), flush=True)
            del kv
    if a.output:
        path = a.output if world == 1 else f"{a.output}.rank{rank}"
        with open(path, "w", newline="") as f:
            wr = csv.writer(f)
            wr.writerow(["batch_id", "dp", "tokens", "seqs", "layers", "layer_forward_round", "forward_ms", "tokens_per_s"])
            for r in rows:
                wr.writerow([r[k] for k in ("batch_id", "dp", "tokens", "seqs", "layers", "layer_forward_round",
                                            "forward_ms", "tokens_per_s")])


def time_layers(model, meta, kv, warmup, rounds, inner, device):
    """A partial model (no embedding / head of its own needed): the decoder layers over a fixed random input."""
    H = model.cfg.hidden_size
    x = torch.randn(meta.total_tokens, H, device=device).to(model.dtype) * 0.1

    def one():
        for _ in range(inner):
            model.forward(meta, kv, hidden_in=x)

    with torch.inference_mode():
        for _ in range(warmup):
            one()
        if device.startswith("cuda"):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(rounds):
                one()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / rounds
        t0 = time.perf_counter()
        for _ in range(rounds):
            one()
        return (time.perf_counter() - t0) / rounds * 1e3


if __name__ == "__main__":
    main()
