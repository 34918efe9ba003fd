#!/usr/bin/env python
"""Serving benchmark: output tokens/s (plus p50 TTFT / TPOT) of Llama-2-7B, bf16, tensor parallel over N GPUs.

Workload (synthetic, seeded): 1000 chat-like requests all arriving at t = 0, prompt lengths lognormal
(median 200, sigma 1.0) clipped to [4, 2048], output lengths lognormal (median 180, sigma 1.0) clipped to
[4, 1024], token ids uniform in [3, 31999], greedy decoding to the exact length (EOS ignored), continuous
batching over a paged KV cache (block 16). If the queue drains before the timed steps are over, more requests
of the same distribution are admitted so that exactly K steps are timed.

A "step" is one engine step: schedule -> one H2D copy of the step's inputs from pinned memory -> forward of
every layer -> sampling -> D2H of the sampled tokens -> scheduler update.

    python bench.py --gpus 1 --steps 400 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference, when it can be installed
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "library"])
    ap.add_argument("--model", default="llama-2-7b")
    ap.add_argument("--requests", type=int, default=1000)
    ap.add_argument("--max-batch", type=int, default=256)
    ap.add_argument("--max-step-tokens", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncates the model (result marked invalid)")
    ap.add_argument("--no-cuda-graph", action="store_true")
    ap.add_argument("--no-async", action="store_true", help="synchronous scheduling (host waits for every step)")
    return ap.parse_args()


def reference_arm(args) -> None:
    """Runs the unmodified reference from baseline/_ref through its own API - when it is installed."""
    ref_dir = os.path.join(REPO, "baseline", "_ref")
    reason = None
    if not os.path.isdir(ref_dir) or not os.listdir(ref_dir):
        reason = ("reference not installed: its pip install fails offline (CMake fetches ~25 "
                  "dependencies + DeepGEMM/flashinfer from the network, submodules are empty, no sm_100 target)")
    else:
        sys.path.insert(0, ref_dir)
        try:
            import ksana_llm  # noqa: F401
        except Exception as ex:  # pragma: no cover
            reason = f"reference import failed: {type(ex).__name__}: {ex}"[:300]
    if reason is None:
        reason = "reference imported but its libtorch_serving engine has no sm_100 build"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": reason}))


class ClockSampler:
    """nvidia-smi clocks / throttle reasons during the timed region (read only)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "200"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            rows = [r.strip().split(",") for r in open(self.path) if r.strip()]
            sm = [float(r[1]) for r in rows if len(r) >= 9]
            if sm:
                out["sm_mhz"] = statistics.median(sm)
                out["sm_max_mhz"] = float(rows[0][2])
                names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                for i, n in enumerate(names):
                    if any(r[5 + i].strip().lower() == "active" for r in rows if len(r) >= 9):
                        out["reasons"].append(n)
                out["samples"] = len(sm)
                out["power_w_max"] = max(float(r[3]) for r in rows if len(r) >= 9)
        except Exception:
            pass
        finally:
            try:
                os.unlink(self.path)
            except Exception:
                pass
        return out


def make_workload(n, seed, vocab):
    import numpy as np
    rng = np.random.default_rng(seed)
    p_len = np.clip(np.exp(rng.normal(math.log(200.0), 1.0, n)), 4, 2048).astype(int)
    o_len = np.clip(np.exp(rng.normal(math.log(180.0), 1.0, n)), 4, 1024).astype(int)
    prompts = [rng.integers(3, vocab, int(l)).tolist() for l in p_len]
    return prompts, o_len.tolist()


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    import numpy as np
    import torch
    import torch.distributed as dist

    from ksanallm_b200.config.model_config import NAMED_CONFIGS
    from ksanallm_b200.config.schema import parse_serving_config
    from ksanallm_b200.engine.llm_engine import LLMEngine
    from ksanallm_b200.engine.sampling_params import SamplingParams
    from ksanallm_b200.models.loader import load_model_weights
    from ksanallm_b200.models.transformer import TransformerModel
    from ksanallm_b200.ops import cuda
    from ksanallm_b200.parallel.comm import init_distributed

    use_library = args.impl == "library"
    if use_library:
        os.environ["KSANA_LIBRARY_BASELINE"] = "1"
    tp = init_distributed("cuda", use_fused=not use_library)
    rank, world = tp.rank, tp.size
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    dev = tp.device
    cfg = NAMED_CONFIGS[args.model]()
    if args.layers:
        cfg.num_layers = args.layers
    weights = load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, tp_rank=rank, tp_size=world, device=dev,
                                 dtype=torch.bfloat16)
    tp.init_fused(cfg.hidden_size, args.max_step_tokens)
    model = TransformerModel(cfg, weights, tp, max_positions=4096)
    serving = parse_serving_config({"setting": {
        "global": {"tensor_para_size": world, "enable_cuda_graph": not args.no_cuda_graph},
        "batch_scheduler": {"max_batch_size": args.max_batch, "max_step_tokens": args.max_step_tokens,
                            "max_token_len": 3200, "max_waiting_queue_len": 100000, "preempt_mode": 1,
                            "enable_async": not args.no_async,
                            "enable_auto_prefix_cache": False},
        "block_manager": {"block_token_num": 16}}})
    eng = LLMEngine(model, serving, tp)
    ctl = dist.new_group(backend="gloo") if world > 1 else None
    if world > 1:
        eng.attach_control_group(ctl)

    result = None
    if rank == 0:
        prompts, out_lens = make_workload(args.requests, 0, cfg.vocab_size)
        cursor = [0]

        def admit(k):
            for _ in range(k):
                i = cursor[0] % len(prompts)
                cursor[0] += 1
                eng.add_request(prompts[i], SamplingParams(topk=1, max_new_tokens=int(out_lens[i]), ignore_eos=True))

        admit(args.requests)
        all_reqs = list(eng.requests.values())

        def run_steps(n):
            toks = 0
            for _ in range(n):
                if eng.sched.num_waiting + eng.sched.num_running + eng.sched.num_swapped < args.max_batch:
                    admit(args.max_batch)
                    all_reqs.extend(r for r in eng.requests.values() if r not in seen)
                toks += eng.step()
            return toks

        seen = set(all_reqs)
        run_steps(args.warmup)
        torch.cuda.synchronize()
        # ---- phase A: device-timed ----
        sampler = ClockSampler(dev.index or 0)
        sampler.start()
        l0 = cuda.launch_count + getattr(eng.runner, "graph_launches", 0)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record()
        toks_a = run_steps(args.steps)
        ev1.record()
        torch.cuda.synchronize()
        ms_a = ev0.elapsed_time(ev1)
        launches = cuda.launch_count + getattr(eng.runner, "graph_launches", 0) - l0
        # ---- phase B: end to end through the public step API, wall clock, byte accounting ----
        h0, d0 = eng.runner.h2d_bytes, eng.runner.d2h_bytes
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        toks_b = run_steps(args.steps)
        torch.cuda.synchronize()
        wall_b = time.perf_counter() - t0
        clocks = sampler.stop()
        h2d = (eng.runner.h2d_bytes - h0) / max(args.steps, 1)
        d2h = (eng.runner.d2h_bytes - d0) / max(args.steps, 1)
        ttft = [r.first_token_time - r.arrival for r in all_reqs if r.first_token_time]
        tpot = []
        for r in all_reqs:
            if r.finished and len(r.token_times) > 1:
                tpot.append((r.token_times[-1] - r.token_times[0]) / (len(r.token_times) - 1))
        st = eng.stats
        host_ms = {k: round(1e3 * st[k] / max(st["steps"], 1), 3) for k in
                   ("schedule_time", "t_broadcast", "t_launch", "t_sample_sync", "t_apply")}
        result = dict(host_ms=host_ms, toks_a=toks_a, ms_a=ms_a, toks_b=toks_b, wall_b=wall_b, launches=launches, clocks=clocks,
                      h2d=h2d, d2h=d2h, ttft=ttft, tpot=tpot, err=cuda.read_error())
        eng.shutdown_followers()
    else:
        eng.follow()
    if world > 1:
        # max over ranks of the device time (followers report 0: rank 0's bracket spans every collective)
        t = torch.tensor([result["ms_a"] if result else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if result:
            result["ms_a"] = float(t.item())
        dist.barrier()
    if rank == 0:
        value = result["toks_a"] / (result["ms_a"] / 1e3)
        e2e = result["toks_b"] / result["wall_b"]
        line = {
            "metric": "output_tokens_per_s", "value": round(value, 2), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(result["ms_a"] / args.steps, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": args.impl,
            "config": {"model": args.model if not args.layers else f"{args.model}-truncated-{args.layers}L-INVALID",
                       "global_batch": args.max_batch, "seq_len": "prompt lognormal(200,1.0)[4,2048] + "
                       "output lognormal(180,1.0)[4,1024]", "parallelism": f"tp{world}",
                       "max_step_tokens": args.max_step_tokens, "requests": args.requests,
                       "scheduling": "sync" if args.no_async else "async (host one step behind the device)",
                       "l2": "weights (13.5 GB) and KV cache far exceed the 126 MB L2: no explicit flush",
                       "weights": "random N(0, 0.02), seed 0"},
            "e2e": {"value": round(e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": int(result["h2d"]),
                    "d2h_bytes_per_step": int(result["d2h"])},
            "gpu_launches": int(result["launches"]),
            "clocks": result["clocks"],
            "p50_ttft_s": round(statistics.median(result["ttft"]), 4) if result["ttft"] else None,
            "p50_tpot_s": round(statistics.median(result["tpot"]), 5) if result["tpot"] else None,
            "kernel_error_word": result["err"],
            "host_ms_per_step": result["host_ms"],
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
