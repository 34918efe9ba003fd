#!/usr/bin/env python
"""Serving benchmark: output tokens/s (plus p50 TTFT / TPOT) under continuous batching, tensor parallel over N GPUs.

Default workload (``--model llama-2-7b``; synthetic, seeded): Llama-2-7B bf16, 1000 chat-like requests all arriving
at t = 0, prompt lengths lognormal (median 200, sigma 1.0) clipped to [4, 2048], output lengths lognormal (median
180, sigma 1.0) clipped to [4, 1024], token ids uniform in [3, 31999], greedy decoding to the exact length (EOS
ignored), paged KV cache (block 16). If the queue drains before the timed steps are over, more requests of the same
distribution are admitted so that exactly K steps are timed. Other named workloads (``--model``):

* ``llama-3-70b``     512 requests, Poisson arrivals at 8 req/s, prompt lognormal(1024, 0.8) in [32, 8192], output
                      lognormal(256, 0.7) in [16, 2048]. Arrivals follow a virtual clock that advances by the measured
                      duration of every step and jumps over idle gaps, so TTFT / TPOT are those of the real-time run
                      without the GPUs sitting idle between arrivals.
* ``qwen3-32b-fp8``   800 requests sharing one of 8 seeded 4096-token prefixes + a unique suffix of uniform [128, 512]
                      tokens, 128 output tokens, prefix caching on, 128 x 128 block-scaled fp8 weights.
* ``deepseek-v3-fp8`` 2048 requests, prompts uniform [512, 4096], 512 output tokens, ``--max-batch`` = decode batch.

A "step" is one engine step through the public ``LLMEngine.step()``: schedule -> one H2D copy of the step's inputs
from pinned memory -> forward of every layer -> sampling -> D2H of the sampled tokens -> scheduler update.

Two identically seeded engines run the SAME W + K steps one after the other: the first is timed on the device (CUDA
events, max over ranks: ``value``), the second end to end with the host clock (``e2e``), so both numbers describe
the same steps and ``e2e`` cannot exceed ``value`` by more than timer noise.

    python bench.py --gpus 1 --steps 400 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl library ...        # same engine on library GEMMs + NCCL collectives (stand-in baseline)
    python bench.py --impl reference ...      # the unmodified reference, when it can be installed
"""
from __future__ import annotations

import argparse
import bisect
import gc
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

WORKLOADS = {
    "llama-2-7b": dict(requests=1000, max_batch=256, max_step_tokens=8192, max_token_len=3200, prefix_cache=False,
                       seq_len="prompt lognormal(200,1.0)[4,2048] + output lognormal(180,1.0)[4,1024]",
                       arrivals="all at t=0"),
    "llama-3-70b": dict(requests=512, max_batch=256, max_step_tokens=8192, max_token_len=10304, prefix_cache=False,
                        seq_len="prompt lognormal(1024,0.8)[32,8192] + output lognormal(256,0.7)[16,2048]",
                        arrivals="Poisson 8 req/s (virtual clock over measured step times)"),
    "qwen3-32b-fp8": dict(requests=800, max_batch=256, max_step_tokens=8192, max_token_len=4800, prefix_cache=True,
                          seq_len="one of 8 shared 4096-token prefixes + suffix uniform[128,512] + 128 output",
                          arrivals="all at t=0"),
    "deepseek-v3-fp8": dict(requests=2048, max_batch=256, max_step_tokens=8192, max_token_len=4672,
                            prefix_cache=False, seq_len="prompt uniform[512,4096] + 512 output",
                            arrivals="all at t=0"),
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "library"])
    ap.add_argument("--model", default="llama-2-7b", choices=sorted(WORKLOADS))
    ap.add_argument("--requests", type=int, default=0, help="0: the workload's own request count")
    ap.add_argument("--max-batch", type=int, default=0)
    ap.add_argument("--max-step-tokens", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncates the model (result marked invalid)")
    ap.add_argument("--no-async", action="store_true", help="synchronous scheduling (host waits for every step)")
    ap.add_argument("--kv-fraction", type=float, default=0.0,
                    help="fraction of device memory given to the KV cache (0: everything but a fixed reserve)")
    ap.add_argument("--no-tp1-check", action="store_true", help="skip the comparison of TP=N tokens with TP=1")
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
                                          "-i", str(self.gpu), "-lms", "100"], stdout=f, stderr=subprocess.DEVNULL)
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
            rows = [r for r in rows if len(r) >= 9]
            sm = [float(r[1]) for r in rows]
            if sm:
                # "under load": samples drawing clearly more than the idle board (falls back to all samples)
                busy = [float(r[1]) for r in rows if float(r[3]) > 250.0] or sm
                out["sm_mhz"] = statistics.median(busy)
                out["sm_max_mhz"] = float(rows[0][2])
                names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                for i, n in enumerate(names):
                    if any(r[5 + i].strip().lower() == "active" for r in rows):
                        out["reasons"].append(n)
                out["samples"] = len(sm)
                out["power_w_max"] = max(float(r[3]) for r in rows)
        except Exception:
            pass
        finally:
            try:
                os.unlink(self.path)
            except Exception:
                pass
        return out


def make_workload(model: str, n: int, seed: int, vocab: int):
    """Returns (prompts, output lengths, arrival times in seconds) of the named workload."""
    import numpy as np
    rng = np.random.default_rng(seed)

    def lognormal(median, sigma, lo, hi):
        return np.clip(np.exp(rng.normal(math.log(median), sigma, n)), lo, hi).astype(int)

    arrivals = np.zeros(n)
    if model == "llama-2-7b":
        p_len, o_len = lognormal(200.0, 1.0, 4, 2048), lognormal(180.0, 1.0, 4, 1024)
        prompts = [rng.integers(3, vocab, int(l)).tolist() for l in p_len]
    elif model == "llama-3-70b":
        p_len, o_len = lognormal(1024.0, 0.8, 32, 8192), lognormal(256.0, 0.7, 16, 2048)
        prompts = [rng.integers(3, vocab, int(l)).tolist() for l in p_len]
        arrivals = np.cumsum(rng.exponential(1.0 / 8.0, n))
    elif model == "qwen3-32b-fp8":
        prefixes = [rng.integers(3, vocab, 4096).tolist() for _ in range(8)]
        which = rng.integers(0, 8, n)
        s_len = rng.integers(128, 513, n)
        prompts = [prefixes[int(w)] + rng.integers(3, vocab, int(l)).tolist() for w, l in zip(which, s_len)]
        o_len = np.full(n, 128)
    else:  # deepseek-v3-fp8
        p_len = rng.integers(512, 4097, n)
        prompts = [rng.integers(3, vocab, int(l)).tolist() for l in p_len]
        o_len = np.full(n, 512)
    return prompts, [int(x) for x in o_len], [float(x) for x in arrivals]


class VirtualClock:
    """Host clock minus the idle gaps that were skipped: arrival times are compared against it, and wall-clock
    stamps of generated tokens are mapped onto it."""

    def __init__(self):
        self.t0 = time.time()
        self.jump_at = [self.t0]
        self.skew = [0.0]

    def now(self) -> float:
        return time.time() - self.t0 + self.skew[-1]

    def skip_to(self, t: float) -> None:
        gap = t - self.now()
        if gap > 0:
            self.jump_at.append(time.time())
            self.skew.append(self.skew[-1] + gap)

    def at(self, wall: float) -> float:
        i = bisect.bisect_right(self.jump_at, wall) - 1
        return wall - self.t0 + self.skew[max(i, 0)]


def run_phase(kind: str, args, wl, model, serving, tp, ctl, cfg):
    """One engine over the seeded workload: W warm-up steps, then K timed steps. kind "device": CUDA events around
    the K steps; kind "e2e": host clock around the same K steps (inputs copied from pinned memory and tokens read
    back every step inside LLMEngine.step())."""
    import torch
    from ksanallm_b200.engine.llm_engine import LLMEngine
    from ksanallm_b200.engine.sampling_params import SamplingParams
    from ksanallm_b200.ops import cuda

    eng = LLMEngine(model, serving, tp)
    if tp.size > 1:
        eng.attach_control_group(ctl)
    if tp.rank != 0:
        eng.follow()
        del eng
        gc.collect()
        torch.cuda.empty_cache()
        return None
    n_req = args.requests or wl["requests"]
    prompts, out_lens, arrivals = make_workload(args.model, n_req, 0, cfg.vocab_size)
    poisson = arrivals[-1] > 0
    clock = VirtualClock()
    cursor = [0]
    reqs = []

    def admit_due():
        """Admits what has arrived by the virtual clock (everything, for workloads that arrive at t = 0)."""
        while cursor[0] < n_req and arrivals[cursor[0]] <= clock.now():
            i = cursor[0]
            cursor[0] += 1
            r = eng.add_request(prompts[i], SamplingParams(topk=1, max_new_tokens=out_lens[i], ignore_eos=True))
            r.v_arrival = arrivals[i]
            reqs.append(r)

    def refill():
        # keeps the step count exact when the finite request list drains inside the timed window
        while eng.sched.num_waiting + eng.sched.num_running + eng.sched.num_swapped < serving.setting.batch_scheduler.max_batch_size \
                and cursor[0] >= n_req and not poisson:
            for i in range(min(n_req, serving.setting.batch_scheduler.max_batch_size)):
                r = eng.add_request(prompts[i], SamplingParams(topk=1, max_new_tokens=out_lens[i], ignore_eos=True))
                r.v_arrival = clock.now()
                reqs.append(r)

    def run_steps(n):
        toks = 0
        for _ in range(n):
            admit_due()
            if not eng.has_unfinished():
                if cursor[0] < n_req:
                    clock.skip_to(arrivals[cursor[0]])  # idle until the next arrival: skipped, not slept
                    admit_due()
                else:
                    refill()
            elif not poisson:
                refill()
            toks += eng.step()
        return toks

    run_steps(args.warmup)
    torch.cuda.synchronize()
    sampler = ClockSampler(tp.device.index or 0)
    sampler.start()
    l0 = cuda.launch_count
    h0, d0 = eng.runner.h2d_bytes, eng.runner.d2h_bytes
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ev0.record()
    toks = run_steps(args.steps)
    ev1.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop()
    res = dict(kind=kind, toks=toks, ms=ms, wall=wall, launches=cuda.launch_count - l0, clocks=clocks,
               h2d=(eng.runner.h2d_bytes - h0) / max(args.steps, 1), d2h=(eng.runner.d2h_bytes - d0) / max(args.steps, 1),
               err=cuda.read_error())
    ttft, tpot = [], []
    for r in reqs:
        if r.first_token_time:
            ttft.append(clock.at(r.first_token_time) - r.v_arrival)
        if r.finished and len(r.token_times) > 1:
            tpot.append((clock.at(r.token_times[-1]) - clock.at(r.token_times[0])) / (len(r.token_times) - 1))
    res["ttft"], res["tpot"] = ttft, tpot
    res["finished"] = sum(1 for r in reqs if r.finished)
    st = eng.stats
    res["host_ms"] = {k: round(1e3 * st[k] / max(st["steps"], 1), 3) for k in
                      ("schedule_time", "t_broadcast", "t_launch", "t_sample_sync", "t_apply")}
    # greedy tokens of the first requests (compared with a TP=1 run of the same weights at N > 1)
    res["head_tokens"] = [(list(r.prompt_tokens), list(r.output_token_ids[0][:4])) for r in reqs[:8]
                          if len(r.output_token_ids[0]) >= 1]
    eng.shutdown_followers()
    del eng, reqs
    gc.collect()
    torch.cuda.empty_cache()
    return res


def tp1_check(args, cfg, head, device):
    """Greedy first tokens of the first requests under TP=N against a TP=1 forward of the same (seeded) weights on
    rank 0. A token counts as matching when it is the TP=1 argmax or its TP=1 logit lies within bf16 rounding of the
    argmax's (sums of N partial products are rounded differently, near-ties may flip)."""
    import torch
    from ksanallm_b200.engine.step_input import make_step_input
    from ksanallm_b200.models.loader import load_model_weights
    from ksanallm_b200.models.transformer import TransformerModel
    from ksanallm_b200.parallel.comm import TPGroup
    w = load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, device=device, dtype=torch.bfloat16)
    m1 = TransformerModel(cfg, w, TPGroup(), max_positions=4096)
    ok, checked = True, 0
    for prompt, toks in head:
        T = len(prompt)
        nb = (T + 15) // 16
        meta = make_step_input(prompt, list(range(T)), list(range(T)), [0, T], [T], [list(range(nb))], device=device)
        kv = m1.allocate_kv_cache(nb + 1, 16)
        h = m1.forward(meta, kv)
        logits = m1.compute_logits(h[T - 1:T])[0].float()
        top = logits.max().item()
        spread = (logits.max() - logits.min()).item()
        checked += 1
        if logits[toks[0]].item() < top - 0.02 * spread:
            ok = False
        del kv
    return ok if checked else None


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return
    import torch
    import torch.distributed as dist

    from ksanallm_b200.config.model_config import NAMED_CONFIGS
    from ksanallm_b200.config.schema import parse_serving_config
    from ksanallm_b200.models.loader import load_model_weights
    from ksanallm_b200.models.transformer import TransformerModel
    from ksanallm_b200.parallel.comm import init_distributed

    use_library = args.impl == "library"
    if use_library:
        os.environ["KSANA_LIBRARY_BASELINE"] = "1"
    tp = init_distributed("cuda", use_fused=not use_library)
    rank, world = tp.rank, tp.size
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    dev = tp.device
    wl = dict(WORKLOADS[args.model])
    if args.max_batch:
        wl["max_batch"] = args.max_batch
    if args.max_step_tokens:
        wl["max_step_tokens"] = args.max_step_tokens
    cfg = NAMED_CONFIGS[args.model]()
    if args.layers:
        cfg.num_layers = args.layers
    is_moe = bool(getattr(cfg, "num_experts", 0))
    # the fp8 workloads quantise the synthetic weights at load time (128 x 128 block scales, like the checkpoints)
    weights = load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.006 if is_moe else 0.02, tp_rank=rank,
                                 tp_size=world, device=dev, dtype=torch.bfloat16,
                                 quantize="fp8_block" if args.model.endswith("-fp8") else None)
    tp.init_fused(cfg.hidden_size, wl["max_step_tokens"])
    model = TransformerModel(cfg, weights, tp, max_positions=max(4096, wl["max_token_len"]))
    mtp = 1 if args.model == "deepseek-v3-fp8" else 0
    serving = parse_serving_config({"setting": {
        "global": {"tensor_para_size": world},
        "batch_scheduler": {"max_batch_size": wl["max_batch"], "max_step_tokens": wl["max_step_tokens"],
                            "max_token_len": wl["max_token_len"], "max_waiting_queue_len": 100000, "preempt_mode": 1,
                            "enable_async": not args.no_async, "mtp_step_num": mtp,
                            "enable_auto_prefix_cache": wl["prefix_cache"]},
        "block_manager": {"block_token_num": 16, "block_device_memory_ratio": args.kv_fraction or -1.0}}})
    ctl = dist.new_group(backend="gloo") if world > 1 else None

    res_a = run_phase("device", args, wl, model, serving, tp, ctl, cfg)
    res_b = run_phase("e2e", args, wl, model, serving, tp, ctl, cfg)
    if world > 1:
        # max over ranks of the device time (followers report 0: rank 0's bracket spans every collective)
        t = torch.tensor([res_a["ms"] if res_a else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if res_a:
            res_a["ms"] = float(t.item())
        dist.barrier()
    if rank == 0:
        match = None
        if world > 1 and not args.no_tp1_check and args.model == "llama-2-7b" and not use_library:
            match = tp1_check(args, cfg, res_a["head_tokens"], dev)
        value = res_a["toks"] / (res_a["ms"] / 1e3)
        e2e = res_b["toks"] / res_b["wall"]
        size_note = {"llama-2-7b": "weights (13.5 GB) and KV cache far exceed the 126 MB L2: no explicit flush"}.get(
            args.model, "weights and KV cache far exceed the 126 MB L2: no explicit flush")
        line = {
            "metric": "output_tokens_per_s", "value": round(value, 2), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(res_a["ms"] / args.steps, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": ("fp8 (e4m3 weights, 128x128 block scales; bf16 activations and KV)"
                      if args.model.endswith("-fp8") else "bf16"),
            "data": "synthetic",
            "impl": args.impl,
            "config": {"model": args.model if not args.layers else f"{args.model}-truncated-{args.layers}L-INVALID",
                       "global_batch": wl["max_batch"], "seq_len": wl["seq_len"], "arrivals": wl["arrivals"],
                       "parallelism": f"tp{world}", "max_step_tokens": wl["max_step_tokens"],
                       "requests": args.requests or wl["requests"], "prefix_cache": wl["prefix_cache"],
                       "scheduling": "sync" if args.no_async else "async (host one step behind the device)",
                       "l2": size_note, "weights": "random N(0, 0.02), seed 0",
                       "timed_steps": "value and e2e time the same steps (W+1 .. W+K) of two identically seeded "
                                      "engines: value with CUDA events, e2e with the host clock"},
            "e2e": {"value": round(e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": int(res_b["h2d"]),
                    "d2h_bytes_per_step": int(res_b["d2h"]), "ms_per_step": round(1e3 * res_b["wall"] / args.steps, 4),
                    "tokens": res_b["toks"], "clocks": res_b["clocks"]},
            "tokens": res_a["toks"],
            "gpu_launches": int(res_a["launches"]),
            "clocks": res_a["clocks"],
            "p50_ttft_s": round(statistics.median(res_b["ttft"]), 4) if res_b["ttft"] else None,
            "p50_tpot_s": round(statistics.median(res_b["tpot"]), 5) if res_b["tpot"] else None,
            "latency_over": {"first_tokens": len(res_b["ttft"]), "finished_requests": res_b["finished"]},
            "tokens_match_tp1": match,
            "kernel_error_word": res_a["err"] | res_b["err"],
            "host_ms_per_step": res_b["host_ms"],
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
