#!/usr/bin/env python
"""Client-side serving benchmark against a running server (``/generate`` streaming endpoint or the OpenAI chat
endpoint): request throughput, token throughput (total or decode only), mean / median / percentile TTFT, ITL and
TPOT, optional request-rate sweep with Poisson arrivals. Same measurements as the reference client
(benchmarks/benchmark_throughput.py:118-177, 722-762) with synthetic random-length prompts built in, so it needs
no dataset files.

    python benchmarks/benchmark_throughput.py --port 8080 --prompt_num 200 --request_rate 8 \
        --input_len_median 1024 --output_len_median 256
"""
import argparse
import asyncio
import json
import math
import random
import statistics
import time

import aiohttp


def pct(v, p):
    if not v:
        return float("nan")
    v = sorted(v)
    return v[min(len(v) - 1, int(math.ceil(p / 100.0 * len(v))) - 1)]


def make_requests(args):
    rng = random.Random(args.seed)
    out = []
    for _ in range(args.prompt_num):
        n_in = int(min(max(math.exp(rng.gauss(math.log(args.input_len_median), args.len_sigma)), args.input_len_min),
                       args.input_len_max))
        n_out = int(min(max(math.exp(rng.gauss(math.log(args.output_len_median), args.len_sigma)), args.output_len_min),
                        args.output_len_max))
        out.append(([rng.randint(3, args.vocab_size - 1) for _ in range(n_in)], n_out))
    return out


async def one_request(session, url, tokens, n_out, results, args, index=0):
    body = {"input_tokens": tokens, "stream": True,
            "sampling_config": {"max_new_tokens": n_out, "topk": 1, "ignore_eos": True}}
    t0 = time.perf_counter()
    stamps, n_prev, last = [], 0, None
    try:
        async with session.post(url, data=json.dumps(body)) as resp:
            buf = b""
            async for chunk in resp.content.iter_any():
                buf += chunk
                while b"\0" in buf:
                    piece, buf = buf.split(b"\0", 1)
                    if not piece:
                        continue
                    last = json.loads(piece)
                    n = len(last["output_token_ids"][0])
                    now = time.perf_counter()
                    stamps.extend([now] * (n - n_prev))
                    n_prev = n
        ok = n_prev > 0
    except Exception:
        ok = False
    results.append(dict(ok=ok, t0=t0, stamps=stamps, n_in=len(tokens), n_out=n_prev, index=index, last=last))


async def run(args):
    reqs = make_requests(args)
    url = f"http://{args.host}:{args.port}/generate"
    results = []
    conn = aiohttp.TCPConnector(limit=args.max_concurrency)
    async with aiohttp.ClientSession(connector=conn, timeout=aiohttp.ClientTimeout(total=None)) as session:
        t_start = time.perf_counter()
        tasks = []
        rng = random.Random(args.seed + 1)
        for i, (toks, n_out) in enumerate(reqs):
            tasks.append(asyncio.create_task(one_request(session, url, toks, n_out, results, args, i)))
            if args.request_rate > 0:
                await asyncio.sleep(rng.expovariate(args.request_rate))
        await asyncio.gather(*tasks)
        elapsed = time.perf_counter() - t_start
    good = [r for r in results if r["ok"]]
    ttft = [r["stamps"][0] - r["t0"] for r in good]
    itl, tpot = [], []
    for r in good:
        s = r["stamps"]
        itl += [b - a for a, b in zip(s[:-1], s[1:]) if b > a]
        if len(s) > 1:
            tpot.append((s[-1] - s[0]) / (len(s) - 1))
    out_tok = sum(r["n_out"] for r in good)
    in_tok = sum(r["n_in"] for r in good)
    rep = {
        "completed": len(good), "failed": len(results) - len(good), "elapsed_s": round(elapsed, 3),
        "request_throughput": round(len(good) / elapsed, 3),
        "output_token_throughput": round(out_tok / elapsed, 2),
        "total_token_throughput": round((in_tok + out_tok) / elapsed, 2),
        "ttft_s": {"mean": statistics.fmean(ttft) if ttft else None, "p50": pct(ttft, 50), "p90": pct(ttft, 90),
                   "p99": pct(ttft, 99)},
        "itl_s": {"mean": statistics.fmean(itl) if itl else None, "p50": pct(itl, 50), "p99": pct(itl, 99)},
        "tpot_s": {"mean": statistics.fmean(tpot) if tpot else None, "p50": pct(tpot, 50), "p99": pct(tpot, 99)},
    }
    print(json.dumps(rep, indent=1))
    if args.output:
        # one line per request, in request order: what benchmarks/check_diff.py compares between two runs
        with open(args.output, "w", encoding="utf-8") as f:
            for r in sorted(results, key=lambda r: r["index"]):
                last = r["last"] or {}
                f.write(json.dumps({"index": r["index"], "output_token_ids": (last.get("output_token_ids") or [[]])[0],
                                    "text": (last.get("texts") or [""])[0]}) + "\n")
    return rep


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--prompt_num", type=int, default=100)
    ap.add_argument("--request_rate", type=float, default=0.0, help="Poisson arrivals per second; 0 = all at once")
    ap.add_argument("--max_concurrency", type=int, default=1024)
    ap.add_argument("--input_len_median", type=float, default=200)
    ap.add_argument("--output_len_median", type=float, default=180)
    ap.add_argument("--len_sigma", type=float, default=1.0)
    ap.add_argument("--input_len_min", type=int, default=4)
    ap.add_argument("--input_len_max", type=int, default=2048)
    ap.add_argument("--output_len_min", type=int, default=4)
    ap.add_argument("--output_len_max", type=int, default=1024)
    ap.add_argument("--vocab_size", type=int, default=32000)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--output", default="", help="write every request's generated tokens / text to this JSONL file")
    asyncio.run(run(ap.parse_args()))


if __name__ == "__main__":
    main()
