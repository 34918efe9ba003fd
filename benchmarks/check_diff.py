"""Compares the generations of two benchmark runs (``benchmark_throughput.py --output``): exact-match rate, the
first position where each pair diverges, and a ROUGE-L style overlap of the token sequences - the quick check that a
kernel or scheduling change did not alter what the model says. Counterpart of the reference's
benchmarks/check_diff.py (mismatch + ROUGE report between result files).

    python benchmarks/check_diff.py run_a.jsonl run_b.jsonl [--threshold 0.98]
"""
import argparse
import json
import sys
from typing import List, Sequence


def lcs(a: Sequence, b: Sequence) -> int:
    prev = [0] * (len(b) + 1)
    for x in a:
        cur = [0]
        for j, y in enumerate(b):
            cur.append(prev[j] + 1 if x == y else max(prev[j + 1], cur[j]))
        prev = cur
    return prev[-1]


def rouge_l(a: Sequence, b: Sequence) -> float:
    if not a or not b:
        return 1.0 if not a and not b else 0.0
    l = lcs(a, b)
    p, r = l / len(b), l / len(a)
    return 0.0 if l == 0 else 2 * p * r / (p + r)


def first_diff(a: Sequence, b: Sequence) -> int:
    for i, (x, y) in enumerate(zip(a, b)):
        if x != y:
            return i
    return -1 if len(a) == len(b) else min(len(a), len(b))


def load(path: str) -> List[dict]:
    with open(path, "r", encoding="utf-8") as f:
        return [json.loads(line) for line in f if line.strip()]


def compare(a: List[dict], b: List[dict]) -> dict:
    n = min(len(a), len(b))
    exact, scores, diffs = 0, [], []
    for x, y in zip(a[:n], b[:n]):
        ta, tb = x.get("output_token_ids") or list(x.get("text", "")), y.get("output_token_ids") or list(y.get("text", ""))
        d = first_diff(ta, tb)
        exact += d < 0
        scores.append(rouge_l(ta, tb))
        if d >= 0:
            diffs.append({"index": x.get("index"), "first_diff_at": d, "rouge_l": round(scores[-1], 4)})
    return {"compared": n, "exact_match": exact, "exact_rate": exact / n if n else 1.0,
            "mean_rouge_l": sum(scores) / n if n else 1.0, "mismatches": diffs}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("a")
    ap.add_argument("b")
    ap.add_argument("--threshold", type=float, default=0.0, help="fail (exit 1) when the mean ROUGE-L is below this")
    ap.add_argument("--show", type=int, default=10, help="mismatching requests to list")
    ns = ap.parse_args(argv)
    rep = compare(load(ns.a), load(ns.b))
    rep["mismatches"] = rep["mismatches"][:ns.show]
    print(json.dumps(rep, indent=1))
    return 1 if rep["mean_rouge_l"] < ns.threshold else 0


if __name__ == "__main__":
    sys.exit(main())
