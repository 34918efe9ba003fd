"""Expert-parallel load balancing: from dumped routing statistics (expert ids chosen per token, per layer) compute a
placement of experts onto EP ranks that equalises the load, optionally replicating the hottest experts.
Counterpart of the reference's tools/eplb/expert_parallel_get_map.py (dump via DUMP_EPLB_PATH, reload via EPLB_WEIGHT).

    python -m ksanallm_b200.tools.eplb stats.json --ranks 8 --out eplb_map.json
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, List


def balance_experts(load: List[float], num_ranks: int, redundant: int = 0) -> Dict[str, object]:
    """Greedy LPT placement. Returns {"rank_of_expert": [...], "replicas": {expert: [ranks]}, "rank_load": [...]}."""
    E = len(load)
    per_rank = (E + redundant + num_ranks - 1) // num_ranks
    items = [(load[e], e, 1.0) for e in range(E)]
    # replicate the hottest experts: each replica carries an equal share of the expert's load
    hot = sorted(range(E), key=lambda e: -load[e])[:redundant]
    for e in hot:
        items = [(l / 2, x, s / 2) if x == e else (l, x, s) for l, x, s in items]
        items.append((load[e] / 2, e, 0.5))
    items.sort(key=lambda t: -t[0])
    rank_load = [0.0] * num_ranks
    rank_cnt = [0] * num_ranks
    placement: Dict[int, List[int]] = {}
    for l, e, _ in items:
        cands = [r for r in range(num_ranks) if rank_cnt[r] < per_rank and r not in placement.get(e, [])]
        r = min(cands, key=lambda x: rank_load[x])
        rank_load[r] += l
        rank_cnt[r] += 1
        placement.setdefault(e, []).append(r)
    return {"rank_of_expert": [placement[e][0] for e in range(E)],
            "replicas": {str(e): rs for e, rs in placement.items() if len(rs) > 1},
            "rank_load": rank_load}


def permutation_from_map(rank_of_expert: List[int], num_ranks: int) -> List[int]:
    """Logical expert id -> physical slot, where rank r hosts the physical slots [r * E / ranks, (r + 1) * E / ranks).
    Experts keep their relative order inside a rank; a rank given more than its share passes the surplus on to the
    ranks with room (the placement must be a permutation: replicas are not expressed here)."""
    E = len(rank_of_expert)
    per = E // num_ranks
    buckets: List[List[int]] = [[] for _ in range(num_ranks)]
    spill = []
    for e, r in enumerate(rank_of_expert):
        (buckets[r] if len(buckets[r]) < per else spill).append(e)
    for b in buckets:
        while len(b) < per and spill:
            b.append(spill.pop(0))
    perm = [0] * E
    for r, b in enumerate(buckets):
        for i, e in enumerate(b):
            perm[e] = r * per + i
    return perm


def load_expert_permutations(path: str, num_experts: int, num_ranks: int) -> Dict[int, List[int]]:
    """Reads a placement file written by this tool ({layer: {"rank_of_expert": [...]}}) or a dump of routing counts
    ({layer: [count per expert]}, balanced here) and returns {layer index: permutation}."""
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    out = {}
    for layer, v in raw.items():
        if isinstance(v, dict) and "rank_of_expert" in v:
            roe = v["rank_of_expert"]
        else:
            roe = balance_experts([float(x) for x in v], num_ranks)["rank_of_expert"]
        if len(roe) == num_experts:
            out[int(str(layer).split("_")[-1])] = permutation_from_map(roe, num_ranks)
    return out


def load_from_topk_ids(ids_per_layer: Dict[str, List[List[int]]], num_experts: int) -> Dict[str, List[float]]:
    out = {}
    for layer, rows in ids_per_layer.items():
        cnt = [0.0] * num_experts
        for row in rows:
            for e in row:
                cnt[e] += 1
        out[layer] = cnt
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("stats")
    ap.add_argument("--ranks", type=int, default=8)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--redundant", type=int, default=0)
    ap.add_argument("--out", default="eplb_map.json")
    a = ap.parse_args(argv)
    with open(a.stats) as f:
        stats = json.load(f)
    first = next(iter(stats.values()))
    if first and isinstance(first[0], (int, float)):  # the engine's dump: routing counts per expert
        loads = {layer: [float(x) for x in v] for layer, v in stats.items()}
    else:
        loads = load_from_topk_ids(stats, a.experts)
    result = {layer: balance_experts(l, a.ranks, a.redundant) for layer, l in loads.items()}
    with open(a.out, "w") as f:
        json.dump(result, f)
    print(f"wrote {a.out}: {len(result)} layers")


if __name__ == "__main__":
    main()
