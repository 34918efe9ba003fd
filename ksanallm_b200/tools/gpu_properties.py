"""Prints what the build and the kernels need to know about the visible GPUs: compute capability (the -gencode
target), SM count, shared memory per block, L2 size, memory size, peer access matrix.
Counterpart of the reference's tools/get_nvidia_gpu_properties.py (which feeds the SM list to CMake).

    python -m ksanallm_b200.tools.gpu_properties [--json]
"""
from __future__ import annotations

import argparse
import json
from typing import Any, Dict, List


def gpu_properties() -> List[Dict[str, Any]]:
    import torch
    out = []
    if not torch.cuda.is_available():
        return out
    n = torch.cuda.device_count()
    for i in range(n):
        p = torch.cuda.get_device_properties(i)
        out.append({
            "index": i, "name": p.name, "compute_capability": f"{p.major}.{p.minor}",
            "gencode": f"arch=compute_{p.major}{p.minor}a,code=sm_{p.major}{p.minor}a" if p.major >= 9
            else f"arch=compute_{p.major}{p.minor},code=sm_{p.major}{p.minor}",
            "sm_count": p.multi_processor_count, "memory_gib": round(p.total_memory / 2 ** 30, 1),
            "l2_mib": round(getattr(p, "L2_cache_size", 0) / 2 ** 20, 1),
            "shared_memory_per_block_optin_kib": round(getattr(p, "shared_memory_per_block_optin", 0) / 1024, 1),
            "peers": [j for j in range(n) if j != i and torch.cuda.can_device_access_peer(i, j)],
        })
    return out


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", action="store_true")
    ns = ap.parse_args(argv)
    props = gpu_properties()
    if ns.json:
        print(json.dumps(props, indent=1))
        return
    if not props:
        print("no CUDA device visible (the sm_100a build needs none: nvcc cross-compiles)")
    for p in props:
        print(f"GPU {p['index']}: {p['name']}  sm_{p['compute_capability'].replace('.', '')}  {p['sm_count']} SMs  "
              f"{p['memory_gib']} GiB  L2 {p['l2_mib']} MiB  smem/block {p['shared_memory_per_block_optin_kib']} KiB  "
              f"peers {p['peers']}")


if __name__ == "__main__":
    main()
