"""Attention data parallelism with expert parallelism for the MoE blocks.

Every rank (DP group of one rank here) owns its own requests, scheduler and KV cache and holds the full attention /
dense weights; only the routed experts are sharded over the ranks. All ranks step in lock-step: each MoE block is
a collective exchange (tokens to the ranks hosting their experts, weighted outputs back), so a rank without work
still runs a "mock" step with zero tokens. This mirrors the reference's attn_data_para_size mode: per-DP-group
strategies and cache managers (src/ksana_llm/service/inference_engine.cpp:201-260), mock requests so idle EP ranks
still run a step (batch_scheduler/batch_scheduler.cpp:472-519) and the cross-DP synchronisation of step sizes.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops


class DPCoordinator:
    """Per-step agreement between the DP ranks: the largest token count of any rank (the slot stride of the
    expert exchange) and whether anybody still has work."""

    def __init__(self, group=None, device: Optional[torch.device] = None):
        self.group = group
        self.device = device or torch.device("cpu")
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)

    def sync(self, local_tokens: int, has_unfinished: bool) -> Tuple[int, bool]:
        t = torch.tensor([local_tokens, 1 if has_unfinished else 0], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return int(t[0]), bool(t[1])


class GatherEPExchange:
    """Same contract as parallel.ep.EPExchange.moe, built from torch.distributed collectives (works on gloo and
    NCCL): all-gather the padded token slots, run the local experts on everything, sum the partial outputs and keep
    the rank's own rows. Used on CPU and wherever symmetric memory is not available."""

    def __init__(self, group, rank: int, size: int, top_k: int, num_experts: int):
        assert num_experts % size == 0
        self.group, self.rank, self.size, self.top_k = group, rank, size, top_k
        self.e_local = num_experts // size
        self.step_stride = 0

    def moe(self, x, ids, weights, w_gate_up, w_down, t_stride, add=None):
        T, H = x.shape
        k = self.top_k
        xp = x.new_zeros(t_stride, H)
        ip = torch.full((t_stride, k), -1, dtype=torch.int32, device=x.device)
        wp = torch.zeros(t_stride, k, dtype=torch.float32, device=x.device)
        if T:
            xp[:T], ip[:T], wp[:T] = x, ids.to(torch.int32), weights.float()
        xg = [torch.empty_like(xp) for _ in range(self.size)]
        ig = [torch.empty_like(ip) for _ in range(self.size)]
        wg = [torch.empty_like(wp) for _ in range(self.size)]
        dist.all_gather(xg, xp, group=self.group)
        dist.all_gather(ig, ip, group=self.group)
        dist.all_gather(wg, wp, group=self.group)
        y = ops.moe_experts(torch.cat(xg), torch.cat(ig), torch.cat(wg), w_gate_up, w_down, self.rank * self.e_local)
        y = y.float()
        dist.all_reduce(y, group=self.group)
        out = y[self.rank * t_stride:self.rank * t_stride + T].to(x.dtype)
        return out if add is None else out + add
