"""Tensor-parallel communication front door.

One process per GPU (``torch.distributed``: NCCL on GPUs, gloo on CPU). The model code talks to a
:class:`TPGroup`; whether a reduction is a library collective (the measured baseline) or one of the
fused peer-memory kernels (``parallel.fused``) is decided here, so model definitions are identical for
TP=1 and TP>1. Reference counterpart: ModelCommunicator / TpCommunicator
(src/ksana_llm/models/base/model_communicator.cpp:158-168, models/communicator/tp_communicator.cpp) and
FusedAllReduceNormAdd (src/ksana_llm/modules/basic/all_reduce_fused_norm_add.cpp:30-53).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops


class TPGroup:
    """Tensor-parallel group handle. ``size == 1`` makes every collective the identity."""

    def __init__(self, rank: int = 0, size: int = 1, group=None, device: Optional[torch.device] = None,
                 use_fused: bool = True):
        self.rank = rank
        self.size = size
        self.group = group
        self.device = device
        self.use_fused = use_fused and size > 1
        self.fused = None  # parallel.fused.FusedComm, attached by init_fused()
        self.ep = None     # parallel.ep.EPExchange, attached by init_ep()
        self.ep_dp = False  # attention data parallelism: this rank's tokens are its own (parallel/attn_dp.py)
        self.ep_rank, self.ep_size = rank, size  # expert sharding (differs from rank/size under attention DP)
        self.stats = {"all_reduce": 0, "all_gather": 0, "fused": 0}

    def init_fused(self, hidden: int, max_tokens: int, use_multicast: Optional[bool] = None) -> bool:
        """Collective: allocates the symmetric heap and attaches the fused kernels. No-op for size 1, on CPU
        or when fused kernels were disabled for this group (library-collective baseline)."""
        if self.size == 1 or not self.use_fused or self.device is None or self.device.type != "cuda":
            return False
        from .fused import FusedComm
        self.fused = FusedComm(self.group, self.rank, self.size, self.device, hidden, max_tokens, use_multicast)
        return True

    # ---- plain collectives ------------------------------------------------------------------------
    def init_ep(self, hidden: int, top_k: int, num_experts: int, max_tokens: int) -> bool:
        """Attaches the peer-memory expert-parallel exchange (token dispatch / combine instead of running every
        local expert over every token). Only for CUDA groups of 2..8 ranks with experts divisible by the size."""
        if self.size < 2 or self.size > 8 or self.device is None or self.device.type != "cuda":
            return False
        if num_experts % self.size:
            return False
        from .ep import EPExchange
        per_rank = (max_tokens + self.size - 1) // self.size
        self.ep = EPExchange(self.group, self.rank, self.size, self.device, hidden, top_k, num_experts, per_rank)
        return True

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        self.stats["all_reduce"] += 1
        if self.fused is not None and x.is_cuda and self.fused.can_all_reduce(x):
            return self.fused.all_reduce(x)
        if x.dtype in (torch.bfloat16, torch.float16) and not x.is_cuda:
            y = x.float()
            dist.all_reduce(y, group=self.group)
            return y.to(x.dtype)
        dist.all_reduce(x, group=self.group)
        return x

    def all_gather(self, x: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if self.size == 1:
            return x
        self.stats["all_gather"] += 1
        x = x.contiguous()
        parts = [torch.empty_like(x) for _ in range(self.size)]
        dist.all_gather(parts, x, group=self.group)
        return torch.cat(parts, dim=dim)

    def broadcast(self, x: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.size > 1:
            dist.broadcast(x, src=dist.get_global_rank(self.group, src) if self.group is not None else src,
                           group=self.group)
        return x

    def barrier(self) -> None:
        if self.size > 1:
            dist.barrier(group=self.group)

    # ---- fused row-parallel paths -------------------------------------------------------------------
    def row_linear(self, x: torch.Tensor, lin, reduce: bool = True) -> torch.Tensor:
        """Row-parallel linear: partial GEMM on each rank, then sum across the group."""
        y = lin(x, add_bias=self.rank == 0)
        return self.all_reduce(y) if reduce else y

    def row_linear_add_norm(self, x: torch.Tensor, lin, residual: torch.Tensor, norm_weight: torch.Tensor,
                            eps: float) -> torch.Tensor:
        """h = RMSNorm(residual += AllReduce(x @ W^T)) * norm_weight, residual updated in place.

        With the fused backend this is ONE kernel: tcgen05 GEMM tiles are pushed to their owner rank over
        NVLink, reduced, the residual add and RMSNorm run on the owner and the normalised rows are
        broadcast back. Otherwise GEMM -> all-reduce -> fused add+norm kernel."""
        if self.fused is not None and x.is_cuda and self.fused.can_linear_reduce_norm(x, lin):
            self.stats["fused"] += 1
            return self.fused.linear_reduce_add_norm(x, lin, residual, norm_weight, eps)
        y = self.row_linear(x, lin)
        return ops.rms_norm(y, norm_weight, eps, residual)


    def reduce_add_norm(self, y: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor,
                        eps: float) -> torch.Tensor:
        """h = RMSNorm(residual += AllReduce(y)) * norm_weight for an already computed partial sum."""
        if self.fused is not None and y.is_cuda and self.fused.can_all_reduce(y):
            self.stats["fused"] += 1
            return self.fused.reduce_add_norm(y, residual, norm_weight, eps)
        return ops.rms_norm(self.all_reduce(y), norm_weight, eps, residual)


_WORLD: Optional[TPGroup] = None


def init_distributed(device_type: str = "cuda", use_fused: bool = True) -> TPGroup:
    """Creates the process group from torchrun-style environment variables (RANK, WORLD_SIZE,
    LOCAL_RANK, MASTER_ADDR, MASTER_PORT). Single-process runs need no environment at all."""
    global _WORLD
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # torchrun names first; the reference's launch variables (NODE_RANK / MASTER_HOST, README "multi-node") are
    # accepted for processes started by hand, one per GPU
    rank = int(os.environ.get("RANK", os.environ.get("NODE_RANK", "0")))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if device_type == "cuda":
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
    else:
        device = torch.device("cpu")
    if world == 1:
        _WORLD = TPGroup(0, 1, None, device, use_fused=False)
        return _WORLD
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", os.environ.get("MASTER_HOST", "127.0.0.1"))
        os.environ.setdefault("MASTER_PORT", "29511")
        backend = "nccl" if device_type == "cuda" else "gloo"
        kwargs = {"device_id": device} if device_type == "cuda" else {}
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    _WORLD = TPGroup(rank, world, dist.group.WORLD, device, use_fused=use_fused)
    return _WORLD


def world_group() -> TPGroup:
    return _WORLD if _WORLD is not None else TPGroup()
