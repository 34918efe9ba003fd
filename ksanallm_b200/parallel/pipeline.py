"""Pipeline parallelism: contiguous layer ranges per stage, hidden states handed from stage to stage with point-to-point
sends, and the micro-batch controller that decides which micro-batch may occupy a stage.

The reference runs PP across nodes only: the master assigns layer ranges (src/ksana_llm/distributed/
control_channel.cpp:577 SynchronizeNodeLayers), hidden units travel over NcclDataChannel / TCP
(distributed/nvidia/nccl_data_channel.cpp:81-336, data_hub/hidden_unit_buffer.cpp) and MultiBatchController
(multi_batch_controller/multi_batch_controller.cpp:8-168) serialises the micro-batches. Here a stage is one rank
(or one TP group) of the same torch.distributed world: NCCL send/recv on GPUs, gloo on CPU.

Only the un-normalised residual stream [T, H] crosses a stage boundary: the receiving stage applies its own first
input norm, so nothing of the next stage's weights is needed upstream.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass
from enum import Enum
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


def split_layers(num_layers: int, num_stages: int, first_stage_offload: int = 0) -> List[range]:
    """Contiguous layer ranges, as even as possible; ``first_stage_offload`` layers are moved off the first stage
    (it also holds the embedding and drives scheduling; the reference's MASTER_OFFLOAD_LAYER_NUM)."""
    assert 1 <= num_stages <= max(num_layers, 1)
    base, rem = divmod(num_layers, num_stages)
    sizes = [base + (1 if i < rem else 0) for i in range(num_stages)]
    off = min(first_stage_offload, max(sizes[0] - 1, 0)) if num_stages > 1 else 0
    sizes[0] -= off
    for i in range(off):
        sizes[1 + i % (num_stages - 1)] += 1
    out, lo = [], 0
    for s in sizes:
        out.append(range(lo, lo + s))
        lo += s
    return out


@dataclass
class StageTopology:
    """World layout: rank = stage * tp_size + tp_rank."""
    world_size: int
    tp_size: int
    rank: int

    @property
    def num_stages(self) -> int:
        return self.world_size // self.tp_size

    @property
    def stage(self) -> int:
        return self.rank // self.tp_size

    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp_size

    @property
    def is_first(self) -> bool:
        return self.stage == 0

    @property
    def is_last(self) -> bool:
        return self.stage == self.num_stages - 1

    def peer(self, stage: int) -> int:
        """Global rank of the same TP position on another stage."""
        return stage * self.tp_size + self.tp_rank

    def tp_ranks(self, stage: Optional[int] = None) -> List[int]:
        s = self.stage if stage is None else stage
        return list(range(s * self.tp_size, (s + 1) * self.tp_size))


class HiddenChannel:
    """Point-to-point transport of [T, H] activations between adjacent stages (and of sampled tokens back to the
    driver). ``torch.distributed`` send/recv: NCCL for CUDA tensors, gloo otherwise."""

    def __init__(self, topo: StageTopology, hidden: int, dtype: torch.dtype, device: torch.device, group=None):
        self.topo, self.hidden, self.dtype, self.device, self.group = topo, hidden, dtype, device, group
        # On GPUs the activations travel over NCCL, whose point-to-point operations run in issue order on one stream
        # per communicator. The results' way back (last stage -> driver) crosses that order as soon as two
        # micro-batches are in flight: the driver's second send waits for the last stage's second receive, which is
        # queued behind its send of the first results, which waits for a receive the driver has queued behind that
        # second send. So the (small) results go back over a host-side group of their own; every rank creates it here,
        # in the same order. Found on two GPUs: the first NCCL run of the two-stage test stopped exactly there.
        self.back_group = None
        if torch.device(device).type == "cuda" and dist.is_initialized() and dist.get_world_size() > 1:
            self.back_group = dist.new_group(backend="gloo")

    def send_hidden(self, x: torch.Tensor) -> None:
        dist.send(x.contiguous(), dst=self.topo.peer(self.topo.stage + 1), group=self.group)

    def recv_hidden(self, tokens: int) -> torch.Tensor:
        buf = torch.empty(tokens, self.hidden, dtype=self.dtype, device=self.device)
        dist.recv(buf, src=self.topo.peer(self.topo.stage - 1), group=self.group)
        return buf

    def send_tokens(self, toks: torch.Tensor, dst_rank: int = 0) -> None:
        """Non-blocking: with several micro-batches in flight the driver only posts the matching receive after it
        has launched the next micro-batch, so a blocking send here could dead-lock against its plan broadcast."""
        buf = toks.to(torch.int32).contiguous()
        self._isend_back(buf, dst_rank)

    def _isend_back(self, buf: torch.Tensor, dst_rank: int) -> None:
        grp = self.group
        if self.back_group is not None:
            buf, grp = buf.cpu(), self.back_group
        self._pending_sends = [(w, b) for w, b in getattr(self, "_pending_sends", []) if not w.is_completed()]
        self._pending_sends.append((dist.isend(buf, dst=dst_rank, group=grp), buf))

    def _recv_back(self, shape, dtype, src_rank: int) -> torch.Tensor:
        if self.back_group is not None:
            buf = torch.empty(shape, dtype=dtype)
            dist.recv(buf, src=src_rank, group=self.back_group)
            return buf.to(self.device)
        buf = torch.empty(shape, dtype=dtype, device=self.device)
        dist.recv(buf, src=src_rank, group=self.group)
        return buf

    def send_logits(self, logits: torch.Tensor, dst_rank: int = 0) -> None:
        """Rows that are not sampled greedily: the sampling state (penalties, generators, grammar masks) lives on the
        driver, so the last stage returns the fp32 logits of those rows instead of tokens (non-blocking, see
        send_tokens). The reference returns the hidden states to the chief node, which owns lm_head + sampler
        (runtime/llm_runtime.cpp:76-110); here lm_head stays with the last stage."""
        self._isend_back(logits.float().contiguous(), dst_rank)

    def recv_logits(self, count: int, vocab: int, src_rank: int) -> torch.Tensor:
        return self._recv_back((count, vocab), torch.float32, src_rank)

    def recv_tokens(self, count: int, src_rank: int) -> torch.Tensor:
        return self._recv_back((count,), torch.int32, src_rank)


class BatchState(Enum):
    NOT_READY = 0   # nothing scheduled for this micro-batch
    STANDBY = 1     # scheduled, waiting for its turn on the device
    RUNNING = 2     # owns the device
    FINISHED = 3    # forward done, results not collected yet


class MultiBatchController:
    """Serialises ``n`` micro-batches over one stage's device. A micro-batch may start running when (a) no other
    one is running and (b) it is the oldest one in STANDBY (arrival order = the order hidden states will arrive
    from the previous stage, so receives never dead-lock). Threads call ``wait_turn`` / ``done``; the single-thread
    engines use ``next_runnable``."""

    def __init__(self, n: int):
        self.n = n
        self.state: List[BatchState] = [BatchState.NOT_READY] * n
        self._order: List[int] = []  # STANDBY micro-batches, oldest first
        self._cv = threading.Condition()
        self.history: List[int] = []

    def ready(self, mb: int) -> None:
        with self._cv:
            assert self.state[mb] in (BatchState.NOT_READY, BatchState.FINISHED), self.state[mb]
            self.state[mb] = BatchState.STANDBY
            self._order.append(mb)
            self._cv.notify_all()

    def next_runnable(self) -> Optional[int]:
        with self._cv:
            if any(s == BatchState.RUNNING for s in self.state) or not self._order:
                return None
            return self._order[0]

    def start(self, mb: int) -> None:
        with self._cv:
            assert self._order and self._order[0] == mb and not any(s == BatchState.RUNNING for s in self.state)
            self._order.pop(0)
            self.state[mb] = BatchState.RUNNING
            self.history.append(mb)

    def wait_turn(self, mb: int, timeout: Optional[float] = None) -> bool:
        with self._cv:
            ok = self._cv.wait_for(lambda: self._order and self._order[0] == mb and
                                   not any(s == BatchState.RUNNING for s in self.state), timeout)
            if ok:
                self._order.pop(0)
                self.state[mb] = BatchState.RUNNING
                self.history.append(mb)
            return ok

    def done(self, mb: int) -> None:
        with self._cv:
            assert self.state[mb] == BatchState.RUNNING
            self.state[mb] = BatchState.FINISHED
            self._cv.notify_all()

    def collected(self, mb: int) -> None:
        with self._cv:
            assert self.state[mb] == BatchState.FINISHED
            self.state[mb] = BatchState.NOT_READY
            self._cv.notify_all()


class PipelineStage:
    """Runs one stage of a step: receive (unless first) -> local layers -> send (unless last)."""

    def __init__(self, model, topo: StageTopology, channel: HiddenChannel):
        self.model, self.topo, self.channel = model, topo, channel

    @torch.inference_mode()
    def run(self, meta, kv_caches, refit=None) -> Optional[torch.Tensor]:
        """Returns the final normalised hidden states on the last stage, None elsewhere."""
        hidden_in = None if self.topo.is_first else self.channel.recv_hidden(meta.total_tokens)
        out = self.model.forward(meta, kv_caches, refit, hidden_in=hidden_in)
        if self.topo.is_last:
            return out
        # every TP rank of a stage holds the same reduced residual: each sends to its own peer
        self.channel.send_hidden(out)
        return None
