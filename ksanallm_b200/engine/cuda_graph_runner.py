"""CUDA-graph capture / replay keyed by (padded) batch size.

The reference carries a ``CudaGraphBuilder`` (which batch sizes to capture, how a batch size is padded) and a
``CudaGraphRunner`` (begin / end capture, launch by key) that its forward pass does not use yet
(src/ksana_llm/runtime/cuda_graph_runner.{h,cpp}; models/base/base_model.h:60-64). This module offers the same two
pieces on top of ``torch.cuda.CUDAGraph``:

* every kernel of this package launches on the current torch stream, so a step made of them can be captured;
* a captured callable must read its inputs from, and write its outputs to, fixed buffers: ``capture`` therefore takes
  the static input tensors, ``replay`` copies fresh values into them before launching;
* on a machine without CUDA the runner records the callable and calls it eagerly, so the keying / padding logic is
  exercised by the CPU tests as well.

The engine's own answer to launch overhead is the one-call-per-step native executor plus asynchronous scheduling;
the graph runner is for callers whose step has host-independent launch parameters (fixed batch size, fixed split
counts).
"""
from __future__ import annotations

from typing import Callable, Dict, Hashable, List, Optional, Sequence

import torch


class CudaGraphBuilder:
    """Which batch sizes get a graph: 1, 2, 4, then every multiple of ``step`` up to ``max_batch_size``."""

    def __init__(self, max_batch_size: int = 256, step: int = 8):
        if max_batch_size < 1 or step < 1:
            raise ValueError("max_batch_size and step must be positive")
        self.max_batch_size, self.step = int(max_batch_size), int(step)

    def capture_list(self) -> List[int]:
        sizes = [b for b in (1, 2, 4) if b <= self.max_batch_size and b < self.step]
        sizes += list(range(self.step, self.max_batch_size + 1, self.step))
        if not sizes or sizes[-1] < self.max_batch_size:
            sizes.append(self.max_batch_size)
        return sizes

    def padded(self, batch_size: int) -> Optional[int]:
        """Smallest captured size that holds ``batch_size`` rows; None when it exceeds every graph."""
        for b in self.capture_list():
            if b >= batch_size:
                return b
        return None


class _Entry:
    __slots__ = ("graph", "fn", "inputs", "outputs")

    def __init__(self, graph, fn, inputs, outputs):
        self.graph, self.fn, self.inputs, self.outputs = graph, fn, inputs, outputs


class CudaGraphRunner:
    def __init__(self, device: Optional[torch.device] = None, warmup_runs: int = 2):
        self.device = torch.device(device) if device is not None else \
            torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.warmup_runs = warmup_runs
        self._entries: Dict[Hashable, _Entry] = {}
        self._pool = None
        self.is_capturing = False
        self.launches = 0

    @property
    def captured_keys(self):
        return set(self._entries)

    def has(self, key: Hashable) -> bool:
        return key in self._entries

    def capture(self, key: Hashable, fn: Callable[..., object], static_inputs: Sequence[torch.Tensor]):
        """Runs ``fn(*static_inputs)`` a few times on a side stream (lazy initialisation, autotuning and workspace
        growth must happen outside the capture), then records it. Returns the static outputs."""
        if key in self._entries:
            raise KeyError(f"graph {key!r} already captured")
        inputs = list(static_inputs)
        if self.device.type != "cuda":
            out = fn(*inputs)
            self._entries[key] = _Entry(None, fn, inputs, out)
            return out
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(self.warmup_runs):
                fn(*inputs)
        torch.cuda.current_stream(self.device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        self.is_capturing = True
        try:
            with torch.cuda.graph(graph, pool=self._pool):
                out = fn(*inputs)
        finally:
            self.is_capturing = False
        if self._pool is None:
            self._pool = graph.pool()  # later graphs share the first one's memory pool
        self._entries[key] = _Entry(graph, fn, inputs, out)
        return out

    def replay(self, key: Hashable, inputs: Optional[Sequence[torch.Tensor]] = None):
        """Copies ``inputs`` (leading rows may be fewer than the static buffers hold) into the static buffers and
        launches the graph. Returns the static outputs: the caller reads them before the next replay of this key."""
        e = self._entries[key]
        if inputs is not None:
            if len(inputs) != len(e.inputs):
                raise ValueError(f"graph {key!r} takes {len(e.inputs)} inputs, got {len(inputs)}")
            for dst, src in zip(e.inputs, inputs):
                if src.shape == dst.shape:
                    dst.copy_(src, non_blocking=True)
                else:
                    if src.dim() != dst.dim() or src.shape[0] > dst.shape[0] or src.shape[1:] != dst.shape[1:]:
                        raise ValueError(f"input of shape {tuple(src.shape)} does not fit {tuple(dst.shape)}")
                    dst[:src.shape[0]].copy_(src, non_blocking=True)
        self.launches += 1
        if e.graph is None:
            e.outputs = e.fn(*e.inputs)
        else:
            e.graph.replay()
        return e.outputs

    def clear(self) -> None:
        self._entries.clear()
        self._pool = None
