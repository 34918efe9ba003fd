"""Debug aids for memory corruption.

* ``GuardedBuffer``: a tensor padded with guard bands filled with a sentinel pattern, checked after kernels ran
  (the reference's MemoryChecker, env ENABLE_MEMORY_CHECK: src/ksana_llm/utils/tensor.h:160-193, tensor.cpp:436-479).
* ``block_checksums`` / ``BlockChecksumTracker``: per-block checksums of the KV cache taken before and after a step to
  catch corruption by swap / merge races (reference: setting.block_manager.enable_block_checksum,
  CalculateChecksumKernel cache_copy.cu:407, verification in models/base/model_input.cpp:380-530).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch

_SENTINEL = 0x5A


class GuardedBuffer:
    def __init__(self, shape, dtype=torch.bfloat16, device="cpu", guard_bytes: int = 256):
        n = 1
        for s in shape:
            n *= s
        esz = torch.empty(0, dtype=dtype).element_size()
        self.guard = guard_bytes
        self.raw = torch.full((n * esz + 2 * guard_bytes,), _SENTINEL, dtype=torch.uint8, device=device)
        self.tensor = self.raw[guard_bytes:guard_bytes + n * esz].view(dtype).view(*shape)

    def check(self) -> bool:
        head = self.raw[:self.guard]
        tail = self.raw[-self.guard:]
        return bool((head == _SENTINEL).all() and (tail == _SENTINEL).all())


def block_checksums(kv_cache: torch.Tensor, blocks: Iterable[int]) -> torch.Tensor:
    """64-bit position-weighted sums (odd multipliers, wrapping) of the raw 32-bit words of the given blocks of one
    layer's cache: a plain byte sum misses changes that move a carry between bytes of one value."""
    idx = torch.as_tensor(list(blocks), dtype=torch.long, device=kv_cache.device)
    sel = kv_cache.index_select(0, idx).contiguous()
    raw = sel.view(sel.shape[0], -1).view(torch.uint8)
    if raw.shape[1] % 4:
        raw = torch.nn.functional.pad(raw, (0, 4 - raw.shape[1] % 4))
    words = raw.view(torch.int32).to(torch.int64)
    weights = torch.arange(words.shape[1], dtype=torch.int64, device=words.device) * 2 + 1
    return (words * weights).sum(dim=1)


class BlockChecksumTracker:
    """Remembers checksums of blocks that must not change (full, committed prefix blocks) and verifies them."""

    def __init__(self):
        self.known: Dict[int, int] = {}

    def remember(self, kv_cache: torch.Tensor, blocks: List[int]) -> None:
        if not blocks:
            return
        for b, c in zip(blocks, block_checksums(kv_cache, blocks).tolist()):
            self.known[b] = c

    def forget(self, blocks: Iterable[int]) -> None:
        for b in blocks:
            self.known.pop(b, None)

    def verify(self, kv_cache: torch.Tensor) -> List[int]:
        """Returns the blocks whose content changed."""
        if not self.known:
            return []
        blocks = list(self.known)
        now = block_checksums(kv_cache, blocks).tolist()
        return [b for b, c in zip(blocks, now) if c != self.known[b]]
