"""Per-step device metadata ("model input").

The scheduler serialises one step into a single int32 staging buffer (pinned on GPU hosts); this
module turns it into device tensor views after ONE host-to-device copy. The reference builds the
same information field by field on side streams (src/ksana_llm/models/base/model_input.cpp,
1711 lines); here every field is a slice of one buffer so the copy and the CUDA-graph input
binding are both trivial.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np
import torch


@dataclass
class StepInput:
    input_ids: torch.Tensor      # [T] int32
    positions: torch.Tensor      # [T] int32
    slot_mapping: torch.Tensor   # [T] int32, block * block_size + offset
    seq_of_token: torch.Tensor   # [T] int32, batch row of each token
    cu_q: torch.Tensor           # [B + 1] int32
    kv_lens: torch.Tensor        # [B] int32, context length including this step's tokens
    q_starts: torch.Tensor       # [B] int32, tokens already cached before this step
    logits_idx: torch.Tensor     # [L] int32, rows of the hidden state that need logits
    block_tables: torch.Tensor   # [B, max_blocks] int32
    num_seqs: int
    num_prefill: int
    num_decode: int
    total_tokens: int
    total_logits: int
    max_q_len: int
    max_kv_len: int
    max_blocks: int
    h2d_bytes: int = 0
    # host copies of the small per-sequence arrays (kernel launch decisions never sync the device)
    cu_q_host: Optional[np.ndarray] = None
    kv_lens_host: Optional[np.ndarray] = None
    # multimodal RoPE: [3, T] (temporal, height, width) positions; None for plain text steps
    mrope_positions: Optional[torch.Tensor] = None
    _mrope_table: Optional[torch.Tensor] = None
    _arange: Optional[torch.Tensor] = None

    @property
    def num_decode_tokens(self) -> int:
        if self.num_decode == 0:
            return 0
        return int(self.cu_q_host[self.num_seqs] - self.cu_q_host[self.num_prefill])

    @property
    def num_prefill_tokens(self) -> int:
        return int(self.cu_q_host[self.num_prefill]) if self.num_prefill else 0


class StepStaging:
    """Host staging buffer + its device mirror."""

    def __init__(self, capacity_words: int, device: torch.device):
        self.device = torch.device(device)
        pin = self.device.type == "cuda"
        # two host buffers: with asynchronous scheduling the next step is packed while the previous step's
        # host-to-device copy may not have run yet
        self._hosts = [torch.empty(capacity_words, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._cur = 0
        self.host = self._hosts[0]
        self.host_np = self.host.numpy()
        self.dev = self.host if self.device.type == "cpu" else torch.empty(
            capacity_words, dtype=torch.int32, device=self.device)

    def flip(self) -> None:
        if self.dev is self.host:
            return  # CPU: the "device" view IS the host buffer and steps run synchronously
        self._cur ^= 1
        self.host = self._hosts[self._cur]
        self.host_np = self.host.numpy()

    def upload(self, layout: Dict[str, int]) -> StepInput:
        n = layout["total_words"]
        if self.dev is not self.host:
            self.dev[:n].copy_(self.host[:n], non_blocking=True)
        d = self.dev
        T, B, L, mb = layout["total_tokens"], layout["num_seqs"], layout["total_logits"], layout["max_blocks"]

        def sl(name, count):
            o = layout[name]
            return d[o:o + count]

        hn = self.host_np
        return StepInput(
            input_ids=sl("input_ids", T), positions=sl("positions", T), slot_mapping=sl("slot_mapping", T),
            seq_of_token=sl("seq_of_token", T), cu_q=sl("cu_q", B + 1), kv_lens=sl("kv_lens", B),
            q_starts=sl("q_starts", B), logits_idx=sl("logits_idx", L),
            block_tables=sl("block_tables", B * mb).view(B, mb),
            num_seqs=B, num_prefill=layout["num_prefill"], num_decode=layout["num_decode"], total_tokens=T,
            total_logits=L, max_q_len=layout["max_q_len"], max_kv_len=layout["max_kv_len"], max_blocks=mb,
            h2d_bytes=n * 4,
            cu_q_host=hn[layout["cu_q"]:layout["cu_q"] + B + 1].copy(),
            kv_lens_host=hn[layout["kv_lens"]:layout["kv_lens"] + B].copy(),
        )


def make_step_input(input_ids, positions, slot_mapping, cu_q, kv_lens, block_tables, logits_idx=None,
                    num_prefill=None, device="cpu") -> StepInput:
    """Builds a StepInput from plain lists/tensors (tests, offline forward, warm-up)."""
    dev = torch.device(device)

    def t(x):
        return torch.as_tensor(x, dtype=torch.int32).to(dev)

    cu = torch.as_tensor(cu_q, dtype=torch.int32)
    kl = torch.as_tensor(kv_lens, dtype=torch.int32)
    B = kl.numel()
    qlens = (cu[1:] - cu[:-1])
    if logits_idx is None:
        logits_idx = (cu[1:] - 1)
    bt = torch.as_tensor(block_tables, dtype=torch.int32)
    if num_prefill is None:
        num_prefill = int(((qlens > 1) | ((kl - qlens) == 0)).sum())
    T = int(cu[-1])
    seq_of_token = torch.repeat_interleave(torch.arange(B, dtype=torch.int32), qlens.long())
    return StepInput(
        input_ids=t(input_ids), positions=t(positions), slot_mapping=t(slot_mapping), seq_of_token=seq_of_token.to(dev),
        cu_q=cu.to(dev), kv_lens=kl.to(dev), q_starts=(kl - qlens).to(dev), logits_idx=t(logits_idx),
        block_tables=bt.to(dev).contiguous(), num_seqs=B, num_prefill=num_prefill, num_decode=B - num_prefill,
        total_tokens=T, total_logits=int(torch.as_tensor(logits_idx).numel()), max_q_len=int(qlens.max()) if B else 0,
        max_kv_len=int(kl.max()) if B else 0, max_blocks=bt.shape[1] if bt.dim() == 2 else 0,
        cu_q_host=cu.numpy().copy(), kv_lens_host=kl.numpy().copy())
