"""Executes one scheduled step on this rank's device.

Owns the model, the per-layer KV block pools, the host swap pool and the step staging buffer. The
reference splits this between LlmRuntime::Step / Worker threads / CommonModel::Forward / LmHead
(src/ksana_llm/runtime/llm_runtime.cpp:76-145, 290-338; models/common/common_model.cpp:424-639); with
one process per GPU it collapses into a single object per rank.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..models.transformer import TransformerModel
from .sampler import SampleOutput, SampleRow, Sampler
from .step_input import StepInput, StepStaging


class ModelRunner:
    def __init__(self, model: TransformerModel, num_blocks: int, block_size: int, num_host_blocks: int = 0,
                 max_step_tokens: int = 4096, max_batch_size: int = 128, max_blocks_per_seq: int = 128,
                 kv_dtype: Optional[torch.dtype] = None, seed: int = 0):
        self.model = model
        self.device = model.device
        self.block_size = block_size
        self.num_blocks = num_blocks
        self.kv_caches = model.allocate_kv_cache(num_blocks, block_size, kv_dtype)
        self.host_caches = None
        if num_host_blocks > 0:
            pin = self.device.type == "cuda"
            self.host_caches = [torch.empty((num_host_blocks,) + tuple(c.shape[1:]), dtype=c.dtype, pin_memory=pin)
                                for c in self.kv_caches]
        self.max_blocks_per_seq = max_blocks_per_seq
        words = 8 * (max_step_tokens + 64) + 8 * (max_batch_size + 64) + max_batch_size * (max_blocks_per_seq + 32) + 4096
        self.staging = StepStaging(words, self.device)
        self.sampler = Sampler(model.cfg.vocab_size, self.device, seed)
        self.copy_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.last_hidden: Optional[torch.Tensor] = None
        self.prev_tokens: Optional[torch.Tensor] = None  # device copy of the last step's greedy tokens

    # ---- block movement -------------------------------------------------------------------------------
    def apply_block_ops(self, swap_out: np.ndarray, swap_in: np.ndarray, copies: np.ndarray) -> None:
        """Swap-out (device->host) must land before the step overwrites the freed blocks, swap-in and
        fork copies before attention reads them: all are issued on the compute stream ahead of the forward."""
        if self.device.type == "cuda" and self._mover_ok():
            # one kernel per kind of move, every layer at once, straight between the device cache and the pinned host
            # pool: nothing blocks the host and no staging copy is made
            from ..ops import cuda as kcuda
            for pairs, src, dst in ((swap_out, self._dev_ptrs, self._host_ptrs), (swap_in, self._host_ptrs, self._dev_ptrs),
                                    (copies, self._dev_ptrs, self._dev_ptrs)):
                if len(pairs):
                    pr = torch.from_numpy(np.ascontiguousarray(pairs[:, :2], dtype=np.int32)).to(self.device,
                                                                                                 non_blocking=True)
                    kcuda.block_copy(src, dst, pr, self._block_bytes)
            return
        if len(swap_out):
            src = torch.from_numpy(np.ascontiguousarray(swap_out[:, 0])).long()
            dst = torch.from_numpy(np.ascontiguousarray(swap_out[:, 1])).long()
            for dev, host in zip(self.kv_caches, self.host_caches):
                host[dst] = dev[src.to(self.device)].to("cpu")
        if len(swap_in):
            src = torch.from_numpy(np.ascontiguousarray(swap_in[:, 0])).long()
            dst = torch.from_numpy(np.ascontiguousarray(swap_in[:, 1])).long().to(self.device)
            for dev, host in zip(self.kv_caches, self.host_caches):
                dev[dst] = host[src].to(self.device, non_blocking=True)
        if len(copies):
            src = torch.from_numpy(np.ascontiguousarray(copies[:, 0])).long().to(self.device)
            dst = torch.from_numpy(np.ascontiguousarray(copies[:, 1])).long().to(self.device)
            for dev in self.kv_caches:
                dev[dst] = dev[src]

    def _mover_ok(self) -> bool:
        """Prepares (once) the per-layer base-address tables of the device cache and the pinned host pool."""
        ok = getattr(self, "_mover", None)
        if ok is None:
            c0 = self.kv_caches[0]
            self._block_bytes = c0[0].numel() * c0.element_size()
            ok = self._block_bytes % 16 == 0 and all(c.is_contiguous() for c in self.kv_caches)
            if ok:
                self._dev_ptrs = torch.tensor([c.data_ptr() for c in self.kv_caches], dtype=torch.int64,
                                              device=self.device)
                self._host_ptrs = None
                if self.host_caches is not None:
                    ok = all(h.is_pinned() and h.is_contiguous() for h in self.host_caches)
                    if ok:
                        self._host_ptrs = torch.tensor([h.data_ptr() for h in self.host_caches], dtype=torch.int64,
                                                       device=self.device)
            self._mover = ok
        return ok

    def apply_flexible(self, rows: np.ndarray) -> None:
        """Flexible cache reuse: ``rows`` = [n, 4] (source slot, destination slot, source position, destination
        position). Values are copied; keys are moved from the rotary phase of their old position to the new one,
        R(dst) = R(dst - src) R(src), with cos / sin of the difference formed from the two table rows (which also
        cancels a YaRN magnitude factor folded into the table). The reference does this with a reverse-RoPE pass
        over per-token copy tasks (cache_manager/prefix_cache_manager.cpp:366-388, model_input flexible-cache copy
        lists)."""
        if not len(rows):
            return
        cfg, model = self.model.cfg, self.model
        r = torch.from_numpy(np.ascontiguousarray(rows)).long().to(self.device)
        src, dst, sp, dp = r[:, 0], r[:, 1], r[:, 2], r[:, 3]
        bs = self.block_size
        sb, so, db, do = src // bs, src % bs, dst // bs, dst % bs
        table = model.rope_cache
        rd = cfg.qk_rope_head_dim if cfg.use_mla else (cfg.rotary_dim or cfg.head_dim)
        if table is not None:
            half = rd // 2
            cs, cd = table[sp].float(), table[dp].float()
            m2 = (cs[:, :1] ** 2 + cs[:, half:half + 1] ** 2)
            cos = (cd[:, :half] * cs[:, :half] + cd[:, half:] * cs[:, half:]) / m2
            sin = (cd[:, half:] * cs[:, :half] - cd[:, :half] * cs[:, half:]) / m2
        from ..ops import reference as ref
        for cache in self.kv_caches:
            if cfg.use_mla:
                rows_ = cache[sb, so].clone()  # [n, r + dr (+ indexer key)]
                if table is not None:
                    lo = cfg.kv_lora_rank
                    k = rows_[:, lo:lo + rd].float().unsqueeze(1)
                    rows_[:, lo:lo + rd] = ref.apply_rope(k, cos, sin, cfg.rope_interleaved, rd)[:, 0].to(cache.dtype)
                cache[db, do] = rows_
            else:
                k = cache[sb, 0, :, so].float()  # [n, hk, d]
                if table is not None:
                    k = ref.apply_rope(k, cos, sin, cfg.rope_interleaved, rd)
                cache[db, 0, :, do] = k.to(cache.dtype)
                cache[db, 1, :, do] = cache[sb, 1, :, so]

    def check_device_status(self) -> None:
        """Kernels whose bounded waits expire (a peer that stopped answering, a barrier that never completed) do not
        hang: they set a bit in a device status word and return. This reads the word (and clears it); a non-zero
        value means a recent step produced garbage on this GPU, so the caller fails the requests in flight."""
        if self.device.type != "cuda":
            return
        from ..ops import cuda as kc
        code = kc.read_error(clear=True)
        if code:
            raise RuntimeError(f"device status word 0x{code:x}: a kernel gave up waiting (peer or barrier timeout)")

    # ---- forward ---------------------------------------------------------------------------------------
    def upload(self, layout: Dict[str, int]) -> StepInput:
        meta = self.staging.upload(layout)
        self.h2d_bytes += meta.h2d_bytes
        return meta

    @torch.inference_mode()
    def forward(self, meta: StepInput, refit=None) -> torch.Tensor:
        hidden = self.model.forward(meta, self.kv_caches, refit)
        self.last_hidden = hidden
        return hidden

    @torch.inference_mode()
    def mock_forward(self, with_mtp: bool = False) -> None:
        """A step with zero tokens: only the collectives inside the layers matter (expert-parallel exchanges of
        the MoE blocks when other data-parallel ranks have work)."""
        from .step_input import make_step_input
        meta = make_step_input([], [], [], [0], [], torch.zeros(0, 1, dtype=torch.int32), logits_idx=[],
                               num_prefill=0, device=self.device)
        h = self.model.forward(meta, self.kv_caches)
        if with_mtp and self.model.mtp_layers:
            # the draft pass of the working ranks goes through the expert exchange once more: join it
            mtp = self.model.mtp_layers[0]
            mtp.forward(h.new_zeros(0, h.shape[-1]), h, meta, self.kv_caches[len(self.model.layers)])

    @torch.inference_mode()
    def mock_mtp_passes(self, n: int) -> None:
        """``n`` passes of the draft module over zero rows: only its expert exchange matters (see mock_forward)."""
        if not self.model.mtp_layers:
            return
        from .step_input import make_step_input
        meta = make_step_input([], [], [], [0], [], torch.zeros(0, 1, dtype=torch.int32), logits_idx=[],
                               num_prefill=0, device=self.device)
        mtp = self.model.mtp_layers[0]
        H = self.model.cfg.hidden_size
        empty = torch.zeros(0, H, dtype=self.model.dtype, device=self.device)
        for _ in range(n):
            mtp.forward(empty, empty, meta, self.kv_caches[len(self.model.layers)])

    @torch.inference_mode()
    def sample(self, hidden: torch.Tensor, meta: StepInput, rows: Optional[Sequence[SampleRow]],
               greedy: Optional[bool] = None) -> SampleOutput:
        """rows is None on ranks that do not own the sampler: they still join the collectives of the
        path (greedy pair exchange, or full logits gather) chosen by the driving rank via ``greedy``."""
        if meta.total_logits == 0:
            return SampleOutput(tokens=[])
        if greedy is None:
            greedy = rows is None or Sampler.all_greedy(rows)
        if greedy:
            toks = self.model.greedy_tokens(hidden, meta.logits_idx)
            self.prev_tokens = toks
            if rows is None:
                return SampleOutput(tokens=[])
            host = toks.to("cpu", non_blocking=False)
            self.d2h_bytes += host.numel() * host.element_size()
            n = len(rows)
            return SampleOutput(tokens=host.tolist(), logprobs=[None] * n, chosen_logprob=[None] * n)
        logits = self.model.compute_logits(hidden, meta.logits_idx)
        if rows is None:
            return SampleOutput(tokens=[])
        out = self.sampler.sample(logits, rows)
        self.d2h_bytes += 4 * len(out.tokens)
        return out

    # ---- asynchronous scheduling support ------------------------------------------------------------------------
    @torch.inference_mode()
    def fixup_inputs(self, meta: StepInput) -> None:
        """Input ids planned before the previous step's tokens reached the host are placeholders -(1 + row): they
        are replaced on the device by row ``row`` of the previous step's token vector."""
        if self.prev_tokens is None or meta.total_tokens == 0:
            return
        ids = meta.input_ids
        src = (-ids - 1).clamp_(min=0, max=self.prev_tokens.numel() - 1).long()
        ids.copy_(torch.where(ids < 0, self.prev_tokens.to(torch.int32).index_select(0, src), ids))

    @torch.inference_mode()
    def sample_greedy_async(self, hidden: torch.Tensor, meta: StepInput):
        """Greedy tokens stay on the device (for ``fixup_inputs`` of the next step); the host copy is started
        without waiting. Returns a handle for ``wait_tokens`` (None when the step has no logits)."""
        if meta.total_logits == 0:
            return None
        toks = self.model.greedy_tokens(hidden, meta.logits_idx).to(torch.int32)
        self.prev_tokens = toks
        if toks.device.type != "cuda":
            return (toks.clone(), None)
        host = torch.empty(toks.shape, dtype=torch.int32, pin_memory=True)
        host.copy_(toks, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.d2h_bytes += host.numel() * 4
        return (host, ev)

    @staticmethod
    def wait_tokens(handle) -> List[int]:
        if handle is None:
            return []
        host, ev = handle
        if ev is not None:
            ev.synchronize()
        return host.tolist()

    @torch.inference_mode()
    def logits(self, hidden: torch.Tensor, meta: StepInput) -> torch.Tensor:
        return self.model.compute_logits(hidden, meta.logits_idx)
