"""Batched device-side sampler.

One pass over ``[rows, vocab]`` logits for the whole step: repetition penalty, n-gram bans, grammar
bitmask, temperature, top-k / top-p (top-p inside the top-k set) and the multinomial draw all run on the
device with per-row parameter vectors; only token ids (not vocab-sized vectors) travel host-to-device.
The reference runs these as per-request host loops on rank 0 (src/ksana_llm/samplers/sampler.cpp:90-217,
371-434, 443-513) around the TRT-LLM two-stage top-k kernel.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..ops import reference as ref
from .sampling_params import SamplingParams


@dataclass
class SampleRow:
    """One logits row: which request it belongs to and the token history that conditions it."""
    params: SamplingParams
    prompt_tokens: Sequence[int]
    output_tokens: Sequence[int]
    bitmask: Optional[np.ndarray] = None  # int32 [ceil(V/32)], grammar-allowed tokens
    generator: Optional[torch.Generator] = None


@dataclass
class SampleOutput:
    tokens: List[int]
    logprobs: List[Optional[List[Tuple[int, float]]]] = field(default_factory=list)  # per row: top-n (id, logprob)
    chosen_logprob: List[Optional[float]] = field(default_factory=list)


def _ngram_bans(tokens: Sequence[int], n: int) -> List[int]:
    """Tokens that would complete an n-gram already present in ``tokens``."""
    if n <= 0 or len(tokens) < n:
        return []
    prefix = tuple(tokens[len(tokens) - n + 1:]) if n > 1 else tuple()
    banned = []
    for i in range(len(tokens) - n + 1):
        if tuple(tokens[i:i + n - 1]) == prefix:
            banned.append(tokens[i + n - 1])
    return banned


class Sampler:
    def __init__(self, vocab_size: int, device: torch.device, seed: int = 0):
        self.vocab_size = vocab_size
        self.device = torch.device(device)
        self.gen = torch.Generator(device=self.device)
        self.gen.manual_seed(seed)
        self.eos_token_ids: List[int] = []  # set by the engine (model EOS ids, for min_tokens)

    @staticmethod
    def all_greedy(rows: Sequence[SampleRow]) -> bool:
        return all(r.params.use_greedy and not r.params.needs_logits_processing and r.params.logprobs == 0
                   and r.bitmask is None for r in rows)

    def _process_device(self, logits: torch.Tensor, rows: Sequence[SampleRow]) -> torch.Tensor:
        """The whole step's logit processing as ONE kernel (csrc/cuda/sampling.cu logits_process_kernel): the host
        only concatenates the token histories and the few (row, token) edits; nothing vocab-sized leaves the device."""
        from ..ops import cuda as kcuda
        L, V = logits.shape
        x = logits.float()
        if x.data_ptr() == logits.data_ptr() or x.stride(1) != 1:
            x = x.clone(memory_format=torch.contiguous_format)
        hist, row_off, plen = [], [0], []
        fpar = np.zeros((L, 3), dtype=np.float32)
        ipar = np.zeros((L, 4), dtype=np.int32)
        e_off, e_tok, e_val, b_off, b_tok = [0], [], [], [0], []
        words = (V + 31) // 32
        bm = None
        for i, r in enumerate(rows):
            p = r.params
            need_hist = (p.repetition_penalty != 1.0 or p.presence_penalty or p.frequency_penalty or
                         p.no_repeat_ngram_size > 0 or p.encoder_no_repeat_ngram_size > 0 or
                         p.decoder_no_repeat_ngram_size > 0)
            if need_hist:
                hist.extend(r.prompt_tokens)
                hist.extend(r.output_tokens)
                plen.append(len(r.prompt_tokens))
            else:
                plen.append(0)
            row_off.append(len(hist))
            fpar[i] = (p.repetition_penalty, p.presence_penalty or 0.0, p.frequency_penalty or 0.0)
            ipar[i, :3] = (p.no_repeat_ngram_size, p.encoder_no_repeat_ngram_size, p.decoder_no_repeat_ngram_size)
            if p.logit_bias:
                for t, b in p.logit_bias.items():
                    e_tok.append(int(t))
                    e_val.append(float(b))
            e_off.append(len(e_tok))
            if p.min_tokens > len(r.output_tokens):
                b_tok.extend(int(t) for t in list(p.stop_token_ids) + ([] if p.ignore_eos else list(self.eos_token_ids)))
            b_off.append(len(b_tok))
            if r.bitmask is not None:
                if bm is None:
                    bm = np.full((L, words), -1, dtype=np.int32)
                bm[i, :min(len(r.bitmask), words)] = r.bitmask[:words]
                ipar[i, 3] = 1

        def dev(a, dt):
            return torch.from_numpy(np.ascontiguousarray(a, dtype=dt)).to(self.device, non_blocking=True)

        return kcuda.logits_process(
            x, dev(hist or [0], np.int32), dev(row_off, np.int32), dev(plen, np.int32), dev(fpar, np.float32),
            dev(ipar, np.int32), dev(e_off, np.int32), dev(e_tok or [0], np.int32), dev(e_val or [0.0], np.float32),
            dev(b_off, np.int32), dev(b_tok or [0], np.int32), dev(bm, np.int32) if bm is not None else None)

    def process_logits(self, logits: torch.Tensor, rows: Sequence[SampleRow]) -> torch.Tensor:
        """Applies penalties / bans / grammar masks. Returns fp32 logits (a copy only when needed)."""
        L, V = logits.shape
        if logits.is_cuda and V <= 200 * 1024 * 8:
            if not any(r.params.needs_logits_processing or r.bitmask is not None or r.params.min_tokens > 0
                       for r in rows):
                return logits.float()
            return self._process_device(logits, rows)
        x = logits.float()
        need_pen = [i for i, r in enumerate(rows) if r.params.repetition_penalty != 1.0]
        if need_pen:
            maxlen = max(len(rows[i].prompt_tokens) + len(rows[i].output_tokens) for i in need_pen)
            ids = np.full((len(need_pen), max(maxlen, 1)), -1, dtype=np.int64)
            for j, i in enumerate(need_pen):
                t = list(rows[i].prompt_tokens) + list(rows[i].output_tokens)
                ids[j, :len(t)] = t
            ids_d = torch.from_numpy(ids).to(self.device, non_blocking=True)
            seen = torch.zeros(len(need_pen), V + 1, dtype=torch.bool, device=self.device)
            seen.scatter_(1, torch.where(ids_d < 0, V, ids_d), True)
            seen = seen[:, :V]
            pen = torch.tensor([rows[i].params.repetition_penalty for i in need_pen], dtype=torch.float32,
                               device=self.device).unsqueeze(1)
            sel = torch.tensor(need_pen, device=self.device)
            sub = x.index_select(0, sel)
            sub = torch.where(seen, torch.where(sub > 0, sub / pen, sub * pen), sub)
            x = x.index_copy(0, sel, sub)
        add_r, add_t, add_v = [], [], []
        for i, r in enumerate(rows):
            p = r.params
            if p.presence_penalty or p.frequency_penalty:
                counts: Dict[int, int] = {}
                for t in r.output_tokens:
                    counts[int(t)] = counts.get(int(t), 0) + 1
                for t, c in counts.items():
                    if 0 <= t < V:
                        add_r.append(i)
                        add_t.append(t)
                        add_v.append(-(p.presence_penalty + p.frequency_penalty * c))
            if p.logit_bias:
                for t, b in p.logit_bias.items():
                    if 0 <= int(t) < V:
                        add_r.append(i)
                        add_t.append(int(t))
                        add_v.append(float(b))
        if add_r:
            if x.data_ptr() == logits.data_ptr():
                x = x.clone()
            x.index_put_((torch.tensor(add_r, device=self.device), torch.tensor(add_t, device=self.device)),
                         torch.tensor(add_v, dtype=torch.float32, device=self.device), accumulate=True)
        ban_r, ban_t = [], []
        for i, r in enumerate(rows):
            p = r.params
            if p.min_tokens > len(r.output_tokens):
                for t in list(p.stop_token_ids) + ([] if p.ignore_eos else list(self.eos_token_ids)):
                    if 0 <= int(t) < V:
                        ban_r.append(i)
                        ban_t.append(int(t))
            hist = list(r.prompt_tokens) + list(r.output_tokens)
            for n, src in ((p.no_repeat_ngram_size, hist), (p.encoder_no_repeat_ngram_size, None),
                           (p.decoder_no_repeat_ngram_size, list(r.output_tokens))):
                if n <= 0:
                    continue
                if src is None:
                    # ban tokens that would continue the generated suffix into an n-gram of the PROMPT
                    out = list(r.output_tokens)
                    pre = tuple(out[len(out) - n + 1:]) if n > 1 else tuple()
                    if len(pre) == n - 1:
                        pt = list(r.prompt_tokens)
                        for s in range(len(pt) - n + 1):
                            if tuple(pt[s:s + n - 1]) == pre:
                                ban_r.append(i)
                                ban_t.append(pt[s + n - 1])
                    continue
                for t in _ngram_bans(src, n):
                    ban_r.append(i)
                    ban_t.append(t)
        if ban_r:
            if x.data_ptr() == logits.data_ptr():
                x = x.clone()
            x[torch.tensor(ban_r, device=self.device), torch.tensor(ban_t, device=self.device)] = float("-inf")
        mask_rows = [i for i, r in enumerate(rows) if r.bitmask is not None]
        if mask_rows:
            words = (V + 31) // 32
            bm = np.full((L, words), -1, dtype=np.int32)
            for i in mask_rows:
                bm[i, :len(rows[i].bitmask)] = rows[i].bitmask[:words]
            x = ref.apply_penalties(x, None, None, torch.from_numpy(bm).to(self.device))
        return x

    def sample(self, logits: torch.Tensor, rows: Sequence[SampleRow]) -> SampleOutput:
        L, V = logits.shape
        x = self.process_logits(logits, rows)
        greedy = [r.params.use_greedy for r in rows]
        if all(greedy):
            toks = ops.argmax(x)
        else:
            temp = torch.tensor([1.0 if g else max(r.params.temperature, 1e-6) for r, g in zip(rows, greedy)],
                                dtype=torch.float32, device=self.device)
            topk = torch.tensor([1 if g else r.params.topk for r, g in zip(rows, greedy)], dtype=torch.int32,
                                device=self.device)
            topp = torch.tensor([1.0 if g else r.params.topp for r, g in zip(rows, greedy)], dtype=torch.float32,
                                device=self.device)
            u = torch.rand(L, generator=self.gen, device=self.device, dtype=torch.float32)
            for i, r in enumerate(rows):
                if r.generator is not None:
                    u[i] = torch.rand(1, generator=r.generator, device=r.generator.device).item()
            toks = ops.sample(x, temp, topk, topp, u)
        out = SampleOutput(tokens=toks.tolist())
        n_lp = max((r.params.logprobs for r in rows), default=0)
        if n_lp > 0:
            lp = torch.log_softmax(x, dim=-1)
            v, idx = lp.topk(n_lp, dim=-1)
            chosen = lp.gather(1, toks.long().unsqueeze(1)).squeeze(1).tolist()
            v, idx = v.tolist(), idx.tolist()
            for i, r in enumerate(rows):
                k = r.params.logprobs
                out.logprobs.append([(idx[i][j], v[i][j]) for j in range(k)] if k else None)
                out.chosen_logprob.append(chosen[i] if k else None)
        else:
            out.logprobs = [None] * L
            out.chosen_logprob = [None] * L
        return out
