"""Beam search on top of the continuous-batching scheduler.

Every live beam is an ordinary sequence of the scheduler. After each step the top ``2 * num_beams`` log-probs of
every beam row are combined with the beams' running scores, the best ``num_beams`` continuations survive:
the first continuation of a parent rewrites the parent's last token in place, further ones fork the parent
(copy-on-write of its private KV blocks), parents without a surviving continuation are retired. Continuations
ending in EOS become finished hypotheses scored ``sum_logprob / len ** length_penalty``.
The reference only sizes an output group and sorts it at the end (src/ksana_llm/utils/request.cpp:45-48,
runtime/infer_request.cpp:89-97, 228-233); there is no per-step expansion or pruning to mirror.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class Hypothesis:
    tokens: List[int]
    score: float
    logprobs: List[Any] = field(default_factory=list)


class BeamState:
    def __init__(self, num_beams: int, num_return: int, length_penalty: float, max_new_tokens: int):
        self.k = num_beams
        self.n_ret = max(1, min(num_return, num_beams))
        self.lp = length_penalty
        self.max_new = max_new_tokens
        self.scores: Dict[int, float] = {}  # seq_id -> cumulative log-prob of live beams
        self.finished: List[Hypothesis] = []
        self.done = False
        self.pending: Dict[int, Tuple[List[int], List[Tuple[int, float]]]] = {}  # beams waiting for their siblings

    def _norm(self, s: float, n: int) -> float:
        return s / (max(n, 1) ** self.lp)

    def required_logprobs(self) -> int:
        return 2 * self.k

    def step(self, engine, req, rows: Dict[int, Tuple[List[int], List[Tuple[int, float]]]], eos_ids) -> None:
        """rows: seq_id -> (output tokens BEFORE this step's token, top-n (token, logprob) of this step's row).

        The beams of a request are ranked against each other, so a position is expanded only once EVERY live beam has
        its candidates: under a batch cap or after a pre-emption some beams run a step later than others. A beam
        that is ahead is paused in the scheduler (it keeps its cache) until the others have caught up."""
        self.pending.update(rows)
        live = set(self.scores) if self.scores else set(self.pending)
        if not live <= set(self.pending):
            for sid in rows:
                engine.sched.set_paused(sid, True)
            return
        rows, self.pending = self.pending, {}
        for sid in rows:
            engine.sched.set_paused(sid, False)
        cands: List[Tuple[float, int, int, float]] = []  # (new cumulative score, parent seq, token, token logprob)
        for sid, (_prev, top) in rows.items():
            base = self.scores.get(sid, 0.0)
            for tok, lp in top[: 2 * self.k]:
                cands.append((base + lp, sid, tok, lp))
        cands.sort(key=lambda c: -c[0])
        keep: List[Tuple[float, int, int, float]] = []
        for c in cands:
            score, sid, tok, _ = c
            prev = rows[sid][0]
            if tok in eos_ids and not req.params.ignore_eos:
                self.finished.append(Hypothesis(prev + [tok], self._norm(score, len(prev) + 1)))
                continue
            keep.append(c)
            if len(keep) == self.k:
                break
        n_after = (len(next(iter(rows.values()))[0]) + 1) if rows else 0
        out_of_budget = n_after >= self.max_new
        best_live = keep[0][0] if keep else float("-inf")
        enough = len(self.finished) >= self.k and \
            sorted(h.score for h in self.finished)[-self.k] >= self._norm(best_live, n_after)
        if out_of_budget or enough or not keep:
            for score, sid, tok, _ in keep:
                self.finished.append(Hypothesis(rows[sid][0] + [tok], self._norm(score, len(rows[sid][0]) + 1)))
            for sid in rows:
                engine.sched.finish(sid, 3)
                engine._finish_seq(sid, 3, notify=False)
            self.done = True
            return
        used: Dict[int, int] = {}
        new_scores: Dict[int, float] = {}
        for score, sid, tok, _ in keep:
            if sid not in used:
                used[sid] = 1
                engine.sched.replace_last_token(sid, tok)
                owner = engine.seq_owner[sid][1]
                owner.output_tokens[-1] = tok
                new_scores[sid] = score
            else:
                child = engine._fork_seq(req, sid)
                if child is None:
                    continue
                engine.sched.replace_last_token(child.seq_id, tok)
                child.output_tokens[-1] = tok
                new_scores[child.seq_id] = score
        for sid in rows:
            if sid not in used:
                engine.sched.finish(sid, 3)
                engine._finish_seq(sid, 3, notify=False)
                # a retired beam is not an output of the request
                req.seqs = [s for s in req.seqs if s.seq_id != sid]
        self.scores = new_scores

    def best(self, req):
        """Final outputs: best ``n_ret`` hypotheses as lightweight sequence records."""
        from .llm_engine import SequenceOutput
        hyps = sorted(self.finished, key=lambda h: -h.score)[: self.n_ret]
        outs = []
        for i, h in enumerate(hyps):
            s = SequenceOutput(seq_id=-(i + 1), output_tokens=list(h.tokens), finished=True, finish_reason="stop")
            s.cum_logprob = h.score
            outs.append(s)
        return outs
