"""Native scheduler + KV manager driven by a fake model whose "KV cache" stores token ids: the next token is a
hash of everything the sequence can read through its block table, so any mistake in block tables, prefix reuse,
swap copies, fork copies, chunked prefill or draft verification changes the generated tokens."""
import numpy as np
import pytest

from ksanallm_b200 import host


def _next_token(history):
    h = 1469598103934665603
    for t in history:
        h = ((h ^ (int(t) + 1)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return int(h % 29989) + 3


def expected_output(prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(_next_token(toks))
    return toks[len(prompt):]


class FakeRunner:
    def __init__(self, num_blocks, num_host_blocks, block_size):
        self.bs = block_size
        self.dev = np.full((num_blocks, block_size), -1, dtype=np.int64)
        self.host = np.full((max(num_host_blocks, 1), block_size), -1, dtype=np.int64)

    def run(self, sched, plan, wrong_drafts=False):
        for s, d in plan.swap_out:
            self.host[d] = self.dev[s]
            self.dev[s] = -7  # poison: a stale read would change the hash
        for s, d in plan.swap_in:
            self.dev[d] = self.host[s]
        for s, d in plan.block_copies:
            self.dev[d] = self.dev[s]
        buf = np.zeros(sched.packed_words(plan, 64) + 64, dtype=np.int32)
        lay = sched.pack(plan, buf, 64)
        T, B, mb = lay["total_tokens"], lay["num_seqs"], lay["max_blocks"]
        ids = buf[lay["input_ids"]:lay["input_ids"] + T]
        slots = buf[lay["slot_mapping"]:lay["slot_mapping"] + T]
        cu = buf[lay["cu_q"]:lay["cu_q"] + B + 1]
        kvl = buf[lay["kv_lens"]:lay["kv_lens"] + B]
        bt = buf[lay["block_tables"]:lay["block_tables"] + B * mb].reshape(B, mb)
        lg = buf[lay["logits_idx"]:lay["logits_idx"] + lay["total_logits"]]
        for t in range(T):
            self.dev[slots[t] // self.bs, slots[t] % self.bs] = ids[t]
        sampled = []
        for row in lg:
            b = int(np.searchsorted(cu, row, side="right") - 1)
            ctx_len = kvl[b] - (cu[b + 1] - 1 - row)  # tokens visible to this row
            hist = [self.dev[bt[b, p // self.bs], p % self.bs] for p in range(ctx_len)]
            assert all(h >= 0 for h in hist), "read of an unwritten / poisoned KV slot"
            sampled.append(_next_token(hist))
        return sampled


def make(num_blocks=64, host_blocks=0, prefix=False, **kw):
    cfg = host.SchedulerConfig()
    cfg.block_size = 4
    cfg.max_batch_size = kw.get("max_batch", 8)
    cfg.max_step_tokens = kw.get("max_step_tokens", 64)
    cfg.max_token_len = kw.get("max_token_len", 256)
    cfg.split_fuse_token_num = kw.get("split_fuse", 0)
    cfg.preempt_mode = kw.get("preempt_mode", 1)
    cfg.max_draft_tokens = kw.get("drafts", 0)
    cfg.waiting_timeout_ms = kw.get("timeout_ms", 3600000)
    cfg.max_waiting_queue_len = kw.get("queue", 100)
    cfg.pp_wb_strategy = kw.get("pp_wb", 0)
    cache = host.KVCacheManager(num_blocks, host_blocks, 4, prefix)
    return host.Scheduler(cfg, cache), cache, FakeRunner(num_blocks, host_blocks, 4)


def drive(sched, runner, outputs, max_steps=2000, on_step=None):
    steps = 0
    while sched.has_unfinished():
        plan = sched.schedule(steps)
        assert not plan.empty() or sched.has_unfinished()
        if plan.empty():
            steps += 1
            assert steps < max_steps
            continue
        sampled = runner.run(sched, plan)
        for r in sched.update(plan, sampled, steps):
            outputs.setdefault(r.seq_id, []).extend(r.new_tokens)
        if on_step:
            on_step(steps, plan)
        steps += 1
        assert steps < max_steps
    return steps


def test_continuous_batching_outputs_are_exact():
    sched, cache, runner = make()
    rng = np.random.default_rng(0)
    prompts = {i: rng.integers(3, 1000, rng.integers(1, 30)).tolist() for i in range(1, 13)}
    for i, p in prompts.items():
        assert sched.enqueue(i, p, 5 + i) == host.RET_SUCCESS
    out = {}
    drive(sched, runner, out)
    for i, p in prompts.items():
        assert out[i] == expected_output(p, 5 + i)
    assert cache.num_free_blocks == 64


def test_prefix_cache_reuses_blocks_and_stays_correct():
    sched, cache, runner = make(prefix=True)
    shared = list(range(100, 117))  # 4 full blocks + 1 token
    out = {}
    sched.enqueue(1, shared + [7, 8], 6)
    drive(sched, runner, out)
    hit0 = cache.stats.prefix_hit_tokens
    sched.enqueue(2, shared + [9], 6)
    sched.enqueue(3, shared + [7, 8], 6)
    drive(sched, runner, out)
    assert cache.stats.prefix_hit_tokens - hit0 >= 2 * 16
    assert out[2] == expected_output(shared + [9], 6)
    assert out[3] == expected_output(shared + [7, 8], 6) == out[1]
    assert cache.num_cached_blocks > 0
    n = cache.num_cached_blocks
    assert cache.clear_unreferenced() == n and cache.num_cached_blocks == 0


def test_recompute_preemption_under_memory_pressure():
    sched, cache, runner = make(num_blocks=14, preempt_mode=1)
    prompts = {i: list(range(10 * i, 10 * i + 9)) for i in range(1, 6)}
    for i, p in prompts.items():
        sched.enqueue(i, p, 20)
    out = {}
    drive(sched, runner, out)
    assert sched.stats.preempt_recompute > 0
    for i, p in prompts.items():
        assert out[i] == expected_output(p, 20)


def test_swap_preemption_round_trip():
    sched, cache, runner = make(num_blocks=14, host_blocks=32, preempt_mode=0)
    prompts = {i: list(range(10 * i, 10 * i + 9)) for i in range(1, 6)}
    for i, p in prompts.items():
        sched.enqueue(i, p, 20)
    out = {}
    drive(sched, runner, out)
    assert sched.stats.preempt_swap > 0 and sched.stats.swap_in > 0
    assert cache.stats.swapped_out_blocks == cache.stats.swapped_in_blocks > 0
    for i, p in prompts.items():
        assert out[i] == expected_output(p, 20)
    assert cache.num_free_host_blocks == 32


def test_chunked_prefill_split_fuse():
    sched, cache, runner = make(split_fuse=8, prefix=True)
    p = list(range(50, 50 + 37))
    sched.enqueue(1, p, 4)
    sched.enqueue(2, [5, 6, 7], 10)
    out, chunks = {}, []
    drive(sched, runner, out, on_step=lambda s, plan: chunks.extend(e.q_len for e in plan.entries if e.seq_id == 1))
    assert chunks[:5] == [8, 8, 8, 8, 5]
    assert out[1] == expected_output(p, 4) and out[2] == expected_output([5, 6, 7], 10)


def test_token_budget_chunks_long_prompt_without_split_fuse():
    sched, cache, runner = make(max_step_tokens=16, num_blocks=64)
    p = list(range(200, 245))
    sched.enqueue(1, p, 3)
    out = {}
    steps = drive(sched, runner, out)
    assert out[1] == expected_output(p, 3) and steps == 5


def test_draft_verification_accepts_only_matching_prefix():
    sched, cache, runner = make(drafts=3)
    p = [11, 12, 13, 14, 15]
    truth = expected_output(p, 12)
    sched.enqueue(1, p, 12)
    out = {}
    step = 0
    while sched.has_unfinished():
        plan = sched.schedule(step)
        sampled = runner.run(sched, plan)
        for r in sched.update(plan, sampled, step):
            out.setdefault(r.seq_id, []).extend(r.new_tokens)
            if r.finish_reason == host.FINISH_NONE:
                n = len(out[1])
                good = truth[n:n + 3]
                # alternate: fully right drafts, drafts with a wrong second token
                drafts = good if step % 2 == 0 else [good[0], 1] + good[2:] if len(good) > 1 else good
                sched.set_drafts(1, drafts)
        step += 1
    assert out[1] == truth
    assert sched.stats.draft_accepted > 0 and sched.stats.draft_accepted < sched.stats.draft_proposed
    assert step < 12  # fewer steps than tokens


def test_fork_copy_on_write():
    sched, cache, runner = make()
    p = [21, 22, 23, 24, 25, 26]
    sched.enqueue(1, p, 6)
    out = {}
    plan = sched.schedule(0)
    for r in sched.update(plan, runner.run(sched, plan), 0):
        out.setdefault(r.seq_id, []).extend(r.new_tokens)
    assert sched.fork(1, 2)
    sched.replace_last_token(2, 999)
    out[2] = [999]
    drive(sched, runner, out)
    assert out[1] == expected_output(p, 6)
    assert out[2][1:] == expected_output(p + [999], 5)


def test_finish_rules_abort_timeout_and_capacity():
    sched, cache, runner = make(queue=2, timeout_ms=5, max_token_len=32)
    assert sched.enqueue(1, list(range(40)), 4) == host.RET_INPUT_LENGTH_EXCEEDED
    eos = _next_token([3, 4, 5])
    assert sched.enqueue(2, [3, 4, 5], 10, False, [eos], []) == host.RET_SUCCESS
    assert sched.enqueue(3, [6, 7], 50) == host.RET_SUCCESS
    assert sched.enqueue(4, [8], 5) == host.RET_EXCEED_CAPACITY
    out, reasons = {}, {}
    step = 0
    while sched.has_unfinished():
        plan = sched.schedule(step)
        for sid, why in plan.dropped:
            reasons[sid] = why
        if not plan.empty():
            for r in sched.update(plan, runner.run(sched, plan), step):
                out.setdefault(r.seq_id, []).extend(r.new_tokens)
                if r.finish_reason:
                    reasons[r.seq_id] = r.finish_reason
        if step == 3:
            sched.abort(3)
        step += 1
    assert reasons[2] == host.FINISH_EOS and out[2] == [eos]
    assert reasons[3] == host.FINISH_ABORTED
    # total length cap
    sched.enqueue(5, list(range(3, 30)), 100)
    out = {}
    drive(sched, runner, out)
    assert len(out[5]) == 32 - 27
    # queue timeout
    sched2, _, runner2 = make(timeout_ms=5, max_batch=1)
    sched2.enqueue(1, [3, 4], 30, False, [], [], 0)
    sched2.enqueue(2, [5, 6], 3, False, [], [], 0)
    dropped = []
    for step in range(40):
        plan = sched2.schedule(step)
        dropped += plan.dropped
        if not plan.empty():
            sched2.update(plan, runner2.run(sched2, plan), step)
    assert (2, host.FINISH_TIMEOUT) in dropped


def test_draft_trie_and_balancer():
    t = host.DraftTrie(16)
    seq = [1, 2, 3, 4, 5, 1, 2, 3, 4, 6, 1, 2, 3]
    t.feed(seq)
    assert t.propose(2)[0] == 4
    assert host.balance_workloads([10, 1, 7, 3], [0, 5]) in ([1, 1, 0, 0], [1, 0, 0, 1], [0, 1, 1, 1], [0, 1, 1, 0])
    a = host.balance_workloads([10, 1, 7, 3], [0, 0])
    loads = [sum(w for w, g in zip([10, 1, 7, 3], a) if g == k) for k in (0, 1)]
    assert max(loads) <= 11



def test_warmup_leaves_a_clean_engine():
    import torch

    from ksanallm_b200.config.model_config import model_config_from_dict
    from ksanallm_b200.config.schema import parse_serving_config
    from ksanallm_b200.engine.llm_engine import LLMEngine
    from ksanallm_b200.models.loader import load_model_weights
    from ksanallm_b200.models.transformer import TransformerModel
    cfg = model_config_from_dict(dict(model_type="llama", hidden_size=64, num_hidden_layers=1, num_attention_heads=2,
                                      num_key_value_heads=2, intermediate_size=128, vocab_size=200,
                                      torch_dtype="float32"))
    serving = parse_serving_config({"setting": {"batch_scheduler": {
        "max_batch_size": 4, "max_step_tokens": 256, "max_token_len": 256, "enable_auto_prefix_cache": True}}})
    eng = LLMEngine(TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, dtype=torch.float32)), serving,
                    num_blocks=64, num_host_blocks=0)
    n = eng.warmup(max_len=128, step=32)
    assert n >= 3 and not eng.has_unfinished()
    assert eng.stats["generated_tokens"] == 0 and eng.cache.num_cached_blocks == 0
    assert eng.cache.num_free_blocks == eng.num_blocks


@pytest.mark.parametrize("strategy", [1, 2, 4])
def test_pipeline_micro_batch_workload_balancing(strategy):
    """Two micro-batches scheduled alternately: new sequences go to the lighter one (by count, or by the tokens they
    still have to compute), an overloaded micro-batch hands work over, and the outputs stay exact."""
    sched, cache, runner = make(num_blocks=256, max_batch=16, max_step_tokens=256, pp_wb=strategy)
    prompts = {1: list(range(10, 90)), 2: [5, 6, 7], 3: [8, 9, 10], 4: [11, 12], 5: [13, 14, 15], 6: [16, 17],
               7: [18, 19], 8: [20, 21, 22]}
    for sid, p in prompts.items():
        sched.enqueue(sid, p, 6)
    outputs, inflight, steps = {}, [None, None], 0
    assignment = None
    while sched.has_unfinished() or any(x is not None for x in inflight):
        mb = steps % 2
        if inflight[mb] is not None:
            plan, sampled = inflight[mb]
            for r in sched.update(plan, sampled, steps):
                outputs.setdefault(r.seq_id, []).extend(r.new_tokens)
            inflight[mb] = None
        sched.set_micro_batch(mb, 2)
        plan = sched.schedule(steps)
        sched.set_micro_batch(-1)
        if steps == 0:
            assignment = {sid: sched.micro_batch_of(sid) for sid in prompts}
        if not plan.empty():
            inflight[mb] = (plan, runner.run(sched, plan))
        steps += 1
        assert steps < 500
    for sid, p in prompts.items():
        assert outputs[sid] == expected_output(p, 6)
    groups = [sorted(s for s, m in assignment.items() if m == k) for k in (0, 1)]
    if strategy == 4:
        # the 80-token prompt weighs as much as all the short ones together
        assert groups[0] == [1] and len(groups[1]) == 7
    else:
        assert len(groups[0]) == 4 and len(groups[1]) == 4


def test_pipeline_micro_batch_offload_moves_running_work():
    sched, cache, runner = make(num_blocks=256, max_batch=16, max_step_tokens=256, pp_wb=2)
    for sid in range(1, 9):
        sched.enqueue(sid, [sid, sid + 1, sid + 2], 8)
    # every sequence is admitted by micro-batch 0 while it is the only one scheduling (count = 1) ...
    sched.set_micro_batch(0, 1)
    plan = sched.schedule(0)
    outs = {}
    for r in sched.update(plan, runner.run(sched, plan), 0):
        outs.setdefault(r.seq_id, []).extend(r.new_tokens)
    assert all(sched.micro_batch_of(s) == 0 for s in range(1, 9))
    # ... then a second micro-batch appears: scheduling micro-batch 0 hands half of its running work over
    sched.set_micro_batch(0, 2)
    plan = sched.schedule(1)
    moved = [s for s in range(1, 9) if sched.micro_batch_of(s) == 1]
    assert len(moved) == 4 and sched.stats.mb_migrations == 4
    assert sorted(plan.seq_ids) == sorted(s for s in range(1, 9) if s not in moved)


@pytest.mark.parametrize("seed,preempt_mode,host_blocks", [(0, 1, 0), (1, 0, 64), (2, 0, 24), (3, 1, 0)])
def test_randomised_many_clients_stress(seed, preempt_mode, host_blocks):
    """Many clients with shared prefixes arrive over time into a small block pool (pre-emption by recompute or swap,
    prefix reuse, chunked prefill, aborts of random victims): every surviving request's output must be exact and
    all blocks must be back when the queue drains."""
    rng = np.random.default_rng(seed)
    sched, cache, runner = make(num_blocks=48, host_blocks=host_blocks, prefix=True, preempt_mode=preempt_mode,
                                split_fuse=int(rng.choice([0, 8, 16])), max_batch=6, max_step_tokens=48,
                                max_token_len=200)
    stems = [list(rng.integers(3, 500, size=n)) for n in (8, 12, 16)]
    arrivals = {}
    for i in range(1, 41):
        stem = stems[int(rng.integers(0, 3))] if rng.random() < 0.7 else []
        prompt = [int(t) for t in stem] + [int(t) for t in rng.integers(3, 500, size=int(rng.integers(1, 20)))]
        arrivals.setdefault(int(rng.integers(0, 60)), []).append((i, prompt, int(rng.integers(1, 24))))
    prompts, outputs, aborted, steps = {}, {}, set(), 0
    while steps < 4000 and (sched.has_unfinished() or any(s >= steps for s in arrivals)):
        for sid, p, n in arrivals.get(steps, []):
            assert sched.enqueue(sid, p, n) == host.RET_SUCCESS
            prompts[sid] = (p, n)
        if steps % 7 == 3 and prompts:
            victim = int(rng.choice(sorted(prompts)))
            if victim not in aborted and len(outputs.get(victim, [])) < prompts[victim][1]:
                sched.abort(victim)
                aborted.add(victim)
        plan = sched.schedule(steps)
        if not plan.empty():
            sampled = runner.run(sched, plan)
            for r in sched.update(plan, sampled, steps):
                outputs.setdefault(r.seq_id, []).extend(r.new_tokens)
        steps += 1
    assert not sched.has_unfinished()
    checked = 0
    for sid, (p, n) in prompts.items():
        want = expected_output(p, n)
        got = outputs.get(sid, [])
        if sid in aborted:
            assert got == want[:len(got)]  # whatever was produced before the abort is still exact
        else:
            assert got == want
            checked += 1
    assert checked >= 20
    cache.clear_unreferenced()
    assert cache.num_free_blocks == 48 and cache.num_free_host_blocks == host_blocks


@pytest.mark.parametrize("preempt_mode,host_blocks", [(1, 0), (0, 16)])
def test_sequence_that_outgrows_the_whole_pool_ends_with_length(preempt_mode, host_blocks):
    """A prompt that fits but whose prompt + generated tokens exceed every block of the pool must finish (reason
    LENGTH) with the tokens it produced, instead of pre-empting itself on every step."""
    sched, cache, runner = make(num_blocks=4, host_blocks=host_blocks, preempt_mode=preempt_mode, max_token_len=4096)
    prompt = list(range(50, 60))  # 10 tokens, blocks of 4 -> the pool holds 16 tokens
    assert sched.enqueue(1, prompt, 200) == host.RET_SUCCESS
    out, dropped = {}, []
    steps = 0
    while sched.has_unfinished():
        plan = sched.schedule(steps)
        dropped += [(sid, reason) for sid, reason in plan.dropped]
        if not plan.empty():
            for r in sched.update(plan, runner.run(sched, plan), steps):
                out.setdefault(r.seq_id, []).extend(r.new_tokens)
        steps += 1
        assert steps < 100, "the sequence neither advances nor ends"
    assert dropped == [(1, host.FINISH_LENGTH)]
    n = len(out[1])
    assert 4 <= n <= 7 and out[1] == expected_output(prompt, n)
    assert cache.num_free_blocks == 4
    # the pool is usable again
    assert sched.enqueue(2, [5, 6, 7], 3) == host.RET_SUCCESS
    drive(sched, runner, out)
    assert out[2] == expected_output([5, 6, 7], 3)
