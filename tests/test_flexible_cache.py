"""Flexible (non-prefix) cache reuse: a prompt whose middle changed length still finds the tokens after the change
in the prefix tree, at other positions; their KV is copied with the keys' rotary phase moved to the new positions.
Keys / values of the first layer depend only on (token, position), so there the copy must equal a fresh computation."""
import torch

from ksanallm_b200 import host as _host
from ksanallm_b200.config.model_config import tiny_llama_config
from ksanallm_b200.config.schema import parse_serving_config
from ksanallm_b200.engine.llm_engine import LLMEngine
from ksanallm_b200.engine.sampling_params import SamplingParams
from ksanallm_b200.models.loader import load_model_weights
from ksanallm_b200.models.transformer import TransformerModel

BS = 16


def test_cache_manager_finds_shifted_runs():
    cm = _host.KVCacheManager(64, 0, BS, True)
    P, Y, X = list(range(100, 132)), list(range(200, 205)), list(range(300, 380))
    a = P + Y + X + [1, 2, 3]
    cm.create_seq(1, a)
    assert cm.ensure_capacity(1, len(a))
    cm.commit_filled(1, a, len(a))
    cm.free_seq(1)
    b = P + X + [7, 8, 9]
    hit = cm.create_seq(2, b)
    assert hit == 32
    run = cm.flexible_reserve(2, b, hit, 32)
    assert run is not None
    dst_begin, src_slots, dst_slots, src_pos = run
    # A's blocks after the prefix: [Y + X[:11]] [X[11:27]] [X[27:43]] [X[43:59]] [X[59:75]]; B continues with X at 32
    assert dst_begin == 32 and src_pos[0] == 32 + 5 and list(src_pos) == list(range(37, 37 + len(src_pos)))
    assert len(src_pos) == 11 + 64  # the parent's tail plus four full blocks, one token at least left to compute
    table = cm.block_table(2)
    assert [s // BS for s in dst_slots] == [table[(32 + i) // BS] for i in range(len(dst_slots))]
    assert cm.flexible_reserve(2, b, hit, 200) is None  # longer than anything cached
    assert cm.stats.flexible_hit_tokens == 75


def _engine(min_flex):
    cfg = tiny_llama_config()
    model = TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, dtype=torch.float32))
    serving = parse_serving_config({"setting": {"batch_scheduler": {
        "max_batch_size": 4, "max_step_tokens": 256, "max_token_len": 512, "enable_auto_prefix_cache": True,
        "min_flexible_cache_num": min_flex}, "block_manager": {"block_token_num": BS}}})
    return LLMEngine(model, serving, num_blocks=64, num_host_blocks=0)


def test_engine_reuses_shifted_context_and_first_layer_kv_is_exact():
    g = torch.Generator().manual_seed(3)
    P = torch.randint(3, 31000, (32,), generator=g).tolist()
    Y = torch.randint(3, 31000, (5,), generator=g).tolist()
    X = torch.randint(3, 31000, (80,), generator=g).tolist()
    a, b = P + Y + X + [11, 12, 13], P + X + [21, 22, 23]
    sp = SamplingParams(topk=1, max_new_tokens=2, ignore_eos=True)
    eng = _engine(32)
    assert eng.sched_cfg.min_flexible_cache_num == 32
    eng.generate([a], sp)
    before = eng.stats["prompt_tokens"], eng.cache.stats.flexible_hit_tokens
    req = eng.add_request(b, sp)
    eng.step()  # the step that admits b: copies + the remaining prompt tokens
    assert eng.cache.stats.flexible_hit_tokens - before[1] == 75
    seq_id = req.seqs[0].seq_id
    table = eng.cache.block_table(seq_id)
    # fresh engine without the feature: same request, same positions
    ref_eng = _engine(0)
    ref_req = ref_eng.add_request(b, sp)
    ref_eng.step()
    ref_table = ref_eng.cache.block_table(ref_req.seqs[0].seq_id)
    n_blk = len(b) // BS
    got0 = eng.runner.kv_caches[0][torch.tensor(table[:n_blk])]
    want0 = ref_eng.runner.kv_caches[0][torch.tensor(ref_table[:n_blk])]
    assert torch.allclose(got0, want0, atol=1e-5)  # first layer: exact up to rounding, keys re-rotated by -5 positions
    got1 = eng.runner.kv_caches[1][torch.tensor(table[:n_blk])]
    want1 = ref_eng.runner.kv_caches[1][torch.tensor(ref_table[:n_blk])]
    assert not torch.allclose(got1[2:], want1[2:], atol=1e-5)  # deeper layers saw a different context: approximate
    eng.run_until_done()
    assert len(req.output_token_ids[0]) == 2


import pytest  # noqa: E402


@pytest.mark.parametrize("seed", list(range(int(__import__("os").environ.get("KSANA_FUZZ_SEEDS", "6")))))
def test_shifted_reuse_under_memory_pressure_keeps_the_pool_consistent(seed):
    """Multi-turn style traffic (a common context with a varying head and tail) against a small block pool with
    non-prefix reuse on: requests are admitted while others are pre-empted and cached blocks are evicted. Reused
    keys are approximations beyond the first layer, so outputs are not compared; every request must finish with
    its full length, the checksum-free accounting must hold (all blocks free or cached at the end), and the copy
    lists must only ever name slots inside the pool (checked by the runner's index_select)."""
    import random
    rnd = random.Random(seed)
    cfg = tiny_llama_config()
    model = TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, dtype=torch.float32))
    host = rnd.choice([0, 24])
    serving = parse_serving_config({"setting": {"batch_scheduler": {
        "max_batch_size": rnd.choice([3, 6]), "max_step_tokens": 128, "max_token_len": 256,
        "enable_auto_prefix_cache": True, "min_flexible_cache_num": rnd.choice([16, 32]),
        "preempt_mode": rnd.choice([0, 1]) if host else 1, "split_fuse_token_num": rnd.choice([0, 32])},
        "block_manager": {"block_token_num": BS}}})
    eng = LLMEngine(model, serving, num_blocks=rnd.randint(18, 30), num_host_blocks=host)
    g = torch.Generator().manual_seed(seed)
    contexts = [torch.randint(3, 31000, (rnd.choice([48, 64, 80]),), generator=g).tolist() for _ in range(2)]
    reqs = []
    for turn in range(14):
        head = torch.randint(3, 31000, (rnd.randint(0, 20),), generator=g).tolist()
        tail = torch.randint(3, 31000, (rnd.randint(1, 12),), generator=g).tolist()
        n = rnd.randint(2, 16)
        reqs.append((n, eng.add_request(head + rnd.choice(contexts) + tail,
                                        SamplingParams(topk=1, max_new_tokens=n, ignore_eos=True))))
        for _ in range(rnd.randint(0, 5)):
            eng.step()
    eng.run_until_done()
    for n, r in reqs:
        assert r.finished and len(r.output_token_ids[0]) == n
    assert eng.cache.num_free_blocks + eng.cache.num_cached_blocks == eng.cache.num_device_blocks
