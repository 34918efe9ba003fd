"""The engine under KV memory pressure on CPU (real model, real cache tensors): swap pre-emption to host blocks,
recompute pre-emption, prefix reuse, chunked prefill and parallel sampling all at once; every request's tokens must
equal those of a run with plenty of memory."""
import pytest
import torch

from ksanallm_b200.config.model_config import tiny_llama_config
from ksanallm_b200.config.schema import parse_serving_config
from ksanallm_b200.engine.llm_engine import LLMEngine
from ksanallm_b200.engine.sampling_params import SamplingParams
from ksanallm_b200.models.loader import load_model_weights
from ksanallm_b200.models.transformer import TransformerModel


def _engine(model, num_blocks, host_blocks, preempt_mode, split_fuse):
    serving = parse_serving_config({"setting": {"batch_scheduler": {
        "max_batch_size": 6, "max_step_tokens": 96, "max_token_len": 256, "enable_auto_prefix_cache": True,
        "preempt_mode": preempt_mode, "split_fuse_token_num": split_fuse}, "block_manager": {"block_token_num": 16}}})
    return LLMEngine(model, serving, num_blocks=num_blocks, num_host_blocks=host_blocks)


@pytest.mark.parametrize("preempt_mode,host_blocks", [(0, 32), (1, 0)])
def test_outputs_survive_preemption(preempt_mode, host_blocks):
    cfg = tiny_llama_config()
    model = TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, dtype=torch.float32))
    g = torch.Generator().manual_seed(5)
    stem = torch.randint(3, 31000, (32,), generator=g).tolist()
    prompts = [stem + torch.randint(3, 31000, (n,), generator=g).tolist() for n in (5, 17, 30, 9, 22, 3)]
    sp = SamplingParams(topk=1, max_new_tokens=40, ignore_eos=True)
    roomy = _engine(model, 128, 0, 1, 0)
    want = [r.output_token_ids[0] for r in roomy.generate(prompts, sp)]
    tight = _engine(model, 20, host_blocks, preempt_mode, 24)  # 20 blocks = 320 tokens for ~6 x 90 tokens of demand
    got = [r.output_token_ids[0] for r in tight.generate(prompts, sp)]
    assert got == want
    st = tight.sched.stats
    assert (st.preempt_swap if preempt_mode == 0 else st.preempt_recompute) > 0
    assert tight.cache.stats.prefix_hit_tokens >= 32
    if preempt_mode == 0:
        assert tight.cache.stats.swapped_out_blocks > 0 and tight.cache.stats.swapped_in_blocks > 0


def test_fp8_kv_cache_with_scales_stays_close_to_the_full_precision_cache():
    """fp8 (e4m3) KV cache with per-layer scaling factors: same engine, 8-bit pages; logits of a long prompt stay
    close to the fp32-cache run and greedy decoding runs to completion."""
    from ksanallm_b200.engine.step_input import make_step_input
    from ksanallm_b200.models.kv_scales import apply_kv_scales
    cfg = tiny_llama_config()
    model = TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, dtype=torch.float32))
    T = 40
    ids = torch.randint(3, 31000, (T,), generator=torch.Generator().manual_seed(2)).tolist()
    meta = make_step_input(ids, list(range(T)), list(range(T)), [0, T], [T], [[0, 1, 2]], device="cpu")
    full = model.compute_logits(model.forward(meta, model.allocate_kv_cache(4, 16)), meta.logits_idx)[0]
    apply_kv_scales(model, [0.05] * cfg.num_layers)
    cache8 = model.allocate_kv_cache(4, 16, torch.float8_e4m3fn)
    assert cache8[0].dtype == torch.float8_e4m3fn
    # prefill in two chunks so that the second one reads 8-bit pages written by the first
    m1 = make_step_input(ids[:24], list(range(24)), list(range(24)), [0, 24], [24], [[0, 1, 2]], device="cpu")
    model.forward(m1, cache8)
    m2 = make_step_input(ids[24:], list(range(24, T)), list(range(24, T)), [0, T - 24], [T], [[0, 1, 2]], device="cpu")
    low = model.compute_logits(model.forward(m2, cache8), m2.logits_idx)[0]
    rel = (low - full).abs().max().item() / full.abs().max().item()
    assert 0 < rel < 0.1
    serving = parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 2, "max_step_tokens": 64,
                                                                     "max_token_len": 128}}})
    eng = LLMEngine(model, serving, num_blocks=16, num_host_blocks=0, kv_dtype=torch.float8_e4m3fn)
    req = eng.generate([ids], SamplingParams(topk=1, max_new_tokens=6, ignore_eos=True))[0]
    assert len(req.output_token_ids[0]) == 6


def test_block_checksum_guard_passes_on_a_clean_run_and_catches_a_stray_write():
    """enable_block_checksum: blocks that were full before a step must leave it unchanged. A clean run (prefix
    reuse + chunked prefill + decode) raises nothing; a forward that scribbles into an old block is caught."""
    cfg = tiny_llama_config()
    model = TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, dtype=torch.float32))
    serving = parse_serving_config({"setting": {"batch_scheduler": {
        "max_batch_size": 4, "max_step_tokens": 64, "max_token_len": 256, "enable_auto_prefix_cache": True,
        "split_fuse_token_num": 16}, "block_manager": {"block_token_num": 16, "enable_block_checksum": True}}})
    eng = LLMEngine(model, serving, num_blocks=32, num_host_blocks=0)
    assert eng._check_blocks
    g = torch.Generator().manual_seed(9)
    stem = torch.randint(3, 31000, (32,), generator=g).tolist()
    sp = SamplingParams(topk=1, max_new_tokens=20, ignore_eos=True)
    eng.generate([stem + [7, 8, 9], stem + [10, 11]], sp)
    # now a "kernel bug": every forward also overwrites slot 0 of block 0 in the first layer
    orig = eng.runner.forward

    def bad_forward(meta, refit=None):
        h = orig(meta, refit)
        eng.runner.kv_caches[0][eng.cache.block_table(req.seqs[0].seq_id)[0]].view(-1)[0] += 1.0
        return h

    eng.runner.forward = bad_forward
    req = eng.add_request(stem + [12, 13, 14], sp)
    with pytest.raises(RuntimeError, match="checksum changed"):
        for _ in range(10):
            eng.step()


@pytest.mark.parametrize("seed", list(range(int(__import__("os").environ.get("KSANA_FUZZ_SEEDS", "10")))))
def test_randomised_configurations_and_arrivals_keep_greedy_outputs(seed):
    """Random block-pool sizes, pre-emption mode, chunk size, trie speculation, asynchronous scheduling and staggered
    arrivals: none of them may change what a greedy request generates."""
    import random
    rnd = random.Random(seed)
    cfg = tiny_llama_config()
    model = TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, dtype=torch.float32))
    g = torch.Generator().manual_seed(100 + seed)
    stem = torch.randint(3, 31000, (rnd.choice([16, 32, 40]),), generator=g).tolist()
    prompts = [(stem if rnd.random() < 0.7 else []) + torch.randint(3, 31000, (rnd.randint(2, 34),), generator=g).tolist()
               for _ in range(8)]
    params = [SamplingParams(topk=1, max_new_tokens=rnd.randint(4, 36), ignore_eos=True) for _ in prompts]
    roomy = _engine(model, 160, 0, 1, 0)
    want = [roomy.generate([p], sp)[0].output_token_ids[0] for p, sp in zip(prompts, params)]
    host_blocks = rnd.choice([0, 24])
    split = rnd.choice([0, 16, 40])
    serving = parse_serving_config({"setting": {"batch_scheduler": {
        "max_batch_size": rnd.choice([3, 6, 8]), "max_step_tokens": 96, "max_token_len": 256,
        "enable_auto_prefix_cache": rnd.random() < 0.8, "preempt_mode": rnd.choice([0, 1]) if host_blocks else 1,
        "split_fuse_token_num": split, "enable_speculative_decoding": rnd.random() < 0.5,
        "enable_async": split == 0 and rnd.random() < 0.6},  # (the two are refused together, as in the reference)
        "block_manager": {"block_token_num": 16}}})
    eng = LLMEngine(model, serving, num_blocks=rnd.randint(14, 26), num_host_blocks=host_blocks)
    reqs = []
    order = list(range(len(prompts)))
    rnd.shuffle(order)
    while order:
        for _ in range(rnd.randint(1, 3)):
            if order:
                i = order.pop()
                reqs.append((i, eng.add_request(prompts[i], params[i])))
        for _ in range(rnd.randint(0, 4)):
            eng.step()
    eng.run_until_done()
    for i, r in reqs:
        assert r.output_token_ids[0] == want[i], (seed, i)
    assert eng.cache.num_free_blocks + eng.cache.num_cached_blocks == eng.cache.num_device_blocks


@pytest.mark.parametrize("seed", list(range(int(__import__("os").environ.get("KSANA_FUZZ_SEEDS", "6")))))
def test_beam_search_and_seeded_parallel_sampling_survive_preemption(seed):
    """Beam search (forks + pruning), seeded sampling with several returned sequences and greedy requests mixed in one
    engine whose block pool forces pre-emption: results equal those of an engine with plenty of blocks."""
    import random
    rnd = random.Random(seed)
    cfg = tiny_llama_config()
    model = TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, dtype=torch.float32))
    g = torch.Generator().manual_seed(300 + seed)
    prompts = [torch.randint(3, 31000, (rnd.randint(3, 40),), generator=g).tolist() for _ in range(6)]

    def params(i):
        kind = i % 3
        n = 6 + (i * 5) % 17
        if kind == 0:
            return SamplingParams(num_beams=2 + i % 2, num_return_sequences=2, max_new_tokens=n, ignore_eos=True)
        if kind == 1:
            return SamplingParams(topk=30, topp=0.9, temperature=0.9, seed=17 + i, num_return_sequences=2,
                                  max_new_tokens=n, ignore_eos=True)
        return SamplingParams(topk=1, max_new_tokens=n, ignore_eos=True)

    def outputs(eng):
        reqs = [eng.add_request(p, params(i)) for i, p in enumerate(prompts)]
        eng.run_until_done()
        res = []
        for r in reqs:
            if r.beam is not None:
                res.append([h.tokens for h in sorted(r.beam.finished, key=lambda h: -h.score)[:2]])
            else:
                res.append(r.output_token_ids)
        return res

    want = outputs(_engine(model, 200, 0, 1, 0))
    host_blocks = rnd.choice([0, 24])
    tight = _engine(model, rnd.randint(16, 24), host_blocks, rnd.choice([0, 1]) if host_blocks else 1,
                    rnd.choice([0, 24]))
    got = outputs(tight)
    assert got == want
    assert tight.cache.num_free_blocks + tight.cache.num_cached_blocks == tight.cache.num_device_blocks


@pytest.mark.parametrize("seed", list(range(int(__import__("os").environ.get("KSANA_FUZZ_SEEDS", "6")))))
def test_spliced_embeddings_with_chunking_preemption_and_prefix_cache(seed):
    """Requests whose prompt embeddings are partly replaced (multimodal splice) share the engine with plain requests
    that hit the prefix cache; chunk boundaries fall inside the spliced spans and pre-emption recomputes them. The
    spliced requests bypass the prefix tree (same token ids, different embeddings) and must still equal a run alone."""
    import random
    rnd = random.Random(seed)
    cfg = tiny_llama_config()
    model = TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, dtype=torch.float32))
    g = torch.Generator().manual_seed(500 + seed)
    stem = torch.randint(3, 31000, (40,), generator=g).tolist()
    items = []
    for i in range(8):
        toks = stem + torch.randint(3, 31000, (rnd.randint(2, 30),), generator=g).tolist()
        refit = None
        if i % 2 == 0:  # the SAME token ids as other requests, but some embeddings replaced
            refit = []
            pos = rnd.randint(0, 10)
            while pos < len(toks) - 2 and len(refit) < 3:
                n = rnd.randint(1, min(12, len(toks) - 1 - pos))
                refit.append((pos, torch.randn(n, cfg.hidden_size, generator=g) * 0.02))
                pos += n + rnd.randint(1, 9)
        items.append((toks, refit, SamplingParams(topk=1, max_new_tokens=rnd.randint(3, 24), ignore_eos=True)))
    roomy = _engine(model, 200, 0, 1, 0)
    want = []
    for toks, refit, sp in items:
        r = roomy.add_request(toks, sp, refit=refit)
        roomy.run_until_done()
        want.append(r.output_token_ids[0])
    host_blocks = rnd.choice([0, 24])
    tight = _engine(model, rnd.randint(16, 26), host_blocks, rnd.choice([0, 1]) if host_blocks else 1,
                    rnd.choice([0, 16, 24]))
    reqs, order = {}, list(range(len(items)))
    rnd.shuffle(order)
    while order:
        for _ in range(rnd.randint(1, 3)):
            if order:
                i = order.pop()
                reqs[i] = tight.add_request(items[i][0], items[i][2], refit=items[i][1])
        for _ in range(rnd.randint(0, 4)):
            tight.step()
    tight.run_until_done()
    for i in range(len(items)):
        assert reqs[i].output_token_ids[0] == want[i], (seed, i)
    assert tight.cache.num_free_blocks + tight.cache.num_cached_blocks == tight.cache.num_device_blocks
