"""Asynchronous scheduling: steps are planned on placeholder tokens and resolved one step late; the output must be
identical to synchronous scheduling, including EOS / stop-token endings discovered late and length limits."""
import torch

from ksanallm_b200 import host as _host
from ksanallm_b200.config.model_config import model_config_from_dict
from ksanallm_b200.config.schema import parse_serving_config
from ksanallm_b200.engine.llm_engine import LLMEngine
from ksanallm_b200.engine.sampling_params import SamplingParams
from ksanallm_b200.models.loader import load_model_weights
from ksanallm_b200.models.transformer import TransformerModel


def _engine(enable_async, **sched):
    cfg = model_config_from_dict(dict(model_type="llama", hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                                      num_key_value_heads=2, intermediate_size=256, vocab_size=500,
                                      torch_dtype="float32", eos_token_id=2))
    bs = {"max_batch_size": 4, "max_step_tokens": 64, "max_token_len": 128, "enable_async": enable_async}
    bs.update(sched)
    serving = parse_serving_config({"setting": {"batch_scheduler": bs}})
    w = load_model_weights(cfg, synthetic_seed=1, dtype=torch.float32)
    return LLMEngine(TransformerModel(cfg, w), serving, num_blocks=64, num_host_blocks=0)


PROMPTS = [[5, 9, 77, 120, 33, 4, 8], [400, 3, 3, 19, 250, 7, 7, 7, 91, 12, 13], [8, 6, 4], [77] * 20,
           [11, 12, 13, 14, 15], [301, 302]]


def _run(enable_async, params):
    eng = _engine(enable_async)
    reqs = eng.generate(PROMPTS, params)
    assert not eng.has_unfinished()
    return [(r.output_token_ids[0], r.seqs[0].finish_reason) for r in reqs], eng


def test_async_equals_sync_with_length_limit():
    p = SamplingParams(topk=1, max_new_tokens=9, ignore_eos=True)
    sync, _ = _run(False, p)
    asyn, eng = _run(True, p)
    assert eng.async_mode and sync == asyn
    assert all(len(t) == 9 and why == "length" for t, why in asyn)


def test_async_finds_stop_tokens_one_step_late():
    # pick, per prompt, a token the model really produces as a stop token so that sequences end early
    base, _ = _run(False, SamplingParams(topk=1, max_new_tokens=12, ignore_eos=True))
    stops = sorted({toks[3] for toks, _ in base} | {toks[6] for toks, _ in base})
    p = SamplingParams(topk=1, max_new_tokens=12, ignore_eos=True, stop_token_ids=stops)
    sync, _ = _run(False, p)
    asyn, eng = _run(True, p)
    assert sync == asyn
    assert any(why != "length" for _, why in asyn)
    # every block went back to the pool (late finishes release their blocks as well)
    assert eng.cache.num_free_blocks + eng.cache.num_cached_blocks == 64


def test_complex_requests_fall_back_to_synchronous_steps():
    eng = _engine(True)
    p = SamplingParams(topk=1, max_new_tokens=5, ignore_eos=True, repetition_penalty=1.3)
    a = eng.generate(PROMPTS[:2], p)
    ref = _engine(False).generate(PROMPTS[:2], p)
    assert [r.output_token_ids for r in a] == [r.output_token_ids for r in ref]
    assert eng._complex_requests == 0


def test_resolve_patches_placeholders():
    cache = _host.KVCacheManager(16, 0, 16, False)
    sc = _host.SchedulerConfig()
    sc.block_size, sc.max_batch_size, sc.max_step_tokens, sc.max_token_len = 16, 4, 64, 64
    s = _host.Scheduler(sc, cache)
    assert s.enqueue(1, [5, 6, 7], 4, False, [2], [], 0, 1) == _host.RET_SUCCESS
    plan = s.schedule(0)
    s.update(plan, [-1], 0)
    assert s.tokens(1)[-1] == -1
    plan2 = s.schedule(0)          # planned on the placeholder
    res = s.resolve(plan, [2])     # ... which turns out to be EOS
    assert s.tokens(1)[-1] == 2 and res[0].finish_reason == _host.FINISH_EOS
    assert s.update(plan2, [-1], 0) == []  # the in-flight follow-up step is ignored
    assert not s.has_unfinished()


import pytest  # noqa: E402


@pytest.mark.parametrize("seed", list(range(int(__import__("os").environ.get("KSANA_FUZZ_SEEDS", "8")))))
def test_async_engine_switching_between_fast_and_host_state_steps(seed):
    """Plain greedy requests run through the asynchronous path; requests with penalties, log-probs, stop ids or
    seeded sampling need per-token host state and force synchronous steps while they live. Arrivals at random times
    make the engine switch back and forth with placeholders in flight; every request must equal a synchronous run."""
    import random
    import torch
    from ksanallm_b200.config.model_config import tiny_llama_config
    from ksanallm_b200.config.schema import parse_serving_config
    from ksanallm_b200.engine.llm_engine import LLMEngine
    from ksanallm_b200.engine.sampling_params import SamplingParams
    from ksanallm_b200.models.loader import load_model_weights
    from ksanallm_b200.models.transformer import TransformerModel
    rnd = random.Random(seed)
    cfg = tiny_llama_config()
    model = TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, dtype=torch.float32))

    def engine(enable_async, blocks):
        serving = parse_serving_config({"setting": {"batch_scheduler": {
            "max_batch_size": 6, "max_step_tokens": 128, "max_token_len": 256, "enable_auto_prefix_cache": True,
            "enable_async": enable_async}, "block_manager": {"block_token_num": 16}}})
        return LLMEngine(model, serving, num_blocks=blocks, num_host_blocks=0)
    g = torch.Generator().manual_seed(2000 + seed)
    prompts = [torch.randint(3, 31000, (rnd.randint(2, 40),), generator=g).tolist() for _ in range(10)]

    def params(i):
        n = 4 + (7 * i + seed) % 20
        kind = (i + seed) % 5
        if kind == 0:
            return SamplingParams(topk=1, max_new_tokens=n, ignore_eos=True, repetition_penalty=1.3, presence_penalty=0.4)
        if kind == 1:
            return SamplingParams(topk=1, max_new_tokens=n, ignore_eos=True, logprobs=2)
        if kind == 2:
            return SamplingParams(topk=25, topp=0.9, seed=3 + i, max_new_tokens=n, ignore_eos=True)
        if kind == 3:
            return SamplingParams(topk=1, max_new_tokens=n, stop_token_ids=[int(prompts[i][0])], min_tokens=2)
        return SamplingParams(topk=1, max_new_tokens=n, ignore_eos=True)
    sync = engine(False, 160)
    want = [sync.generate([p], params(i))[0].output_token_ids[0] for i, p in enumerate(prompts)]
    eng = engine(True, rnd.randint(20, 40))
    assert eng.async_mode
    reqs, order = {}, list(range(len(prompts)))
    rnd.shuffle(order)
    while order:
        for _ in range(rnd.randint(1, 2)):
            if order:
                i = order.pop()
                reqs[i] = eng.add_request(prompts[i], params(i))
        for _ in range(rnd.randint(0, 6)):
            eng.step()
    eng.run_until_done()
    for i in range(len(prompts)):
        assert reqs[i].output_token_ids[0] == want[i], (seed, i)
    assert eng.cache.num_free_blocks + eng.cache.num_cached_blocks == eng.cache.num_device_blocks
