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
