"""Parallel token prediction: N register tokens follow the last real token, every position yields a token, all of
them are kept and the registers' KV entries are dropped. The engine must match a plain forward that appends the
registers by hand, including across chunked prefill and batches of several requests."""
import dataclasses

import torch

from ksanallm_b200.config.model_config import tiny_llama_config
from ksanallm_b200.config.schema import parse_serving_config
from ksanallm_b200.engine.llm_engine import LLMEngine
from ksanallm_b200.engine.sampling_params import SamplingParams
from ksanallm_b200.models.loader import load_model_weights, synthetic_checkpoint
from ksanallm_b200.models.transformer import TransformerModel
from test_tiny_llama_oracle import plain_forward_all

REG, N = 31999, 2


def _oracle(sd, cfg, prompt, n_new):
    toks = list(prompt)
    toks.append(int(plain_forward_all(sd, cfg, toks)[-1].argmax()))  # the prompt's own step carries no registers
    while len(toks) - len(prompt) < n_new:
        lg = plain_forward_all(sd, cfg, toks + [REG] * N)
        toks.extend(int(t) for t in lg[-(N + 1):].argmax(-1))
    return toks[len(prompt):len(prompt) + n_new]


def test_ptp_matches_manual_register_forward():
    cfg = dataclasses.replace(tiny_llama_config(), num_register_token=N, reg_token_id=REG)
    sd = dict(synthetic_checkpoint(cfg, seed=0, std=0.02, dtype=torch.float32))
    model = TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, dtype=torch.float32))
    serving = parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 4, "max_step_tokens": 64,
                                                                     "max_token_len": 256, "split_fuse_token_num": 24},
                                                "block_manager": {"block_token_num": 16}}})
    eng = LLMEngine(model, serving, num_blocks=64, num_host_blocks=0)
    assert eng.ptp_steps == N and not eng.async_mode
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(3, 31000, (n,), generator=g).tolist() for n in (5, 33, 50)]
    reqs = eng.generate(prompts, SamplingParams(topk=1, max_new_tokens=13, ignore_eos=True))
    for prompt, req in zip(prompts, reqs):
        assert req.output_token_ids[0] == _oracle(sd, cfg, prompt, 13)
    # 1 + 3 * 4 = 13 tokens: five model steps per request instead of thirteen
    assert eng.stats["steps"] <= 5 + 3


import pytest  # noqa: E402


@pytest.mark.parametrize("seed", list(range(int(__import__("os").environ.get("KSANA_FUZZ_SEEDS", "6")))))
def test_ptp_outputs_do_not_depend_on_memory_pressure_or_arrival_order(seed):
    """Register-token decoding with a block pool that forces pre-emption, chunked prefill and requests arriving
    between steps: every request generates what it generates alone in an engine with plenty of blocks."""
    import random
    rnd = random.Random(seed)
    cfg = dataclasses.replace(tiny_llama_config(), num_register_token=N, reg_token_id=REG)
    model = TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, dtype=torch.float32))

    def serving(**bs):
        return parse_serving_config({"setting": {"batch_scheduler": dict(
            {"max_batch_size": 6, "max_step_tokens": 96, "max_token_len": 256}, **bs),
            "block_manager": {"block_token_num": 16}}})
    g = torch.Generator().manual_seed(700 + seed)
    stem = torch.randint(3, 31000, (32,), generator=g).tolist()
    prompts = [(stem if rnd.random() < 0.6 else []) + torch.randint(3, 31000, (rnd.randint(2, 30),), generator=g).tolist()
               for _ in range(7)]
    params = [SamplingParams(topk=1, max_new_tokens=rnd.randint(3, 30), ignore_eos=True) for _ in prompts]
    roomy = LLMEngine(model, serving(), num_blocks=160, num_host_blocks=0)
    want = [roomy.generate([p], sp)[0].output_token_ids[0] for p, sp in zip(prompts, params)]
    host_blocks = rnd.choice([0, 24])
    eng = LLMEngine(model, serving(preempt_mode=rnd.choice([0, 1]) if host_blocks else 1,
                                   split_fuse_token_num=rnd.choice([0, 16, 40]),
                                   enable_auto_prefix_cache=rnd.random() < 0.7, max_batch_size=rnd.choice([3, 6])),
                    num_blocks=rnd.randint(14, 24), num_host_blocks=host_blocks)
    reqs, order = [], list(range(len(prompts)))
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
