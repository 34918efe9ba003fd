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
