"""Sampler on CPU: logit processing (repetition penalty with the transformers semantics, the three no-repeat-n-gram
rules, grammar bitmask), greedy / top-k / top-p / temperature selection, per-request seeds, log-probabilities."""
import numpy as np
import torch

from ksanallm_b200.engine.sampler import SampleRow, Sampler
from ksanallm_b200.engine.sampling_params import SamplingParams

V = 50


def _row(prompt=(), out=(), gen_seed=None, **kw):
    g = None
    if gen_seed is not None:
        g = torch.Generator().manual_seed(gen_seed)
    return SampleRow(SamplingParams(**kw), list(prompt), list(out), None, g)


def test_repetition_penalty_divides_positive_and_multiplies_negative_logits():
    s = Sampler(V, torch.device("cpu"))
    logits = torch.zeros(1, V)
    logits[0, 3], logits[0, 4], logits[0, 5] = 2.0, -2.0, 2.0
    x = s.process_logits(logits, [_row(prompt=[3], out=[4], topk=1, repetition_penalty=2.0)])
    assert x[0, 3].item() == 1.0 and x[0, 4].item() == -4.0 and x[0, 5].item() == 2.0


def test_no_repeat_ngram_rules():
    s = Sampler(V, torch.device("cpu"))
    logits = torch.zeros(1, V)
    # history (prompt + output) 7 8 9 7 8 -> the 3-gram 7 8 9 exists, so 9 is banned after "7 8"
    x = s.process_logits(logits, [_row(prompt=[7, 8, 9], out=[7, 8], topk=1, no_repeat_ngram_size=3)])
    assert torch.isinf(x[0, 9]) and torch.isfinite(x[0, 10])
    # decoder rule: only the generated tokens count
    x = s.process_logits(logits, [_row(prompt=[7, 8, 9], out=[7, 8], topk=1, decoder_no_repeat_ngram_size=3)])
    assert torch.isfinite(x).all()
    x = s.process_logits(logits, [_row(prompt=[1], out=[7, 8, 9, 7, 8], topk=1, decoder_no_repeat_ngram_size=3)])
    assert torch.isinf(x[0, 9])
    # encoder rule: the output may not reproduce an n-gram of the prompt
    x = s.process_logits(logits, [_row(prompt=[7, 8, 9, 4], out=[2, 7, 8], topk=1, encoder_no_repeat_ngram_size=3)])
    assert torch.isinf(x[0, 9]) and torch.isfinite(x[0, 4])


def test_bitmask_limits_the_choice_even_for_greedy_rows():
    s = Sampler(V, torch.device("cpu"))
    logits = torch.zeros(2, V)
    logits[:, 40] = 9.0
    bm = np.zeros(2, dtype=np.int32)
    bm[0] = (1 << 5) | (1 << 6)
    rows = [SampleRow(SamplingParams(topk=1), [1], [], bm, None), _row(prompt=[1], topk=1)]
    logits[0, 6] = 1.0
    out = s.sample(logits, rows)
    assert out.tokens == [6, 40]


def test_topk_topp_temperature_and_seeds():
    s = Sampler(V, torch.device("cpu"))
    logits = torch.full((1, V), -10.0)
    logits[0, :4] = torch.tensor([3.0, 2.0, 1.0, 0.0])
    seen = set()
    for seed in range(40):
        seen.add(s.sample(logits.clone(), [_row(prompt=[1], topk=2, temperature=1.5, gen_seed=seed)]).tokens[0])
    assert seen == {0, 1}                                   # never outside the top 2
    seen = set()
    for seed in range(40):
        seen.add(s.sample(logits.clone(), [_row(prompt=[1], topk=40, topp=0.6, gen_seed=seed)]).tokens[0])
    assert seen == {0}                                      # p(0) = 0.64 covers the nucleus alone
    a = [s.sample(logits.clone(), [_row(prompt=[1], topk=4, temperature=2.0, gen_seed=123)]).tokens[0] for _ in range(3)]
    assert len(set(a)) == 1                                 # same seed, same draw
    # rows of one batch keep their own parameters
    rows = [_row(prompt=[1], topk=1), _row(prompt=[1], topk=2, temperature=1.0, gen_seed=5)]
    out = s.sample(logits.repeat(2, 1), rows)
    assert out.tokens[0] == 0 and out.tokens[1] in (0, 1)


def test_logprobs_report_the_chosen_token_and_the_top_n():
    s = Sampler(V, torch.device("cpu"))
    logits = torch.full((1, V), -20.0)
    logits[0, :3] = torch.tensor([2.0, 1.0, 0.0])
    out = s.sample(logits, [_row(prompt=[1], topk=1, logprobs=2)])
    lp = torch.log_softmax(logits[0], -1)
    assert out.tokens == [0] and abs(out.chosen_logprob[0] - lp[0].item()) < 1e-5
    assert [t for t, _ in out.logprobs[0]] == [0, 1] and abs(out.logprobs[0][1][1] - lp[1].item()) < 1e-5


def test_openai_style_penalties_bias_and_min_tokens():
    s = Sampler(V, torch.device("cpu"))
    s.eos_token_ids = [2]
    logits = torch.zeros(1, V)
    logits[0, 7], logits[0, 8], logits[0, 2] = 3.0, 2.5, 9.0
    # presence + frequency: token 7 was generated twice -> 3 - (0.5 + 2 * 0.4) = 1.7 < 2.5
    x = s.process_logits(logits, [_row(prompt=[7], out=[7, 7, 9], topk=1, presence_penalty=0.5, frequency_penalty=0.4,
                                       ignore_eos=True)])
    assert abs(x[0, 7].item() - 1.7) < 1e-6 and abs(x[0, 9].item() + 0.9) < 1e-6 and x[0, 8].item() == 2.5
    # logit_bias accepts string keys as the OpenAI API sends them
    x = s.process_logits(logits, [_row(prompt=[1], topk=1, logit_bias={"8": 5.0, 7: -100.0}, ignore_eos=True)])
    assert x[0, 8].item() == 7.5 and x[0, 7].item() == -97.0
    # min_tokens: EOS and stop ids are out of reach until enough tokens exist
    out = s.sample(logits.clone(), [_row(prompt=[1], out=[4], topk=1, min_tokens=3, stop_token_ids=[7])])
    assert out.tokens == [8]
    out = s.sample(logits.clone(), [_row(prompt=[1], out=[4, 5, 6], topk=1, min_tokens=3, stop_token_ids=[7])])
    assert out.tokens == [2]
