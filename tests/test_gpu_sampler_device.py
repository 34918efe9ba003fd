"""The one-kernel device logits processor (penalties, n-gram rules, bias, min_tokens bans, grammar mask) against the
host implementation of the same rules (the CPU path of engine/sampler.py)."""
import numpy as np
import pytest
import torch

from ksanallm_b200.engine.sampler import SampleRow, Sampler
from ksanallm_b200.engine.sampling_params import SamplingParams

pytestmark = pytest.mark.gpu


def test_device_logits_processing_matches_host_rules():
    V = 1000
    rng = np.random.default_rng(0)
    rows = []
    specs = [dict(repetition_penalty=1.3), dict(presence_penalty=0.5, frequency_penalty=0.25),
             dict(no_repeat_ngram_size=2), dict(decoder_no_repeat_ngram_size=3), dict(encoder_no_repeat_ngram_size=2),
             dict(logit_bias={5: 2.5, 17: -3.0}), dict(min_tokens=50, stop_token_ids=[7, 9]), dict(),
             dict(repetition_penalty=0.8, frequency_penalty=0.1, no_repeat_ngram_size=1)]
    for i, kw in enumerate(specs):
        prompt = rng.integers(0, 40, int(rng.integers(3, 60))).tolist()
        out = rng.integers(0, 40, int(rng.integers(0, 30))).tolist()
        bm = None
        if i % 4 == 3:
            bm = rng.integers(-2 ** 31, 2 ** 31 - 1, (V + 31) // 32, dtype=np.int64).astype(np.int32)
        rows.append(SampleRow(SamplingParams(topk=1, **kw), prompt, out, bm, None))
    logits = torch.randn(len(rows), V)
    host = Sampler(V, torch.device("cpu"))
    host.eos_token_ids = [2]
    want = host.process_logits(logits.clone(), rows)
    dev = Sampler(V, torch.device("cuda"))
    dev.eos_token_ids = [2]
    got = dev.process_logits(logits.cuda(), rows).cpu()
    assert torch.equal(torch.isinf(got), torch.isinf(want))
    fin = torch.isfinite(want)
    assert torch.allclose(got[fin], want[fin], atol=1e-5, rtol=1e-5)
    # bf16 logits in, fp32 out; the input is left untouched
    lb = logits.to(torch.bfloat16).cuda()
    keep = lb.clone()
    got2 = dev.process_logits(lb, rows)
    assert got2.dtype == torch.float32 and torch.equal(lb, keep)
