"""Synthetic weights under expert parallelism: a rank generates only the routed experts it owns, and what it gets
equals the corresponding slice of a full load."""
import torch

from ksanallm_b200.config.model_config import NAMED_CONFIGS
from ksanallm_b200.models import loader


def test_ep_rank_generates_only_its_experts_and_matches_the_full_load():
    cfg = NAMED_CONFIGS["tiny-moe"]()
    full = loader.load_model_weights(cfg, synthetic_seed=3, device="cpu", dtype=torch.float32)
    E = cfg.num_experts
    seen = []
    real = loader.synthetic_checkpoint

    def spy(*a, **kw):
        for name, t in real(*a, **kw):
            if ".experts." in name:
                seen.append(name)
            yield name, t
    loader.synthetic_checkpoint = spy
    try:
        parts = [loader.load_model_weights(cfg, synthetic_seed=3, device="cpu", dtype=torch.float32, tp_rank=0, tp_size=1,
                                           ep_rank=r, ep_size=2) for r in range(2)]
    finally:
        loader.synthetic_checkpoint = real
    # 2 ranks x (E / 2 experts) x 3 matrices x layers: nothing generated for the other rank's experts
    assert len(seen) == 2 * (E // 2) * 3 * cfg.num_layers
    for key, w in full.items():
        if ".experts." in key:
            got = torch.cat([p[key] for p in parts], 0)
            assert torch.equal(got, w), key
        else:
            assert torch.equal(parts[0][key], w) and torch.equal(parts[1][key], w), key
