"""KV block mover kernel: swap-out to the pinned host pool, swap-in and copy-on-write copies, every layer per launch."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_swap_out_in_and_fork_copies_round_trip():
    from ksanallm_b200.config.model_config import model_config_from_dict
    from ksanallm_b200.engine.model_runner import ModelRunner
    from ksanallm_b200.models.loader import load_model_weights
    from ksanallm_b200.models.transformer import TransformerModel
    cfg = model_config_from_dict(dict(model_type="llama", hidden_size=256, num_hidden_layers=3, num_attention_heads=2,
                                      num_key_value_heads=2, head_dim=128, intermediate_size=512, vocab_size=500,
                                      torch_dtype="bfloat16"))
    w = load_model_weights(cfg, synthetic_seed=1, device="cuda", dtype=torch.bfloat16)
    runner = ModelRunner(TransformerModel(cfg, w, max_positions=128), num_blocks=32, block_size=16, num_host_blocks=16,
                         max_step_tokens=64, max_batch_size=4, max_blocks_per_seq=8)
    assert runner._mover_ok()
    for c in runner.kv_caches:
        c.normal_()
    before = [c.clone() for c in runner.kv_caches]
    none = np.zeros((0, 2), dtype=np.int64)
    out_pairs = np.array([[3, 0], [7, 5], [30, 15]], dtype=np.int64)  # device block -> host block
    runner.apply_block_ops(out_pairs, none, none)
    for c in runner.kv_caches:
        c[[3, 7, 30]] = 0
    in_pairs = np.array([[0, 9], [5, 3], [15, 31]], dtype=np.int64)  # host block -> device block
    runner.apply_block_ops(none, in_pairs, none)
    runner.apply_block_ops(none, none, np.array([[9, 20], [1, 21]], dtype=np.int64))  # fork copies
    torch.cuda.synchronize()
    for c, b, h in zip(runner.kv_caches, before, runner.host_caches):
        assert torch.equal(h[0].cuda(), b[3]) and torch.equal(h[5].cuda(), b[7]) and torch.equal(h[15].cuda(), b[30])
        assert torch.equal(c[9], b[3]) and torch.equal(c[3], b[7]) and torch.equal(c[31], b[30])
        assert torch.equal(c[20], b[3]) and torch.equal(c[21], b[1])
        assert torch.equal(c[2], b[2])
