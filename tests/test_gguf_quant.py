"""Quantised GGML block types are expanded at load: checked against the ``gguf`` package's own decoder."""
import numpy as np
import pytest
import torch

from ksanallm_b200.models import gguf_reader

gguf = pytest.importorskip("gguf")
T = gguf.GGMLQuantizationType


def _random_blocks(rng, gtype, n_blocks):
    """Random block bytes with finite fp16 scale fields (every other field may hold any bit pattern)."""
    per, nbytes, _ = gguf_reader._GGML_QUANT[int(gtype)]
    b = rng.integers(0, 256, (n_blocks, nbytes), dtype=np.uint8)
    halves = {T.Q4_0: [0], T.Q4_1: [0, 2], T.Q5_0: [0], T.Q5_1: [0, 2], T.Q8_0: [0], T.Q4_K: [0, 2], T.Q5_K: [0, 2],
              T.Q6_K: [208]}[gtype]
    for off in halves:
        b[:, off:off + 2] = rng.uniform(-0.5, 0.5, (n_blocks, 1)).astype(np.float16).view(np.uint8)
    return b


@pytest.mark.parametrize("gtype", [T.Q4_0, T.Q4_1, T.Q5_0, T.Q5_1, T.Q8_0, T.Q4_K, T.Q5_K, T.Q6_K])
def test_block_decoders_match_the_gguf_package(gtype):
    rng = np.random.default_rng(int(gtype))
    per = gguf_reader._GGML_QUANT[int(gtype)][0]
    rows, cols = 6, 2 * 256
    raw = _random_blocks(rng, gtype, rows * cols // per)
    got = gguf_reader.dequantize_ggml(raw.reshape(-1), int(gtype), [rows, cols])
    want = gguf.quants.dequantize(raw.reshape(rows, -1), gtype)
    assert got.shape == want.shape == (rows, cols)
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)


def test_quantised_file_loads_as_fp16(tmp_path):
    rng = np.random.default_rng(0)
    w = rng.standard_normal((64, 256)).astype(np.float32)
    q8 = gguf.quants.quantize(w, T.Q8_0)
    q4k = _random_blocks(rng, T.Q4_K, 64)  # [64, 256] in Q4_K
    path = str(tmp_path / "q.gguf")
    gguf_reader.write_gguf(path, {"blk.0.attn_q.weight": (int(T.Q8_0), [64, 256], q8.tobytes()),
                                  "blk.0.ffn_up.weight": (int(T.Q4_K), [64, 256], q4k.tobytes()),
                                  "output_norm.weight": torch.ones(256)},
                           {"general.architecture": "qwen2", "qwen2.block_count": 1})
    names = dict(gguf_reader.iter_gguf(path))
    a = names["model.layers.0.self_attn.q_proj.weight"]
    assert a.dtype == torch.float16 and tuple(a.shape) == (64, 256)
    assert (a.float() - torch.from_numpy(w)).abs().max().item() < 0.05
    b = names["model.layers.0.mlp.up_proj.weight"]
    want = gguf.quants.dequantize(q4k.reshape(64, -1), T.Q4_K)
    assert torch.allclose(b.float(), torch.from_numpy(want).half().float())
    assert names["model.norm.weight"].dtype == torch.float32


def test_unknown_block_type_raises(tmp_path):
    path = str(tmp_path / "bad.gguf")
    gguf_reader.write_gguf(path, {"blk.0.attn_q.weight": (10, [2, 256], bytes(2 * 84))}, {"general.architecture": "llama"})
    with pytest.raises(ValueError):
        gguf_reader.read_gguf(path)
