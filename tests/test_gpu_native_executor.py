"""The one-call-per-step native executor must reproduce the per-layer Python path exactly (same kernels, same order)."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(model_type="llama", quantize=None, **over):
    from ksanallm_b200.config.model_config import model_config_from_dict
    from ksanallm_b200.models.loader import load_model_weights
    from ksanallm_b200.models.transformer import TransformerModel
    d = dict(model_type=model_type, hidden_size=1024, num_hidden_layers=3, num_attention_heads=8,
             num_key_value_heads=4, intermediate_size=2816, vocab_size=1000, torch_dtype="bfloat16")
    d.update(over)
    cfg = model_config_from_dict(d)
    w = load_model_weights(cfg, synthetic_seed=4, device="cuda", dtype=torch.bfloat16, quantize=quantize)
    return TransformerModel(cfg, w, max_positions=512)


def _mixed_meta():
    from ksanallm_b200.engine.step_input import make_step_input
    # one prefill of 37 tokens, one chunk continuing at position 20 (9 new tokens), three decodes
    q_lens = [37, 9, 1, 1, 1]
    kv_lens = [37, 29, 50, 17, 64]
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    bt = torch.zeros(5, 4, dtype=torch.int32)
    nxt = 0
    pos, slots = [], []
    for b, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        nb = (kl + 15) // 16
        bt[b, :nb] = torch.arange(nxt, nxt + nb, dtype=torch.int32)
        for p in range(kl - ql, kl):
            pos.append(p)
            slots.append(int(bt[b, p // 16]) * 16 + p % 16)
        nxt += nb
    ids = [(7 * i + 3) % 1000 for i in range(cu[-1])]
    return make_step_input(ids, pos, slots, cu, kv_lens, bt, num_prefill=2, device="cuda"), nxt


@pytest.mark.parametrize("model_type,extra", [("llama", {}), ("qwen3", {"head_dim": 128}), ("qwen2", {}),
                                              ("qwen3", {"head_dim": 128, "quantize": "fp8_block"})])
def test_native_matches_python_path(model_type, extra):
    from ksanallm_b200.ops import cuda
    m = _build(model_type, **extra)
    meta, nblocks = _mixed_meta()
    assert m._native_executor() is not None
    kv_a = m.allocate_kv_cache(nblocks + 1, 16)
    for c in kv_a:
        c.normal_(0, 0.3)
    kv_b = [c.clone() for c in kv_a]
    base = cuda.launch_count
    out_native = m.forward(meta, kv_a).clone()
    native_launches = cuda.launch_count - base
    m._native = None  # per-layer Python path
    out_python = m.forward(meta, kv_b).clone()
    torch.cuda.synchronize()
    assert cuda.read_error() == 0
    if extra.get("quantize"):
        # block-scaled e4m3 weights: same kernels as the Python path (quantise, fp8 GEMM, fused SiLU-mul-quantise)
        assert m.layers[0].attn.qkv.kind == "fp8_block"
        assert (out_native.float() - out_python.float()).abs().max().item() <= 2e-2 * out_python.float().abs().max().item()
    else:
        assert torch.equal(out_native, out_python)
    for a, b in zip(kv_a, kv_b):
        assert torch.equal(a, b) or extra.get("quantize")
    assert native_launches >= 8 * 3


def test_native_declines_unsupported():
    m = _build("llama", num_hidden_layers=1, hidden_size=512, num_attention_heads=8, num_key_value_heads=8,
               intermediate_size=1024)  # head_dim 64
    assert m._native_executor() is None


def test_native_rebinds_a_new_cache_at_the_old_address():
    """A second KV cache (a new engine on the same model) may start where the freed one started while its other
    layers sit elsewhere: the executor must not keep the old layer pointers."""
    m = _build("llama")
    meta, nblocks = _mixed_meta()
    kv_1 = m.allocate_kv_cache(nblocks + 1, 16)
    m.forward(meta, kv_1)
    torch.cuda.synchronize()
    first_ptr = kv_1[0].data_ptr()
    del kv_1
    # same first layer tensor size (the allocator hands the block back), other layers allocated after a spacer
    kv_2 = [torch.zeros(nblocks + 1, 2, 4, 16, 128, dtype=torch.bfloat16, device="cuda")]
    spacer = torch.zeros(3 << 20, dtype=torch.uint8, device="cuda")
    kv_2 += [torch.zeros(nblocks + 1, 2, 4, 16, 128, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    kv_3 = [c.clone() for c in kv_2]
    out_native = m.forward(meta, kv_2).clone()
    m._native = None
    out_python = m.forward(meta, kv_3).clone()
    torch.cuda.synchronize()
    assert torch.equal(out_native, out_python)
    for a, b in zip(kv_2, kv_3):
        assert torch.equal(a, b)
    del spacer, first_ptr


def test_native_with_fused_silu_mul_gemm(monkeypatch):
    """KSANA_FUSED_SWIGLU=1: prefill-sized steps run the gated FFN's first GEMM with the activation as its epilogue
    (fp32 SiLU-mul on the accumulators instead of on the bf16-rounded GEMM output: close, not bit-equal)."""
    from ksanallm_b200.engine.step_input import make_step_input
    from ksanallm_b200.ops import cuda
    monkeypatch.setenv("KSANA_FUSED_SWIGLU", "1")
    m = _build("llama")
    T = 450
    nb = (T + 15) // 16
    bt = torch.arange(nb, dtype=torch.int32).view(1, nb)
    meta = make_step_input([(7 * i + 3) % 1000 for i in range(T)], list(range(T)), list(range(T)), [0, T], [T], bt,
                           num_prefill=1, device="cuda")
    ex = m._native_executor()
    assert ex is not None and len(ex._wgu_il) == len(m.layers)
    out_fused = m.forward(meta, m.allocate_kv_cache(nb + 1, 16)).clone()
    m._native = None
    out_python = m.forward(meta, m.allocate_kv_cache(nb + 1, 16)).clone()
    torch.cuda.synchronize()
    assert cuda.read_error() == 0
    err = (out_fused.float() - out_python.float()).abs().max().item()
    assert err <= 3e-2 * out_python.float().abs().max().item(), err
