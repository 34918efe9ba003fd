"""Absorbed MLA attention over the latent cache (tcgen05) and the latent cache append against the fp32 reference."""
import pytest
import torch

from ksanallm_b200.engine.step_input import make_step_input
from ksanallm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _run(q_lens, kv_lens, h, seed=0):
    from ksanallm_b200.ops import cuda, cuda_mla
    g = torch.Generator(device="cuda").manual_seed(seed)
    bs = 64
    nblk = [(L + bs - 1) // bs for L in kv_lens]
    total = sum(nblk) + 2
    cache = (torch.randn(total, bs, 576, device="cuda", generator=g) * 0.3).to(torch.bfloat16)
    perm = torch.randperm(total, device="cuda", generator=g).tolist()
    bt = torch.zeros(len(kv_lens), max(nblk) + 1, dtype=torch.int32)
    it = iter(perm)
    for b, n in enumerate(nblk):
        for j in range(n):
            bt[b, j] = next(it)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    ql = (torch.randn(T, h, 512, device="cuda", generator=g) * 0.3).to(torch.bfloat16)
    qr = (torch.randn(T, h, 64, device="cuda", generator=g) * 0.3).to(torch.bfloat16)
    meta = make_step_input([0] * T, [0] * T, [0] * T, cu, kv_lens, bt, device="cuda")
    scale = 0.1147
    out = cuda_mla.mla_paged_attention(ql, qr, cache, meta, scale)
    torch.cuda.synchronize()
    assert cuda.read_error() == 0
    want = ref.mla_paged_attention(ql, qr, cache, meta.block_tables, meta.cu_q, meta.kv_lens, scale)
    err = (out.float() - want.float()).abs().max().item()
    assert err < 2e-2, f"max err {err}"


def test_mla_decode_single_token():
    _run([1, 1, 1], [1, 70, 500], h=128)


def test_mla_decode_split_kv_long_context():
    _run([1], [5000], h=128)


def test_mla_decode_mtp_two_tokens_and_fewer_heads():
    _run([2, 2], [130, 64], h=16)


def test_mla_prefill_chunk():
    _run([40, 7], [40, 7 + 128], h=32)


def test_mla_cache_append():
    from ksanallm_b200.ops import cuda_mla
    T = 77
    latent = torch.randn(T, 512, device="cuda").to(torch.bfloat16)
    rope = torch.randn(T, 64, device="cuda").to(torch.bfloat16)
    slots = torch.randperm(5 * 64, device="cuda")[:T].to(torch.int32)
    c1 = torch.zeros(5, 64, 576, device="cuda", dtype=torch.bfloat16)
    c2 = c1.clone()
    cuda_mla.mla_cache_append(latent, rope, slots, c1)
    ref.mla_cache_append(latent, rope, slots, c2)
    assert torch.equal(c1, c2)


def test_head_batched_gemm_strided_operands():
    """C[t, b, :] = A[t, b, :] @ W[b]^T with A and C as views into wider rows (the absorb steps of MLA)."""
    from ksanallm_b200.ops import cuda, cuda_mla
    for T, B, N, K in ((1, 16, 512, 128), (300, 5, 128, 512), (129, 128, 512, 128)):
        g = torch.Generator(device="cuda").manual_seed(T + B)
        q = (torch.randn(T, B, K + 64, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
        w = (torch.randn(B, N, K, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
        out = torch.zeros(T, B, N + 64, device="cuda", dtype=torch.bfloat16)
        cuda_mla.gemm_batched(q[..., :K], w, out[..., :N])
        torch.cuda.synchronize()
        assert cuda.read_error() == 0
        want = torch.einsum("tbk,bnk->tbn", q[..., :K].float(), w.float())
        assert (out[..., :N].float() - want).abs().max().item() < 2e-2 * max(1.0, want.abs().max().item())
        assert out[..., N:].abs().max().item() == 0


def test_mla_layer_fused_core_matches_the_pytorch_formulation():
    """MLAttention.core through the kernels (absorb GEMMs, fused RoPE + cache append, attention) against the same layer
    forced onto the PyTorch formulation of these steps."""
    from ksanallm_b200.config.model_config import model_config_from_dict
    from ksanallm_b200.models.loader import load_model_weights
    from ksanallm_b200.models.transformer import TransformerModel
    cfg = model_config_from_dict(dict(
        model_type="deepseek_v3", hidden_size=1024, num_hidden_layers=1, num_attention_heads=16,
        num_key_value_heads=16, intermediate_size=2048, moe_intermediate_size=256, n_routed_experts=8,
        n_shared_experts=1, num_experts_per_tok=2, first_k_dense_replace=1, n_group=1, topk_group=1,
        scoring_func="sigmoid", topk_method="noaux_tc", norm_topk_prob=True, routed_scaling_factor=1.0,
        q_lora_rank=256, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
        rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=1000, max_position_embeddings=4096,
        torch_dtype="bfloat16"))
    w = load_model_weights(cfg, synthetic_seed=2, device="cuda", dtype=torch.bfloat16)
    m = TransformerModel(cfg, w, max_positions=512)
    attn = m.layers[0].attn
    q_lens, kv_lens = [70, 1, 1], [70, 130, 9]
    cu, pos, slots, bt = [0], [], [], torch.zeros(3, 4, dtype=torch.int32)
    nxt = 0
    for b, (ql, kl) in enumerate(zip(q_lens, kv_lens)):
        nb = (kl + 63) // 64
        bt[b, :nb] = torch.arange(nxt, nxt + nb, dtype=torch.int32)
        for p in range(kl - ql, kl):
            pos.append(p)
            slots.append(int(bt[b, p // 64]) * 64 + p % 64)
        nxt += nb
        cu.append(cu[-1] + ql)
    T = cu[-1]
    meta = make_step_input([1] * T, pos, slots, cu, kv_lens, bt, device="cuda")
    h = (torch.randn(T, 1024, device="cuda") * 0.5).to(torch.bfloat16)
    c1 = (torch.randn(nxt + 1, 64, 576, device="cuda") * 0.2).to(torch.bfloat16)
    c2 = c1.clone()
    out_fused = attn.core(h, meta, c1)
    assert attn._fused_ok, "the kernel path was not taken"
    attn._fused_ok = False
    out_torch = attn.core(h, meta, c2)
    torch.cuda.synchronize()
    assert (out_fused.float() - out_torch.float()).abs().max().item() < 3e-2 * max(1.0, out_torch.float().abs().max().item())
    assert (c1.float() - c2.float()).abs().max().item() < 2e-2
