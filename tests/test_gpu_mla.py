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
