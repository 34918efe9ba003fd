"""MoE kernels: router variants, expert pipeline (permute -> grouped tcgen05 GEMMs -> combine)."""
import pytest
import torch

from ksanallm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("E,k,scoring,norm,ng,tg,bias", [(8, 2, "softmax", True, 1, 1, False),
                                                         (64, 6, "softmax", False, 1, 1, False),
                                                         (256, 8, "sigmoid", True, 8, 4, True),
                                                         (160, 6, "softmax", False, 8, 3, False)])
def test_route(E, k, scoring, norm, ng, tg, bias):
    from ksanallm_b200.ops import cuda_moe
    torch.manual_seed(E)
    logits = torch.randn(37, E, device="cuda")
    b = torch.randn(E, device="cuda") * 0.1 if bias else None
    ids, w = cuda_moe.moe_route(logits, k, scoring, norm, ng, tg, 2.5, b)
    ids2, w2 = ref.moe_route(logits, k, scoring, norm, ng, tg, 2.5, b)
    assert torch.equal(ids.sort(-1).values, ids2.sort(-1).values)
    a = torch.zeros(37, E, device="cuda").scatter_(1, ids.long(), w)
    c = torch.zeros(37, E, device="cuda").scatter_(1, ids2.long(), w2)
    assert torch.allclose(a, c, atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("T,E,k,H,I,off,e_local", [(50, 8, 2, 256, 384, 0, 8), (300, 16, 4, 512, 256, 4, 8),
                                                   (3, 32, 8, 1024, 128, 0, 32)])
def test_experts(T, E, k, H, I, off, e_local):
    from ksanallm_b200.ops import cuda, cuda_moe
    torch.manual_seed(T)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda")
    ids, w = ref.moe_route(logits, k, "softmax", True)
    w1 = (torch.randn(e_local, 2 * I, H, device="cuda") * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(e_local, H, I, device="cuda") * 0.05).to(torch.bfloat16)
    y = cuda_moe.moe_experts(x, ids, w, w1, w2, off)
    torch.cuda.synchronize()
    assert cuda.read_error() == 0
    want = ref.moe_experts(x, ids, w, w1, w2, off)
    err = (y.float() - want.float()).abs().max().item()
    assert err < 3e-2 * max(1.0, want.float().abs().max().item()), err
    y2 = cuda_moe.moe_experts(x, ids, w, w1, w2, off)  # the count buffer was left clean
    torch.cuda.synchronize()
    assert torch.equal(y, y2)


@pytest.mark.parametrize("T,E,k,H,I,off,e_local", [(50, 8, 2, 256, 384, 0, 8), (300, 16, 4, 512, 256, 4, 8),
                                                   (3, 32, 8, 1024, 128, 0, 32), (700, 8, 2, 1024, 512, 0, 8)])
def test_experts_fp8_block_scaled(T, E, k, H, I, off, e_local):
    """Grouped block-scaled fp8 expert GEMMs + fused SiLU * mul + re-quantisation against the per-expert fp32
    restatement of the same quantised math."""
    from ksanallm_b200.ops import cuda, cuda_moe
    torch.manual_seed(T + E)
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    ids, w = ref.moe_route(torch.randn(T, E, device="cuda"), k, "softmax", True)
    q1, s1, q2, s2 = [], [], [], []
    for _ in range(e_local):
        a, b = ref.quant_fp8_block_weight(torch.randn(2 * I, H, device="cuda") * 0.05)
        c, d = ref.quant_fp8_block_weight(torch.randn(H, I, device="cuda") * 0.05)
        q1.append(a), s1.append(b), q2.append(c), s2.append(d)
    q1, s1, q2, s2 = torch.stack(q1), torch.stack(s1), torch.stack(q2), torch.stack(s2)
    assert cuda_moe.supports_fp8(x, q1, s1, q2, s2)
    y = cuda_moe.moe_experts_fp8(x, ids, w, q1, s1, q2, s2, off)
    torch.cuda.synchronize()
    assert cuda.read_error() == 0
    want = ref.moe_experts_fp8(x, ids, w, q1, s1, q2, s2, off)
    err = (y.float() - want.float()).abs().max().item()
    assert err < 4e-2 * max(1.0, want.float().abs().max().item()), err
    y2 = cuda_moe.moe_experts_fp8(x, ids, w, q1, s1, q2, s2, off)
    torch.cuda.synchronize()
    assert torch.equal(y, y2)


def test_silu_mul_quant_fp8():
    from ksanallm_b200.ops import cuda
    T, I = 77, 384
    h = torch.randn(T, 2 * I, device="cuda").to(torch.bfloat16)
    q = torch.empty(T, I, dtype=torch.float8_e4m3fn, device="cuda")
    s = torch.empty(T, I // 128, dtype=torch.float32, device="cuda")
    cuda._check(cuda.lib().ksana_silu_mul_quant_fp8(cuda._ptr(h), 2 * I, cuda._ptr(q), I, cuda._ptr(s), T, I,
                                                    cuda._stream()), "silu_mul_quant_fp8")
    torch.cuda.synchronize()
    a = ref.silu_and_mul(h)
    q2, s2 = ref.quant_fp8_group(a)
    assert torch.allclose(s, s2, rtol=2e-2, atol=1e-6)
    got = q.float().view(T, I // 128, 128) * s.unsqueeze(-1)
    want = q2.float().view(T, I // 128, 128) * s2.unsqueeze(-1)
    assert (got - want).abs().max().item() < 0.07 * max(1.0, want.abs().max().item())
