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
