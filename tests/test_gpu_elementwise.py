"""Bandwidth-bound kernels against the fp32 reference implementations."""
import pytest
import torch

from ksanallm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _close(a, b, atol=2e-2, rtol=2e-2):
    a, b = a.float(), b.float()
    assert torch.allclose(a, b, atol=atol, rtol=rtol), f"max err {(a - b).abs().max().item()}"


@pytest.mark.parametrize("H", [256, 4096, 5120, 7168, 8192])
def test_rms_norm(H):
    from ksanallm_b200.ops import cuda
    x = torch.randn(37, H, device="cuda").to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
    _close(cuda.rms_norm(x, w, 1e-6), ref.rms_norm(x, w, 1e-6))
    r1 = torch.randn(37, H, device="cuda").to(torch.bfloat16)
    r2 = r1.clone()
    y1 = cuda.rms_norm(x, w, 1e-6, r1)
    y2 = ref.rms_norm(x, w, 1e-6, r2)
    _close(r1, r2)
    _close(y1, y2, atol=4e-2)


def test_silu_mul_and_embedding():
    from ksanallm_b200.ops import cuda
    x = torch.randn(19, 2 * 11008, device="cuda").to(torch.bfloat16)
    _close(cuda.silu_and_mul(x), ref.silu_and_mul(x))
    table = torch.randn(1000, 4096, device="cuda").to(torch.bfloat16)
    ids = torch.randint(0, 1000, (33,), device="cuda", dtype=torch.int32)
    assert torch.equal(cuda.embedding(ids, table), ref.embedding(ids, table))


@pytest.mark.parametrize("interleaved,qknorm,rotary_dim", [(False, False, 0), (True, False, 0), (False, True, 0),
                                                           (True, False, 64)])
def test_rope_qknorm_cache(interleaved, qknorm, rotary_dim):
    from ksanallm_b200.ops import cuda
    T, h, hk, d, bs, nb = 45, 8, 2, 128, 16, 12
    qkv = torch.randn(T, (h + 2 * hk) * d, device="cuda").to(torch.bfloat16)
    qkv2 = qkv.clone()
    rd = rotary_dim or d
    cs = ref.build_rope_cache(rd, 512, 10000.0, None, "cuda")
    pos = torch.randint(0, 512, (T,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(nb * bs, device="cuda")[:T].to(torch.int32)
    qw = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16) if qknorm else None
    kw = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16) if qknorm else None

    def views(buf):
        return (buf[:, :h * d].view(T, h, d), buf[:, h * d:(h + hk) * d].view(T, hk, d),
                buf[:, (h + hk) * d:].view(T, hk, d))

    c1 = torch.zeros(nb, 2, hk, bs, d, device="cuda", dtype=torch.bfloat16)
    c2 = c1.clone()
    q1, k1, v1 = views(qkv)
    q2, k2, v2 = views(qkv2)
    cuda.rope_qknorm_cache(q1, k1, v1, pos, cs, slots, c1, qw, kw, 1e-6, interleaved, rotary_dim)
    ref.rope_qknorm_cache(q2, k2, v2, pos, cs, slots, c2, qw, kw, 1e-6, interleaved, rotary_dim)
    _close(qkv, qkv2, atol=3e-2)
    _close(c1, c2, atol=3e-2)


def test_quant_fp8_group():
    from ksanallm_b200.ops import cuda
    x = (torch.randn(33, 1024, device="cuda") * 3).to(torch.bfloat16)
    q, s = cuda.quant_fp8_group(x)
    q2, s2 = ref.quant_fp8_group(x)
    _close(s, s2, atol=1e-6, rtol=1e-5)
    d1 = q.float().view(33, 8, 128) * s.unsqueeze(-1)
    _close(d1.view(33, 1024), x, atol=0.3, rtol=0.07)


def test_argmax_and_sampling():
    from ksanallm_b200.ops import cuda
    logits = torch.randn(9, 32000, device="cuda")
    assert torch.equal(cuda.argmax(logits).long(), logits.argmax(-1))
    B, V = 64, 32000
    logits = torch.randn(B, V, device="cuda") * 3
    temp = torch.rand(B, device="cuda") + 0.5
    topk = torch.randint(1, 200, (B,), device="cuda", dtype=torch.int32)
    topp = torch.rand(B, device="cuda") * 0.6 + 0.4
    u = torch.rand(B, device="cuda")
    got = cuda.sample(logits, temp, topk, topp, u)
    want = ref.sample(logits, temp, topk, topp, u)
    assert (got != want).sum().item() <= 2, f"{(got != want).sum().item()} mismatches"
    # every sampled token lies inside the support the reference distribution allows
    probs = ref.sample_probs(logits, temp, topk, topp)
    assert (probs.gather(1, got.long().unsqueeze(1)) > 0).all()
    # k = 1 is greedy
    got = cuda.sample(logits, temp, torch.ones_like(topk), topp, u)
    assert torch.equal(got.long(), logits.argmax(-1))


def test_bounded_flag_wait_times_out_cleanly():
    """A wait on a flag that nobody sets must give up by itself, report KERR_PEER_TIMEOUT in the status word and
    leave the context usable (no trap, no hang)."""
    import ctypes
    from ksanallm_b200.ops import cuda
    lib = cuda.lib()
    lib.ksana_flag_timeout_probe.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p, ctypes.c_void_p]
    lib.ksana_flag_timeout_probe.restype = ctypes.c_int
    cuda.read_error()
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    result = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    assert lib.ksana_flag_timeout_probe(flag.data_ptr(), 5, result.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert result.item() == 0
    assert cuda.read_error() & 8  # KERR_PEER_TIMEOUT
    # satisfied flag: returns immediately with success, context still fine
    flag.fill_(7)
    lib.ksana_flag_timeout_probe(flag.data_ptr(), 5, result.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert result.item() == 1 and cuda.read_error() == 0
