"""fp8 GEMM with tensor-core-applied power-of-two scales (csrc/cuda/gemm_mxf8.cu) and its quantisation kernels,
against plain PyTorch fp32 references of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _sfa_unpack(sfa, T, K):
    """packed A-scale bytes -> exponent bytes [T_pad, K / 128]"""
    groups = K // 128
    gq = (groups + 3) // 4
    atoms = (T + 127) // 128
    a = sfa.view(atoms, gq, 32, 4, 4)  # [atom, block of 4 groups, r % 32, r / 32, group in block]
    return a.permute(0, 3, 2, 1, 4).reshape(atoms * 128, gq * 4)[:, :groups]


def test_quant_ue8m0_matches_reference():
    from ksanallm_b200.ops import cuda_fp8, reference as ref
    torch.manual_seed(0)
    T, K = 300, 1280  # 10 groups: the last block of 4 is half used
    x = (torch.randn(T, K, device="cuda") * torch.rand(T, 1, device="cuda") * 4).to(torch.bfloat16)
    x[5] = 0
    q, s, sfa = cuda_fp8.quant_fp8_ue8m0(x, scales=True, packed=True)
    q_ref, s_ref = ref.quant_fp8_group(x, ue8m0=True)
    torch.cuda.synchronize()
    assert ref.is_pow2(s)
    nz = torch.ones(T, dtype=torch.bool, device="cuda")
    nz[5] = False  # an all-zero row: any scale is right, the values are zero
    assert torch.equal(s[nz], s_ref[nz])
    assert torch.equal(q.float()[nz], q_ref.float()[nz])
    assert q.float()[5].abs().max().item() == 0
    e = _sfa_unpack(sfa, T, K)
    want = (torch.log2(s).round().to(torch.int32) + 127).to(torch.uint8)
    assert torch.equal(e[:T], want)
    assert (e[T:] == 127).all()


def test_silu_mul_quant_ue8m0_matches_reference():
    from ksanallm_b200.ops import cuda_fp8, reference as ref
    torch.manual_seed(1)
    T, I = 130, 768
    x = torch.randn(T, 2 * I, device="cuda").to(torch.bfloat16)
    q, s, sfa = cuda_fp8.silu_mul_quant_ue8m0(x, scales=True, packed=True)
    act = ref.silu_and_mul(x)
    q_ref, s_ref = ref.quant_fp8_group(act, ue8m0=True)
    torch.cuda.synchronize()
    # __expf against torch's exp: an activation may land on the other side of a bf16 rounding boundary
    dq = (q.float() * s.repeat_interleave(128, 1) - q_ref.float() * s_ref.repeat_interleave(128, 1)).abs()
    assert dq.max().item() <= 0.07 * act.float().abs().max().item()
    assert (s != s_ref).float().mean().item() < 0.01
    e = _sfa_unpack(sfa, T, I)
    assert torch.equal(e[:T], (torch.log2(s).round().to(torch.int32) + 127).to(torch.uint8))


def test_pack_sfb_layout_and_rejects_other_scales():
    from ksanallm_b200.ops import cuda_fp8
    N, K = 520, 768  # 3 tiles of 192 rows, 5 scale rows, 6 k groups (two blocks of 4, the second half used)
    nb, kb = (N + 127) // 128, K // 128
    ex = torch.randint(-12, 3, (nb, kb), device="cuda")
    sw = torch.ldexp(torch.ones(nb, kb, device="cuda"), ex)
    sfb = cuda_fp8.pack_sfb(sw, N, K)
    tiles = (N + 191) // 192
    gq = (kb + 3) // 4
    got = sfb.view(gq, tiles, 2, 32, 4, 4).permute(0, 1, 2, 4, 3, 5).reshape(gq, tiles, 256, 4)  # [block, tile, row, c]
    for nt in range(tiles):
        for r in (0, 31, 32, 127, 128, 191, 192, 255):
            n = nt * 192 + r
            for g in (1, 4, 5):
                want = int(ex[n // 128, g].item()) + 127 if (n < N and r < 192) else 127
                assert int(got[g // 4, nt, r, g % 4]) == want, (nt, r, g)
    with pytest.raises(ValueError):
        cuda_fp8.pack_sfb(sw * 1.5, N, K)


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("M,N,K,bias", [(128, 192, 128, False), (300, 1000, 640, True), (1024, 5120, 5120, False),
                                        (2048, 2560, 6400, True), (77, 200, 256, False), (4000, 1536, 1024, False)])
def test_gemm_mxf8_matches_fp32_reference(M, N, K, bias, variant):
    from ksanallm_b200.ops import cuda, cuda_fp8, reference as ref
    torch.manual_seed(M + N)
    x = (torch.randn(M, K, device="cuda") * (0.25 + 4 * torch.rand(M, 1, device="cuda"))).to(torch.bfloat16)
    w = torch.randn(N, K, device="cuda") * 0.05 * (0.5 + torch.rand(N, 1, device="cuda"))
    wq, sw = ref.quant_fp8_block_weight(w, ue8m0=True)
    b = (torch.randn(N, device="cuda") * 0.5).to(torch.bfloat16) if bias else None
    sfb = cuda_fp8.pack_sfb(sw, N, K)
    xq, xs, sfa = cuda_fp8.quant_fp8_ue8m0(x, scales=True, packed=True)
    y = cuda_fp8.gemm_mxf8(xq, sfa, wq, sfb, b, variant=variant)  # 1: one CTA per tile, 2: CTA pairs
    torch.cuda.synchronize()
    assert cuda.read_error() == 0
    xd = xq.float() * xs.repeat_interleave(128, 1)
    want = xd @ ref.dequant_fp8_block_weight(wq, sw).t()
    if b is not None:
        want = want + b.float()
    err = (y.float() - want).abs().max().item()
    assert err <= 1e-2 * want.abs().max().item(), (err, want.abs().max().item())
    # the kernel with fp32 scales computes the same function from the same operands
    y2 = cuda.gemm_fp8_block(xq, xs, wq, sw, b)
    torch.cuda.synchronize()
    assert (y.float() - y2.float()).abs().max().item() <= 1e-2 * want.abs().max().item()


def test_linear_is_the_same_function_at_every_batch_size():
    from ksanallm_b200.ops import cuda_fp8, reference as ref
    import ksanallm_b200.ops as ops
    torch.manual_seed(9)
    N, K = 1536, 1024
    w = torch.randn(N, K, device="cuda") * 0.03
    wq, sw = ref.quant_fp8_block_weight(w, ue8m0=True)
    sfb = cuda_fp8.pack_sfb(sw, N, K)
    x = torch.randn(cuda_fp8.MXF8_MIN_ROWS + 40, K, device="cuda").to(torch.bfloat16)
    big = ops.linear_fp8_block(x, wq, sw, None, sfb, True)                    # scaled tensor-core kernel
    small = ops.linear_fp8_block(x[:64], wq, sw, None, sfb, True)             # fp32-scale kernel, same quantisation
    want = ref.linear_fp8_block(x, wq, sw, ue8m0=True)
    torch.cuda.synchronize()
    tol = 1e-2 * want.float().abs().max().item()
    assert (big.float() - want.float()).abs().max().item() <= tol
    assert (small.float() - big[:64].float()).abs().max().item() <= tol
