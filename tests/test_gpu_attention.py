"""Paged attention kernels (tcgen05 prefill, split-KV decode) against the fp32 reference."""
import pytest
import torch

from ksanallm_b200.engine.step_input import make_step_input
from ksanallm_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _setup(q_lens, kv_lens, h, hk, d=128, bs=16, seed=0):
    """Random cache + block tables for sequences with the given new-token and context lengths."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    B = len(q_lens)
    nblk = [(L + bs - 1) // bs for L in kv_lens]
    total = sum(nblk) + 3
    cache = (torch.randn(total, 2, hk, bs, d, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(total, device="cuda", generator=g).tolist()
    maxb = max(nblk) + 2
    bt = torch.zeros(B, maxb, dtype=torch.int32)
    it = iter(perm)
    for b in range(B):
        for j in range(nblk[b]):
            bt[b, j] = next(it)
    T = sum(q_lens)
    q = (torch.randn(T, h, d, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    return q, cache, bt, cu


def _run(q_lens, kv_lens, h, hk, num_prefill, seed=0, tol=2e-2):
    from ksanallm_b200.ops import cuda
    q, cache, bt, cu = _setup(q_lens, kv_lens, h, hk, seed=seed)
    T = q.shape[0]
    meta = make_step_input([0] * T, [0] * T, [0] * T, cu, kv_lens, bt, num_prefill=num_prefill, device="cuda")
    scale = 1.0 / (128 ** 0.5)
    out = cuda.paged_attention(q, cache, meta, scale)
    torch.cuda.synchronize()
    assert cuda.read_error() == 0
    want = ref.paged_attention(q, cache, meta.block_tables, meta.cu_q, meta.kv_lens, scale)
    err = (out.float() - want.float()).abs().max().item()
    assert err < tol, f"max err {err}"


def test_decode_mha():
    _run([1, 1, 1, 1, 1], [1, 17, 160, 1000, 33], h=8, hk=8, num_prefill=0)


def test_decode_gqa():
    _run([1, 1, 1], [300, 5, 2049], h=16, hk=2, num_prefill=0)


def test_decode_multi_token_queries():
    _run([2, 2, 2], [50, 700, 3], h=8, hk=1, num_prefill=0)
    _run([3, 1], [130, 64], h=4, hk=4, num_prefill=0)


@pytest.mark.parametrize("variant", [0, 1])
def test_decode_gqa_tensor_core_kernel_cases(variant):
    """Group sizes 4 / 8 / 16, ragged lengths (short sequences leave KV splits empty), several new tokens per sequence
    (speculative drafts), many sequences (no split) and one long one (many splits). Variant 0: up to 16 query rows
    take the transposed kernel (KV tokens on the MMA rows), more the row kernel; variant 1: always the row kernel."""
    from ksanallm_b200.ops import cuda
    cuda.lib().ksana_paged_decode_gqa_set_variant(variant)
    try:
        _gqa_cases()
    finally:
        cuda.lib().ksana_paged_decode_gqa_set_variant(0)


def _gqa_cases():
    _run([1] * 5, [1, 129, 4000, 16, 700], h=8, hk=2, num_prefill=0, seed=1)
    _run([1] * 3, [5000, 3, 260], h=32, hk=2, num_prefill=0, seed=2)
    _run([4, 2, 3], [900, 131, 4], h=8, hk=1, num_prefill=0, seed=3)
    _run([1] * 200, [37 + 11 * i for i in range(200)], h=8, hk=1, num_prefill=0, seed=4)
    _run([2], [9000], h=16, hk=2, num_prefill=0, seed=5)
    _run([2, 1, 2, 1], [128, 128, 257, 1], h=16, hk=2, num_prefill=0, seed=6)  # tile-boundary lengths
    _run([1] * 64, [2048] * 64, h=64, hk=8, num_prefill=0, seed=7)


def test_decode_long_context_split_kv():
    _run([1], [8000], h=8, hk=8, num_prefill=0)


def test_prefill_single_tile():
    _run([100], [100], h=4, hk=4, num_prefill=1)


def test_prefill_multi_tile_causal():
    _run([300], [300], h=2, hk=2, num_prefill=1)
    _run([513], [513], h=2, hk=1, num_prefill=1)


def test_prefill_with_cached_prefix():
    _run([70], [70 + 256], h=4, hk=2, num_prefill=1)
    _run([200], [200 + 48], h=4, hk=4, num_prefill=1)


def test_prefill_batch_ragged():
    _run([129, 16, 250, 5], [129, 16 + 32, 250, 5 + 400], h=8, hk=2, num_prefill=4)


def test_mixed_prefill_and_decode():
    _run([150, 40, 1, 1, 1], [150, 40 + 64, 77, 1300, 16], h=8, hk=4, num_prefill=2)
