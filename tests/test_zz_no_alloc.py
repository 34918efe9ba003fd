"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at all (a latency-critical loop that must not
touch the allocator, or a host program that only passes finished buffers). For them the library exports
``ksana_paged_decode_static``, which keeps its split-KV scratch in a fixed array inside the library. This test
checks that it produces what the regular entry point (caller-provided workspace) produces, twice in a row with
different inputs so that whatever the first call left in the shared array cannot leak into the second result,
and that an oversized problem is refused with an explanation instead of being run.
"""
import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, num_seqs, h, hk, kv_max):
    g = torch.Generator(device="cuda").manual_seed(seed)
    d, bs = 128, 16
    kv_lens = torch.randint(kv_max // 2, kv_max + 1, (num_seqs,), generator=g, device="cuda").tolist()
    nblk = [(L + bs - 1) // bs for L in kv_lens]
    total = sum(nblk) + 1
    cache = (torch.randn(total, 2, hk, bs, d, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    bt = torch.zeros(num_seqs, max(nblk), dtype=torch.int32)
    nxt = 0
    for b in range(num_seqs):
        for j in range(nblk[b]):
            bt[b, j] = nxt
            nxt += 1
    q = (torch.randn(num_seqs, h, d, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    cu = torch.arange(num_seqs + 1, dtype=torch.int32, device="cuda")
    return q, cache, bt.cuda(), cu, torch.tensor(kv_lens, dtype=torch.int32, device="cuda"), max(kv_lens)


def test_static_scratch_entry_matches_workspace_entry():
    from ksanallm_b200.ops import cuda
    lib = cuda.lib()
    fn = lib.ksana_paged_decode_static
    P, I, F = c_void_p, c_int, c_float
    fn.argtypes = [P, I, P, I, P, I, P, P, I, I, I, I, I, I, I, I, F, P, F, F, P, I, P]
    fn.restype = c_int
    lib.ksana_paged_decode_static_error.argtypes = [c_int]
    lib.ksana_paged_decode_static_error.restype = ctypes.c_char_p
    lib.ksana_paged_decode_static_scratch_floats.restype = c_longlong
    cap = lib.ksana_paged_decode_static_scratch_floats()
    assert cap == 2 << 20
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1.0 / 128 ** 0.5
    ws = torch.empty(8 << 20, dtype=torch.float32, device="cuda")

    for seed, (num_seqs, h, hk, kv_max) in enumerate([(3, 8, 8, 2000), (2, 16, 2, 3000)]):
        q, cache, bt, cu, kv_lens, max_kv = _case(seed, num_seqs, h, hk, kv_max)
        out_static = torch.zeros_like(q)
        out_ws = torch.zeros_like(q)
        args = [q.data_ptr(), q.stride(0), cache.data_ptr(), 0, bt.data_ptr(), bt.shape[1], cu.data_ptr(),
                kv_lens.data_ptr(), 0, num_seqs, 1, max_kv, h, hk, 128, 16, scale, None, 1.0, 1.0]
        code = fn(*args, out_static.data_ptr(), out_static.stride(0), stream)
        assert code == 0, lib.ksana_paged_decode_static_error(code).decode()
        code = lib.ksana_paged_decode(*args, out_ws.data_ptr(), out_ws.stride(0), ws.data_ptr(), ws.numel(), stream)
        assert code == 0
        torch.cuda.synchronize()
        err = (out_static.float() - out_ws.float()).abs().max().item()
        assert err <= 2e-2, f"call {seed}: max err {err}"
        assert out_static.float().abs().sum().item() > 0

    # a problem that cannot fit the built-in array is refused, with a message, and nothing runs
    num_seqs, h = 64, 64
    q = torch.zeros(num_seqs, h, 128, dtype=torch.bfloat16, device="cuda")
    cu = torch.arange(num_seqs + 1, dtype=torch.int32, device="cuda")
    kv_lens = torch.full((num_seqs,), 4096, dtype=torch.int32, device="cuda")
    bt = torch.zeros(num_seqs, 256, dtype=torch.int32, device="cuda")
    cache = torch.zeros(2, 2, 1, 16, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros_like(q)
    code = fn(q.data_ptr(), q.stride(0), cache.data_ptr(), 0, bt.data_ptr(), 256, cu.data_ptr(), kv_lens.data_ptr(), 0,
              num_seqs, 1, 4096, h, 1, 128, 16, scale, None, 1.0, 1.0, out.data_ptr(), out.stride(0), stream)
    assert code == -7
    assert b"too large" in lib.ksana_paged_decode_static_error(code)
    torch.cuda.synchronize()
