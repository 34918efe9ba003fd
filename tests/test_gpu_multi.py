"""Multi-GPU tests (2, 4 or 8 ranks, one process per GPU): fused reduce + residual + RMSNorm + gather kernel over
symmetric memory, with and without the NVLS multicast path, and a tensor-parallel model forward."""
import ctypes
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, use_mc, q):
    import torch.distributed as dist
    from ksanallm_b200.config.model_config import model_config_from_dict
    from ksanallm_b200.engine.step_input import make_step_input
    from ksanallm_b200.models.loader import load_model_weights
    from ksanallm_b200.models.transformer import TransformerModel
    from ksanallm_b200.ops import cuda
    from ksanallm_b200.ops import reference as ref
    from ksanallm_b200.parallel.comm import TPGroup, init_distributed

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    tp = init_distributed("cuda")
    dev = tp.device
    H = 1024
    tp.init_fused(H, 2048, use_multicast=use_mc)
    fc = tp.fused
    report = {"multicast": fc.multicast}
    errs = []
    ll_default = fc.ll_max_tokens
    # every size through the small-step word-flagged kernel (where it applies) and through the reduce kernel
    for ll, T in [(ll_default, t) for t in (1, 7, 64, 300)] + [(0, t) for t in (1, 7, 64)]:
        fc.ll_max_tokens = ll
        g = torch.Generator(device=dev).manual_seed(100 + T)
        parts = [torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16) for _ in range(world)]
        res0 = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(H, device=dev, generator=g)).to(torch.bfloat16)
        total = sum(p.float() for p in parts)
        res_ref = (total + res0.float()).to(torch.bfloat16)
        want = ref.rms_norm(res_ref, w, 1e-6)
        residual = res0.clone()
        out = fc.reduce_add_norm(parts[rank], residual, w, 1e-6).clone()
        torch.cuda.synchronize()
        rows_per = (T + world - 1) // world
        lo, hi = rank * rows_per, min(T, (rank + 1) * rows_per)
        e1 = (out.float() - want.float()).abs().max().item()
        e2 = (residual[lo:hi].float() - res_ref[lo:hi].float()).abs().max().item() if hi > lo else 0.0
        errs.append((T, e1, e2))
        ar = fc.all_reduce(parts[rank])
        torch.cuda.synchronize()
        errs.append((T, (ar.float() - total).abs().max().item() / max(1.0, total.abs().max().item()), 0.0))
    fc.ll_max_tokens = ll_default
    # small-step single kernel: GEMM + word-flagged reduce-scatter + norm + gather
    llerrs = []
    for T, K in ((1, 256), (64, 512), (200, 1024), (256, 384), (33, 2048)) if ll_default else ():
        g = torch.Generator(device=dev).manual_seed(11 * T + K)
        xs = [(torch.randn(T, K, device=dev, generator=g) * 0.5).to(torch.bfloat16) for _ in range(world)]
        wsl = [(torch.randn(H, K, device=dev, generator=g) * 0.05).to(torch.bfloat16) for _ in range(world)]
        res0 = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(H, device=dev, generator=g)).to(torch.bfloat16)
        total = sum((x.float() @ ww.float().t()).to(torch.bfloat16).float() for x, ww in zip(xs, wsl))
        res_ref = (total + res0.float()).to(torch.bfloat16)
        want = ref.rms_norm(res_ref, w, 1e-6)
        residual = res0.clone()
        out = fc.gemm_ll_reduce_add_norm(xs[rank], wsl[rank], residual, w, 1e-6).clone()
        torch.cuda.synchronize()
        rows_per = (T + world - 1) // world
        lo, hi = rank * rows_per, min(T, (rank + 1) * rows_per)
        e1 = (out.float() - want.float()).abs().max().item()
        e2 = (residual[lo:hi].float() - res_ref[lo:hi].float()).abs().max().item() if hi > lo else 0.0
        llerrs.append((T, K, e1, e2))
        out2 = fc.gemm_ll_reduce_add_norm(xs[rank], wsl[rank], res0.clone(), w, 1e-6).clone()
        torch.cuda.synchronize()
        llerrs.append((T, K, 0.0 if torch.equal(out, out2) else 1.0, 0.0))  # deterministic
    # the instantiation for up to 8 ranks (other register array sizes and load batching), run on this many ranks:
    # same sums in the same order, so the same bits
    if ll_default:
        lib = cuda.lib()
        lib.ksana_ll_set_kernel_ranks.argtypes, lib.ksana_ll_set_kernel_ranks.restype = [ctypes.c_int], None
        for T, K in ((64, 512), (256, 384)):
            g = torch.Generator(device=dev).manual_seed(11 * T + K)
            xs = [(torch.randn(T, K, device=dev, generator=g) * 0.5).to(torch.bfloat16) for _ in range(world)]
            wsl = [(torch.randn(H, K, device=dev, generator=g) * 0.05).to(torch.bfloat16) for _ in range(world)]
            res0 = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
            w = (1 + 0.1 * torch.randn(H, device=dev, generator=g)).to(torch.bfloat16)
            base = fc.gemm_ll_reduce_add_norm(xs[rank], wsl[rank], res0.clone(), w, 1e-6).clone()
            r_base = fc.reduce_add_norm((xs[rank].float() @ wsl[rank].float().t()).to(torch.bfloat16), res0.clone(), w,
                                        1e-6).clone()
            torch.cuda.synchronize()
            dist.barrier()
            lib.ksana_ll_set_kernel_ranks(8)
            wide = fc.gemm_ll_reduce_add_norm(xs[rank], wsl[rank], res0.clone(), w, 1e-6).clone()
            r_wide = fc.reduce_add_norm((xs[rank].float() @ wsl[rank].float().t()).to(torch.bfloat16), res0.clone(), w,
                                        1e-6).clone()
            torch.cuda.synchronize()
            dist.barrier()
            lib.ksana_ll_set_kernel_ranks(0)
            llerrs.append((T, K, 0.0 if torch.equal(base, wide) else 1.0, 0.0 if torch.equal(r_base, r_wide) else 1.0))
    report["llerrs"] = llerrs
    # single-kernel GEMM + reduce-scatter + norm + all-gather vs (local GEMMs summed in fp32 -> reference norm)
    ferrs = []
    for T, K in ((1, 256), (64, 512), (300, 1024), (500, 384)):
        g = torch.Generator(device=dev).manual_seed(7 * T + K)
        xs = [(torch.randn(T, K, device=dev, generator=g) * 0.5).to(torch.bfloat16) for _ in range(world)]
        wsl = [(torch.randn(H, K, device=dev, generator=g) * 0.05).to(torch.bfloat16) for _ in range(world)]
        res0 = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(H, device=dev, generator=g)).to(torch.bfloat16)
        total = sum((x.float() @ ww.float().t()).to(torch.bfloat16).float() for x, ww in zip(xs, wsl))
        res_ref = (total + res0.float()).to(torch.bfloat16)
        want = ref.rms_norm(res_ref, w, 1e-6)
        residual = res0.clone()
        out = fc.gemm_reduce_add_norm(xs[rank], wsl[rank], residual, w, 1e-6).clone()
        torch.cuda.synchronize()
        rows_per = (T + world - 1) // world
        lo, hi = rank * rows_per, min(T, (rank + 1) * rows_per)
        e1 = (out.float() - want.float()).abs().max().item()
        e2 = (residual[lo:hi].float() - res_ref[lo:hi].float()).abs().max().item() if hi > lo else 0.0
        ferrs.append((T, K, e1, e2))
        out2 = fc.gemm_reduce_add_norm(xs[rank], wsl[rank], res0.clone(), w, 1e-6).clone()
        torch.cuda.synchronize()
        ferrs.append((T, K, 0.0 if torch.equal(out, out2) else 1.0, 0.0))  # deterministic
    report["ferrs"] = ferrs
    # all-gather -> GEMM: every rank contributes rows_per rows, all ranks get the full product
    aerrs = []
    cap = fc.rows_cap
    for it, (rows_per, T_total, N) in enumerate(((5, 5 * world - 2, 512), (min(128, cap), min(128, cap) * world, 768),
                                                 (min(200, cap), min(200, cap) * world - 37, 256),
                                                 (cap, cap * world, 1024))):
        g = torch.Generator(device=dev).manual_seed(900 + it)
        full = (torch.randn(world * rows_per, H, device=dev, generator=g) * 0.5).to(torch.bfloat16)
        wt = (torch.randn(N, H, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        mine = fc.ag_rows(rows_per)
        mine.copy_(full[rank * rows_per:(rank + 1) * rows_per])
        got = fc.gemm_allgather(rows_per, T_total, wt)
        torch.cuda.synchronize()
        want = full[:T_total].float() @ wt.float().t()
        aerrs.append((rows_per, N, (got.float() - want).abs().max().item(), want.abs().max().item()))
    report["aerrs"] = aerrs
    report["errs"] = errs
    report["kernel_error"] = cuda.read_error()

    # tensor-parallel forward vs the single-rank forward of the same weights
    cfg = model_config_from_dict(dict(model_type="llama", hidden_size=H, num_hidden_layers=2, num_attention_heads=8,
                                      num_key_value_heads=8, intermediate_size=2816, vocab_size=1000,
                                      torch_dtype="bfloat16"))
    w_tp = load_model_weights(cfg, synthetic_seed=3, tp_rank=rank, tp_size=world, device=dev, dtype=torch.bfloat16)
    m_tp = TransformerModel(cfg, w_tp, tp, max_positions=2048)
    T = 40
    ids = list(range(5, 5 + T))
    meta = make_step_input(ids, list(range(T)), list(range(T)), [0, T], [T], [[0, 1, 2, 3]], device=dev)
    kv = m_tp.allocate_kv_cache(8, 16)
    h_tp = m_tp.forward(meta, kv).clone()
    torch.cuda.synchronize()
    report["native"] = m_tp._native_executor() is not None
    # the other row-parallel strategies (small-step kernel off: single fused kernel <-> GEMM + reduce kernel) must agree
    old, old_ll = fc.two_kernel_max_tokens, fc.ll_max_tokens
    alt = 0.0
    for two in (0, 4096):
        fc.ll_max_tokens, fc.two_kernel_max_tokens = 0, two
        h_alt = m_tp.forward(meta, m_tp.allocate_kv_cache(8, 16)).clone()
        torch.cuda.synchronize()
        alt = max(alt, (h_alt.float() - h_tp.float()).abs().max().item())
    fc.two_kernel_max_tokens, fc.ll_max_tokens = old, old_ll
    report["alt_err"] = alt
    # prefill-sized step of three sequences + two decode sequences: two half-batches on two streams (the collectives of
    # one half overlap the compute of the other) against the same step run as one batch
    lens = [500, 420, 380]
    ids2, pos2, slots2, cu2, kvl2, bt2 = [], [], [], [0], [], []
    blk = 0
    for n in lens + [1, 1]:
        ctx = n if n > 1 else 33  # the decode sequences own 32 cached tokens (zeros) + the new one
        nb = (ctx + 15) // 16
        row = list(range(blk, blk + nb))
        first = ctx - n
        ids2 += [7 + (i * 13 + n) % 900 for i in range(n)]
        pos2 += list(range(first, ctx))
        slots2 += [row[p // 16] * 16 + p % 16 for p in range(first, ctx)]
        cu2.append(cu2[-1] + n)
        kvl2.append(ctx)
        bt2.append(row + [0] * (40 - nb))
        blk += nb
    meta2 = make_step_input(ids2, pos2, slots2, cu2, kvl2, bt2, num_prefill=3, device=dev)
    ex = m_tp._native_executor()
    h_ov = m_tp.forward(meta2, m_tp.allocate_kv_cache(blk + 1, 16)).clone()
    torch.cuda.synchronize()
    report["overlap_split"] = int(ex._step.split_seq)
    keep = ex.overlap_min_tokens
    ex.overlap_min_tokens = 1 << 30
    h_one = m_tp.forward(meta2, m_tp.allocate_kv_cache(blk + 1, 16)).clone()
    ex.overlap_min_tokens = keep
    torch.cuda.synchronize()
    report["overlap_err"] = (h_ov.float() - h_one.float()).abs().max().item()
    if rank == 0:
        w_1 = load_model_weights(cfg, synthetic_seed=3, device=dev, dtype=torch.bfloat16)
        m_1 = TransformerModel(cfg, w_1, TPGroup(), max_positions=2048)
        kv1 = m_1.allocate_kv_cache(8, 16)
        h_1 = m_1.forward(meta, kv1)
        torch.cuda.synchronize()
        report["model_err"] = (h_tp.float() - h_1.float()).abs().max().item()
        report["model_ref_max"] = h_1.float().abs().max().item()
        h_1b = m_1.forward(meta2, m_1.allocate_kv_cache(blk + 1, 16))
        torch.cuda.synchronize()
        report["overlap_model_err"] = (h_ov.float() - h_1b.float()).abs().max().item()
        report["overlap_ref_max"] = h_1b.float().abs().max().item()
    # the same two steps with 128 x 128 block-scaled e4m3 weights (the shards cut at block boundaries, so the
    # quantised values equal the single-rank model's): fp8 GEMM into the partial buffer + reduce kernel
    cfg8 = model_config_from_dict(dict(model_type="qwen3", hidden_size=H, num_hidden_layers=2, num_attention_heads=8,
                                       num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=1000,
                                       torch_dtype="bfloat16"))
    w8 = load_model_weights(cfg8, synthetic_seed=5, tp_rank=rank, tp_size=world, device=dev, dtype=torch.bfloat16,
                            quantize="fp8_block")
    m8 = TransformerModel(cfg8, w8, tp, max_positions=2048)
    report["fp8_native"] = m8._native_executor() is not None and m8._native_executor().fp8
    h8 = m8.forward(meta, m8.allocate_kv_cache(8, 16)).clone()
    h8_ov = m8.forward(meta2, m8.allocate_kv_cache(blk + 1, 16)).clone()
    torch.cuda.synchronize()
    report["fp8_overlap_split"] = int(m8._native_executor()._step.split_seq) if report["fp8_native"] else 0
    if rank == 0:
        w8_1 = load_model_weights(cfg8, synthetic_seed=5, device=dev, dtype=torch.bfloat16, quantize="fp8_block")
        m8_1 = TransformerModel(cfg8, w8_1, TPGroup(), max_positions=2048)
        r1 = m8_1.forward(meta, m8_1.allocate_kv_cache(8, 16))
        r2 = m8_1.forward(meta2, m8_1.allocate_kv_cache(blk + 1, 16))
        torch.cuda.synchronize()
        report["fp8_err"] = (h8.float() - r1.float()).abs().max().item()
        report["fp8_overlap_err"] = (h8_ov.float() - r2.float()).abs().max().item()
        report["fp8_mean_err"] = max((h8.float() - r1.float()).abs().mean().item(),
                                     (h8_ov.float() - r2.float()).abs().mean().item())
        report["fp8_ref_max"] = max(r1.float().abs().max().item(), r2.float().abs().max().item())
    dist.barrier()
    report["kernel_error2"] = cuda.read_error()
    if rank == 0:
        q.put(report)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("use_mc", [False, True])
def test_fused_reduce_norm_ranks(use_mc, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, use_mc, q)) for r in range(world)]
    for p in procs:
        p.start()
    rep = None
    import queue
    import time
    deadline = time.time() + 240
    while rep is None and time.time() < deadline:
        try:
            rep = q.get(timeout=2)
        except queue.Empty:
            # a rank that died (assertion, CUDA error) never reports: stop waiting for it
            if any(p.exitcode not in (None, 0) for p in procs):
                break
    if rep is None:
        # The survivors are NOT killed: their device waits are bounded (8 s per kernel) and the process group has
        # a timeout, so they leave by themselves; a rank whose buffers are bound to a multicast object must not be
        # ended in the middle of a kernel.
        for p in procs:
            p.join(timeout=120)
        pytest.fail("a rank exited without reporting: " + str([p.exitcode for p in procs]))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    print(rep)
    assert rep["kernel_error"] == 0 and rep["kernel_error2"] == 0
    # sums of `world` unit-variance terms: one bf16 ulp grows with the magnitude of the sum
    tol = 6e-2 * max(1.0, (world / 2) ** 0.5)
    for T, e1, e2 in rep["errs"]:
        assert e1 < tol and e2 < tol, (T, e1, e2)
    for T, K, e1, e2 in rep["ferrs"] + rep["llerrs"]:
        assert e1 < 8e-2 and e2 < 8e-2, (T, K, e1, e2)
    for rows_per, N, e, m in rep["aerrs"]:
        assert e < 2e-2 * max(1.0, m), (rows_per, N, e, m)
    assert rep["native"]
    assert rep["alt_err"] < 0.05 * max(1.0, rep["model_ref_max"])
    assert rep["model_err"] < 0.05 * max(1.0, rep["model_ref_max"])
    assert rep["overlap_split"] > 0, "the prefill-sized step did not take the two-stream path"
    assert rep["overlap_err"] < 0.05 * max(1.0, rep["overlap_ref_max"])
    assert rep["overlap_model_err"] < 0.05 * max(1.0, rep["overlap_ref_max"])
    assert rep["fp8_native"], "the block-scaled fp8 model did not take the native executor"
    assert rep["fp8_overlap_split"] > 0
    # a bf16 rounding difference in a partial sum can move an activation across an e4m3 rounding boundary of the next
    # layer's quantiser, so single elements differ by up to an fp8 step; the mean shows that nothing else does
    assert rep["fp8_err"] < 0.12 * max(1.0, rep["fp8_ref_max"]), rep
    assert rep["fp8_overlap_err"] < 0.12 * max(1.0, rep["fp8_ref_max"]), rep
    assert rep["fp8_mean_err"] < 0.01 * max(1.0, rep["fp8_ref_max"]), rep
