"""Multi-process layouts of the serving engine on GPUs (NCCL): pipeline stages, attention data parallelism with the
experts exchanged over peer memory, and a prefill -> decode hand-over with the KV leaving layer by layer. The same
layouts run over gloo on CPU in test_serving_parallel_cpu.py / test_pd_serving_cpu.py; here the tiny models run in
bf16 on the device, the pipeline's data channel is NCCL send / recv and the layer tracker waits on CUDA events."""
import asyncio
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BODY = {"input_tokens": [(7 * i + 3) % 200 + 3 for i in range(23)], "stream": False,
        "sampling_config": {"max_new_tokens": 8, "topk": 1, "ignore_eos": True}}


def _serving(**glob):
    from ksanallm_b200.config.schema import parse_serving_config
    return parse_serving_config({"setting": {"global": glob, "batch_scheduler": {
        "max_batch_size": 4, "max_step_tokens": 64, "max_token_len": 128, "max_pp_batch_num": 2},
        "block_manager": {"block_token_num": 16, "block_device_memory_ratio": 0.02}}})


def _engine(model="tiny-llama", **glob):
    from ksanallm_b200.serving.ksana_engine import EngineArgs, KsanaLLMEngine
    eng = KsanaLLMEngine(EngineArgs(config_file="", synthetic_model=model, device="cuda", serving=_serving(**glob)))
    eng.initialize()
    return eng


def _bodies(n):
    out = []
    for k in range(n):
        b = dict(BODY)
        b["input_tokens"] = [(t + 11 * k) % 200 + 3 for t in BODY["input_tokens"]][:23 - 3 * k]
        out.append(b)
    return out


def _worker(rank, world, port, out, glob, model, n):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), KSANA_SKIP_WARMUP="1", NCCL_NVLS_ENABLE="0")
    eng = _engine(model, **glob)
    if rank == 0:
        async def run():
            return await asyncio.gather(*[eng.generate(b, streamer=False) for b in _bodies(n)])
        res = asyncio.run(run())
        placed = list(eng.llm.dp_router.placed) if eng.llm.dp_router is not None else []
        from ksanallm_b200.ops import cuda
        out.put(([o.output_tokens[0] if st.OK() else "error: " + st.GetMessage() for st, o in res], placed,
                 cuda.read_error()))
        eng.shutdown()
    else:
        eng.serve_follower()
    import gc
    import torch.distributed as dist
    del eng
    gc.collect()
    if dist.is_initialized():
        dist.destroy_process_group()


def _free_port() -> int:
    """A rendezvous port below the ephemeral range whose derived ports (+17 request router, +23 control channel) are
    free too (a port from bind(0) has neighbours that outgoing connections may be using)."""
    import random
    import time
    rng = random.Random(os.getpid() * 7919 + int(time.time() * 1000) % 100003)
    for _ in range(200):
        base = rng.randrange(20000, 30000)
        socks = []
        try:
            for off in (0, 17, 23):
                s = socket.socket()
                s.bind(("127.0.0.1", base + off))
                socks.append(s)
            return base
        except OSError:
            continue
        finally:
            for s in socks:
                s.close()
    raise RuntimeError("no free port found")


def _spawn(world, glob, model, n):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, glob, model, n)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=150)
    for p in procs:
        p.join(timeout=60)  # nobody is killed: the process groups have their own timeouts
    assert [p.exitcode for p in procs] == [0] * world
    return got


def _single_worker(out, model, n):
    os.environ["KSANA_SKIP_WARMUP"] = "1"
    eng = _engine(model)
    res = []
    for b in _bodies(n):
        st, o = asyncio.run(eng.generate(b, streamer=False))
        res.append(o.output_tokens[0] if st.OK() else None)
    eng.shutdown()
    out.put(res)


def _single(model, n):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_single_worker, args=(q, model, n))
    p.start()
    got = q.get(timeout=300)
    p.join(timeout=60)
    return got


def test_pipeline_stages_over_nccl():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    want = _single("tiny-llama", 3)
    got, _, status = _spawn(2, dict(pipeline_para_size=2, tensor_para_size=1), "tiny-llama", 3)
    assert status == 0
    assert got == want  # the same kernels over the same values, only cut into two stages


def test_attention_dp_with_expert_exchange_over_peer_memory():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    # "tiny-moe-128": shapes the grouped expert GEMM takes, so the peer-memory exchange (moe_ep.cu) is what runs
    want = _single("tiny-moe-128", 4)
    got, placed, status = _spawn(2, dict(tensor_para_size=2, attn_data_para_size=2, expert_para_size=2),
                                 "tiny-moe-128", 4)
    assert status == 0 and placed == [2, 2]
    assert all(isinstance(g, list) and len(g) == len(w) for g, w in zip(got, want)), (got, want)
    # the exchange sums the experts' outputs in another order than one rank does: in bf16 over random weights a later
    # token may flip, the first one of every request must not
    assert [g[0] for g in got] == [w[0] for w in want]


def _pd_worker(out):
    os.environ["KSANA_SKIP_WARMUP"] = "1"
    os.environ["KSANA_PD_LAYERWISE_WAIT_MS"] = "5000"
    from ksanallm_b200.serving.ksana_engine import EngineArgs, KsanaLLMEngine

    def make(role, **extra):
        args = EngineArgs.from_config_file(os.path.join(ROOT, "examples", "tiny_cpu.yaml"),
                                           synthetic_model="tiny-llama", device="cuda")
        args.serving.setting.block_manager.block_device_memory_ratio = 0.02
        cs = args.serving.setting.connector
        cs.group_role, cs.connector_waiting_sec = role, 60
        cs.extra.update(extra)
        eng = KsanaLLMEngine(args)
        eng.initialize()
        return eng

    body = dict(BODY, input_tokens=[(7 * i + 3) % 200 + 3 for i in range(40)],
                sampling_config={"max_new_tokens": 6, "topk": 1, "ignore_eos": True})
    single = make("none")
    st, want = asyncio.run(single.generate(dict(body), streamer=False))
    single.shutdown()
    decode = make("decode")
    prefill = make("prefill", peer_transfer_addr="%s:%d" % decode.connector.transfer_addr)
    prefill.llm.async_mode = False

    async def both():
        ctx = {"kv-comm-request-id": "g1"}
        d = asyncio.create_task(decode.generate(dict(body), streamer=False, req_ctx=ctx))
        p = asyncio.create_task(prefill.generate(dict(body), streamer=False, req_ctx=ctx))
        return await asyncio.gather(p, d)
    (pst, pout), (dst, dout) = asyncio.run(both())
    from ksanallm_b200.ops import cuda
    out.put(dict(ok=st.OK() and pst.OK() and dst.OK(), want=want.output_tokens, got=dout.output_tokens,
                 first=pout.output_tokens, layerwise=prefill.connector.layerwise_exports,
                 imported=decode.connector.imported, hit=decode.llm.cache.stats.prefix_hit_tokens,
                 status=cuda.read_error()))
    decode.shutdown()
    prefill.shutdown()


def test_prefill_decode_hand_over_layer_by_layer_on_a_gpu():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_pd_worker, args=(q,))
    p.start()
    r = q.get(timeout=300)
    p.join(timeout=60)
    assert r["ok"] and r["status"] == 0
    assert r["got"] == r["want"] and r["first"] == [r["want"][0][:1]]
    assert r["layerwise"] == 1 and r["imported"] == 1 and r["hit"] >= 32
