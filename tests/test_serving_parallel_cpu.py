"""The serving entry (KsanaLLMEngine) configured from YAML-style settings for multi-process layouts, on CPU / gloo:
pipeline_para_size = 2 (two stages, two micro-batches) must generate what a single process generates."""
import asyncio
import os
import socket
import time

import pytest
import torch.multiprocessing as mp

from ksanallm_b200.config.schema import parse_serving_config
from ksanallm_b200.serving.ksana_engine import EngineArgs, KsanaLLMEngine

def _free_port() -> int:
    """A rendezvous port below the ephemeral range whose derived ports (+17 request router, +23 control channel) are
    free too: ports handed out by bind(0) sit in the range the kernel also uses for outgoing connections, so a derived
    port could already be some connection's source port."""
    import random
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


BODY = {"input_tokens": [(7 * i + 3) % 200 + 3 for i in range(23)], "stream": False,
        "sampling_config": {"max_new_tokens": 8, "topk": 1, "ignore_eos": True}}


def _serving(**glob):
    sched = {"max_batch_size": 4, "max_step_tokens": 64, "max_token_len": 128, "max_pp_batch_num": 2}
    if glob.pop("balance", False):
        sched["attention_dp_lb_config"] = {"enable_balance": True, "max_waiting_steps": 3,
                                           "max_waiting_time_in_ms": 600000}
    return parse_serving_config({"setting": {"global": glob, "batch_scheduler": sched,
                                             "block_manager": {"block_token_num": 16}}})


def _engine(model="tiny-llama", **glob):
    eng = KsanaLLMEngine(EngineArgs(config_file="", synthetic_model=model, device="cpu", serving=_serving(**glob)))
    eng.initialize()
    return eng


def _bodies(n):
    out = []
    for k in range(n):
        b = dict(BODY)
        b["input_tokens"] = [(t + 11 * k) % 200 + 3 for t in BODY["input_tokens"]][:23 - 3 * k]
        out.append(b)
    return out


def _worker(rank, world, port, out, glob, model="tiny-llama", n=3):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), KSANA_SKIP_WARMUP="1")
    eng = _engine(model, **glob)
    if rank == 0:
        async def run():
            return await asyncio.gather(*[eng.generate(b, streamer=False) for b in _bodies(n)])
        res = asyncio.run(run())
        placed = list(eng.llm.dp_router.placed) if eng.llm.dp_router is not None else []
        out.put(([o.output_tokens[0] for st, o in res if st.OK()], placed))
        eng.shutdown()
    else:
        eng.serve_follower()
    import gc
    import torch.distributed as dist
    del eng
    gc.collect()  # the engine's references to the process groups go first ...
    if dist.is_initialized():
        dist.destroy_process_group()  # ... then the backend's threads are joined before the interpreter goes away


def _spawn(world, glob, model="tiny-llama", n=3):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, glob, model, n)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
    assert [p.exitcode for p in procs] == [0] * world
    return got


def _single(model, n):
    os.environ["KSANA_SKIP_WARMUP"] = "1"
    eng = _engine(model)
    outs = []
    for b in _bodies(n):
        st, out = asyncio.run(eng.generate(b, streamer=False))
        assert st.OK()
        outs.append(out.output_tokens[0])
    eng.shutdown()
    return outs


@pytest.fixture(scope="module")
def want():
    return _single("tiny-llama", 3)


def test_pipeline_stages_from_serving_config(want):
    got, _ = _spawn(2, dict(pipeline_para_size=2, tensor_para_size=1))
    assert got == want


def test_tensor_parallel_from_serving_config(want):
    got, _ = _spawn(2, dict(tensor_para_size=2))
    assert got == want


def test_attention_dp_with_expert_parallel_from_serving_config():
    """Two DP ranks, experts sharded over them; rank 0 owns the front-end and deals the requests by load."""
    want = _single("tiny-moe", 4)
    got, placed = _spawn(2, dict(tensor_para_size=2, attn_data_para_size=2, expert_para_size=2), "tiny-moe", 4)
    assert got == want
    assert placed == [2, 2]


def test_attention_dp_groups_with_tensor_parallel_inside():
    """Four ranks = two DP groups of two tensor-parallel ranks; experts sharded over all four. Each group's leader
    schedules its own requests, its follower hears about every step (also the empty ones) and joins the exchange."""
    want = _single("tiny-moe", 4)
    got, placed = _spawn(4, dict(tensor_para_size=4, attn_data_para_size=2, expert_para_size=4), "tiny-moe", 4)
    assert got == want
    assert placed == [2, 2]


def test_prefill_balancer_between_the_leaders_of_tensor_parallel_dp_groups():
    """attention_dp_lb_config.enable_balance with tensor parallelism inside the DP groups: the leaders agree per step
    on holding new prompts back (a group of their own), the followers just execute; same tokens as without."""
    want = _single("tiny-moe", 4)
    got, placed = _spawn(4, dict(tensor_para_size=4, attn_data_para_size=2, expert_para_size=4, balance=True),
                         "tiny-moe", 4)
    assert got == want
    assert placed == [2, 2]


def _pd_worker(role, rank, world, port, out, transfer_port, peer):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), KSANA_SKIP_WARMUP="1")
    serving = _serving(tensor_para_size=world)
    serving.setting.batch_scheduler.enable_auto_prefix_cache = True
    cs = serving.setting.connector
    cs.group_role, cs.connector_waiting_sec = role, 60
    if role == "decode":
        cs.extra["transfer_port"] = transfer_port
    else:
        cs.extra["peer_transfer_addr"] = peer
    eng = KsanaLLMEngine(EngineArgs(config_file="", synthetic_model="tiny-llama", device="cpu", serving=serving))
    eng.initialize()
    if rank == 0:
        body = dict(BODY, input_tokens=[(5 * i + 1) % 200 + 3 for i in range(40)])
        st, o = asyncio.run(eng.generate(body, streamer=False, req_ctx={"kv-comm-request-id": "tp-pd-1"}))
        hits = eng.llm.cache.stats.prefix_hit_tokens
        out.put((role, st.OK(), o.output_tokens[0] if o is not None else None, hits))
        time.sleep(1.0 if role == "prefill" else 0.0)  # the followers' shards are still on their way
        eng.shutdown()
    else:
        eng.serve_follower()
        out.put((role + "-follower", eng.connector.exported, eng.connector.imported, 0))
    import gc
    import torch.distributed as dist
    del eng
    gc.collect()
    if dist.is_initialized():
        dist.destroy_process_group()


def test_prefill_decode_disaggregation_between_tensor_parallel_instances():
    """A two-rank prefill instance hands a request to a two-rank decode instance: rank 0 of each moves the request
    and its own KV shard, the other ranks move theirs when the message in the plan stream tells them which blocks."""
    import time as _t
    os.environ["KSANA_SKIP_WARMUP"] = "1"
    eng = _engine()
    body = dict(BODY, input_tokens=[(5 * i + 1) % 200 + 3 for i in range(40)])
    st, o = asyncio.run(eng.generate(body, streamer=False))
    eng.shutdown()
    want = o.output_tokens[0]
    ports = []
    while len(ports) < 3:
        c = _free_port()
        if all(abs(c - o) > 64 for o in ports):
            ports.append(c)
    tport = ports[2]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_pd_worker, args=("decode", r, 2, ports[0], q, tport, "")) for r in range(2)]
    procs += [ctx.Process(target=_pd_worker, args=("prefill", r, 2, ports[1], q, 0, f"127.0.0.1:{tport}"))
              for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(4):
        role, a, b, c = q.get(timeout=180)
        got[role] = (a, b, c)
    for p in procs:
        p.join(timeout=60)
    assert [p.exitcode for p in procs] == [0, 0, 0, 0]
    assert got["prefill"][0] and got["decode"][0]
    assert got["prefill"][1] == want[:1] and got["decode"][1] == want
    assert got["decode"][2] >= 32  # the prompt's two full blocks arrived instead of being computed
    assert got["prefill-follower"][0] == 1 and got["decode-follower"][1] == 1


def _hb_worker(rank, world, port, out):
    import threading
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), KSANA_SKIP_WARMUP="1", KSANA_HEARTBEAT_TIMEOUT_S="1.0")
    eng = _engine(tensor_para_size=2)
    if rank == 0:
        st1, _ = asyncio.run(eng.generate(dict(BODY), streamer=False))
        deadline = time.time() + 20
        while not eng.failed_ranks and time.time() < deadline:
            time.sleep(0.1)
        st2, o2 = asyncio.run(eng.generate(dict(BODY), streamer=False))
        out.put((st1.OK(), list(eng.failed_ranks), st2.OK(), st2.GetMessage()))
        eng.shutdown()
    else:
        # a host-side failure: this rank keeps working but falls silent on the control channel
        threading.Timer(1.0, lambda: setattr(eng.control, "paused", True)).start()
        eng.serve_follower()
    import gc
    import torch.distributed as dist
    del eng
    gc.collect()
    if dist.is_initialized():
        dist.destroy_process_group()


def test_a_silent_rank_is_detected_and_new_requests_are_refused():
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_hb_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok1, failed, ok2, msg = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
    assert [p.exitcode for p in procs] == [0, 0]
    assert ok1 and failed == [1] and not ok2 and "gone" in msg


def _fault_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), KSANA_SKIP_WARMUP="1", KSANA_STATUS_CHECK_STEPS="1")
    eng = _engine(tensor_para_size=2)
    if rank == 0:
        st1, _ = asyncio.run(eng.generate(dict(BODY), streamer=False))

        # a fake of the failing call: the read of the device status word finds the peer-timeout bit set, which is
        # what the runner reports after a kernel gave up waiting for a peer
        def status_word_set():
            raise RuntimeError("device status word 0x8: a kernel gave up waiting (peer or barrier timeout)")
        eng.llm.runner.check_device_status = status_word_set
        st2, _ = asyncio.run(eng.generate(dict(BODY), streamer=False))      # in flight when the word is read
        st3, _ = asyncio.run(eng.generate(dict(BODY), streamer=False))      # arrives afterwards
        out.put((st1.OK(), st2.OK(), st2.GetMessage(), st3.OK(), st3.GetMessage(), eng.llm.device_fault))
        eng.shutdown()
    else:
        eng.serve_follower()
    import gc
    import torch.distributed as dist
    del eng
    gc.collect()
    if dist.is_initialized():
        dist.destroy_process_group()


def test_a_set_device_status_word_fails_what_is_in_flight_and_refuses_new_requests():
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_fault_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok1, ok2, msg2, ok3, msg3, fault = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
    assert [p.exitcode for p in procs] == [0, 0]
    assert ok1
    assert not ok2 and "engine step failed" in msg2 and "status word" in msg2
    assert not ok3 and "device fault" in msg3
    assert fault and "0x8" in fault
