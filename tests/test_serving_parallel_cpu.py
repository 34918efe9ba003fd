"""The serving entry (KsanaLLMEngine) configured from YAML-style settings for multi-process layouts, on CPU / gloo:
pipeline_para_size = 2 (two stages, two micro-batches) must generate what a single process generates."""
import asyncio
import os
import socket

import pytest
import torch.multiprocessing as mp

from ksanallm_b200.config.schema import parse_serving_config
from ksanallm_b200.serving.ksana_engine import EngineArgs, KsanaLLMEngine

BODY = {"input_tokens": [(7 * i + 3) % 200 + 3 for i in range(23)], "stream": False,
        "sampling_config": {"max_new_tokens": 8, "topk": 1, "ignore_eos": True}}


def _serving(**glob):
    return parse_serving_config({"setting": {"global": glob, "batch_scheduler": {
        "max_batch_size": 4, "max_step_tokens": 64, "max_token_len": 128, "max_pp_batch_num": 2},
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
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
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
