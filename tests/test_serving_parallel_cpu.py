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


def _engine(**glob):
    eng = KsanaLLMEngine(EngineArgs(config_file="", synthetic_model="tiny-llama", device="cpu", serving=_serving(**glob)))
    eng.initialize()
    return eng


def _worker(rank, world, port, out, glob):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), KSANA_SKIP_WARMUP="1")
    eng = _engine(**glob)
    if rank == 0:
        async def run():
            return await asyncio.gather(*[eng.generate(dict(BODY), streamer=False) for _ in range(3)])
        res = asyncio.run(run())
        out.put([o.output_tokens[0] for st, o in res if st.OK()])
        eng.shutdown()
    else:
        eng.serve_follower()


def _spawn(world, glob):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, glob)) for r in range(world)]
    for p in procs:
        p.start()
    got = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return got


@pytest.fixture(scope="module")
def want():
    os.environ["KSANA_SKIP_WARMUP"] = "1"
    eng = _engine()
    st, out = asyncio.run(eng.generate(dict(BODY), streamer=False))
    eng.shutdown()
    assert st.OK()
    return out.output_tokens[0]


def test_pipeline_stages_from_serving_config(want):
    got = _spawn(2, dict(pipeline_para_size=2, tensor_para_size=1))
    assert got == [want, want, want]


def test_tensor_parallel_from_serving_config(want):
    got = _spawn(2, dict(tensor_para_size=2))
    assert got == [want, want, want]
