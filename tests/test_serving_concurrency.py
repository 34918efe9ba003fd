"""Many concurrent clients against one engine (asyncio, the serving loop running in its thread): streaming and
non-streaming requests interleave, some streaming clients go away mid-answer, and under a small block pool every
surviving greedy request still returns what it returns alone; afterwards nothing is left in the engine."""
import asyncio
import os
import random

import pytest

from ksanallm_b200.serving.ksana_engine import EngineArgs, KsanaLLMEngine

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def engine():
    args = EngineArgs.from_config_file(os.path.join(ROOT, "examples", "tiny_cpu.yaml"), synthetic_model="tiny-llama",
                                       device="cpu")
    os.environ["KSANA_SKIP_WARMUP"] = "1"
    eng = KsanaLLMEngine.from_engine_args(args)
    eng.initialize()
    yield eng
    eng.shutdown()


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_concurrent_clients_streaming_aborts_and_results(engine, seed):
    rnd = random.Random(seed)
    n = 28
    prompts = [[rnd.randint(3, 30000) for _ in range(rnd.randint(2, 40))] for _ in range(n)]
    lens = [rnd.randint(2, 24) for _ in range(n)]

    def body(i):
        return {"input_tokens": prompts[i], "sampling_config": {"topk": 1, "max_new_tokens": lens[i], "ignore_eos": True}}

    async def alone(i):
        st, out = await engine.generate(body(i), streamer=False)
        assert st.OK()
        return out.output_tokens[0]

    async def client(i, mode):
        await asyncio.sleep(rnd.random() * 0.05)
        if mode == "plain":
            st, out = await engine.generate(body(i), streamer=False)
            assert st.OK()
            return out.output_tokens[0]
        st, it = await engine.generate(body(i), streamer=True)
        assert st.OK()
        last, seen = None, 0
        async for out in it:
            last, seen = out, seen + 1
            if mode == "leave" and seen >= 2:
                it.abort()
                return None
        return last.output_tokens[0]

    async def main():
        want = [await alone(i) for i in range(n)]
        modes = [rnd.choice(["plain", "stream", "stream", "leave"]) for _ in range(n)]
        got = await asyncio.gather(*[client(i, m) for i, m in enumerate(modes)])
        return want, modes, got

    want, modes, got = asyncio.run(main())
    for i in range(n):
        if modes[i] != "leave" or got[i] is not None:
            assert got[i] == want[i], (seed, i, modes[i])
    llm = engine.llm
    for _ in range(200):  # aborted requests leave at the next step
        if not llm.requests and llm.sched.num_running == 0 and llm.sched.num_waiting == 0:
            break
        import time
        time.sleep(0.02)
    assert not llm.requests and llm.sched.num_running == 0 and llm.sched.num_waiting == 0
    assert llm.cache.num_free_blocks + llm.cache.num_cached_blocks == llm.cache.num_device_blocks
