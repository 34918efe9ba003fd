"""Pipeline parallelism on CPU (gloo): layer split, micro-batch controller, and a 2-stage engine whose greedy
output must equal the single-process run."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ksanallm_b200.config.model_config import model_config_from_dict
from ksanallm_b200.config.schema import parse_serving_config
from ksanallm_b200.engine.llm_engine import LLMEngine
from ksanallm_b200.engine.sampling_params import SamplingParams
from ksanallm_b200.models.loader import load_model_weights
from ksanallm_b200.models.transformer import TransformerModel
from ksanallm_b200.parallel.comm import TPGroup
from ksanallm_b200.parallel.pipeline import (BatchState, HiddenChannel, MultiBatchController, PipelineStage,
                                             StageTopology, split_layers)


def test_split_layers():
    assert [list(r) for r in split_layers(5, 2)] == [[0, 1, 2], [3, 4]]
    assert [len(r) for r in split_layers(61, 4)] == [16, 15, 15, 15]
    assert [len(r) for r in split_layers(8, 2, first_stage_offload=2)] == [2, 6]
    r = split_layers(32, 8)
    assert r[0].start == 0 and r[-1].stop == 32 and all(a.stop == b.start for a, b in zip(r, r[1:]))


def test_multi_batch_controller_orders_micro_batches():
    c = MultiBatchController(3)
    assert c.next_runnable() is None
    c.ready(1)
    c.ready(0)
    assert c.next_runnable() == 1
    c.start(1)
    assert c.next_runnable() is None  # one micro-batch owns the device
    c.done(1)
    assert c.state[1] == BatchState.FINISHED and c.next_runnable() == 0
    c.start(0)
    c.collected(1)
    c.ready(1)  # re-scheduled while 0 runs
    c.done(0)
    assert c.wait_turn(1, timeout=1.0)
    c.done(1)
    assert c.history == [1, 0, 1]


def _cfg():
    return model_config_from_dict(dict(model_type="llama", hidden_size=128, num_hidden_layers=4, num_attention_heads=4,
                                       num_key_value_heads=2, intermediate_size=256, vocab_size=500,
                                       torch_dtype="float32", eos_token_id=2))


def _serving():
    return parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 4, "max_step_tokens": 64,
                                                                 "max_token_len": 128}}})


PROMPTS = [[5, 9, 77, 120, 33, 4, 8], [400, 3, 3, 19, 250, 7, 7, 7, 91, 12, 13], [8, 6, 4]]


GREEDY = dict(topk=1, max_new_tokens=6, ignore_eos=True)
SAMPLED = dict(topk=20, topp=0.9, temperature=0.8, repetition_penalty=1.1, seed=1234, max_new_tokens=6, ignore_eos=True)


def _worker(rank, world, port, out, micro_batches=1, sampling=None):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    topo = StageTopology(world, 1, rank)
    cfg = _cfg()
    ranges = split_layers(cfg.num_layers, topo.num_stages)
    w = load_model_weights(cfg, synthetic_seed=1, dtype=torch.float32, layer_range=ranges[topo.stage])
    model = TransformerModel(cfg, w, TPGroup(), layer_range=ranges[topo.stage])
    if not topo.is_last:
        model.norm_w = None  # the next stage normalises
    eng = LLMEngine(model, _serving(), num_blocks=64, num_host_blocks=0)
    eng.attach_control_group(dist.group.WORLD)
    eng.attach_pipeline(PipelineStage(model, topo, HiddenChannel(topo, cfg.hidden_size, torch.float32,
                                                                 torch.device("cpu"))), micro_batches)
    if rank == 0:
        reqs = eng.generate(PROMPTS, SamplingParams(**(sampling or GREEDY)))
        eng.shutdown_followers()
        out.put(([r.output_token_ids[0] for r in reqs], list(getattr(eng, "mbc").history)))
    else:
        eng.follow()
    dist.destroy_process_group()


import pytest


@pytest.mark.parametrize("micro_batches", [1, 2])
def test_pp2_matches_single_process(micro_batches):
    cfg = _cfg()
    w = load_model_weights(cfg, synthetic_seed=1, dtype=torch.float32)
    eng = LLMEngine(TransformerModel(cfg, w), _serving(), num_blocks=64, num_host_blocks=0)
    want = [r.output_token_ids[0] for r in eng.generate(PROMPTS, SamplingParams(topk=1, max_new_tokens=6, ignore_eos=True))]
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, micro_batches)) for r in range(2)]
    for p in procs:
        p.start()
    got, history = q.get(timeout=120)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert got == want
    if micro_batches == 2:
        assert set(history) == {0, 1}, "both micro-batches must have carried work"


@pytest.mark.parametrize("micro_batches", [1, 2])
def test_pp2_seeded_sampling_matches_single_process(micro_batches):
    """Top-k / top-p / temperature / repetition penalty with a per-request seed: the last stage returns the rows'
    logits, the driver samples, and the tokens equal the single-process run with the same seed."""
    cfg = _cfg()
    w = load_model_weights(cfg, synthetic_seed=1, dtype=torch.float32)
    eng = LLMEngine(TransformerModel(cfg, w), _serving(), num_blocks=64, num_host_blocks=0)
    want = [r.output_token_ids[0] for r in eng.generate(PROMPTS, SamplingParams(**SAMPLED))]
    greedy = [r.output_token_ids[0] for r in eng.generate(PROMPTS, SamplingParams(**GREEDY))]
    assert want != greedy
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, micro_batches, SAMPLED)) for r in range(2)]
    for p in procs:
        p.start()
    got, _ = q.get(timeout=120)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert got == want


def _pressure_case(seed):
    import random
    rnd = random.Random(seed)
    g = torch.Generator().manual_seed(1200 + seed)
    stem = torch.randint(3, 490, (32,), generator=g).tolist()
    prompts = [(stem if rnd.random() < 0.6 else []) + torch.randint(3, 490, (rnd.randint(2, 30),), generator=g).tolist()
               for _ in range(8)]
    kw = []
    for i in range(len(prompts)):
        n = rnd.randint(4, 24)
        kw.append([dict(topk=1, max_new_tokens=n, ignore_eos=True),
                   dict(topk=20, topp=0.9, seed=5 + i, max_new_tokens=n, ignore_eos=True),
                   dict(num_beams=2, num_return_sequences=2, max_new_tokens=n, ignore_eos=True)][i % 3])
    host = rnd.choice([0, 24])
    bs = {"max_batch_size": rnd.choice([4, 6]), "max_step_tokens": 96, "max_token_len": 200,
          "enable_auto_prefix_cache": True, "preempt_mode": rnd.choice([0, 1]) if host else 1,
          "split_fuse_token_num": rnd.choice([0, 24]), "pp_multibatch_wb_strategy": rnd.choice([0, 1, 2, 3, 4])}
    return prompts, kw, bs, rnd.randint(16, 24), host, rnd.choice([1, 2, 3]), rnd


def _pressure_run(eng, prompts, kw, rnd=None):
    reqs, order = {}, list(range(len(prompts)))
    while order:
        for _ in range(rnd.randint(1, 3) if rnd else len(order)):
            if order:
                i = order.pop(0)
                reqs[i] = eng.add_request(prompts[i], SamplingParams(**kw[i]))
        for _ in range(rnd.randint(0, 3) if rnd else 0):
            eng.step()
    eng.run_until_done()
    out = []
    for i in range(len(prompts)):
        r = reqs[i]
        out.append([h.tokens for h in sorted(r.beam.finished, key=lambda h: -h.score)[:2]] if r.beam is not None
                   else r.output_token_ids)
    return out


def _pressure_worker(rank, world, port, out, seed):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    topo = StageTopology(world, 1, rank)
    cfg = _cfg()
    prompts, kw, bs, blocks, host, mbs, rnd = _pressure_case(seed)
    serving = parse_serving_config({"setting": {"batch_scheduler": bs, "block_manager": {"block_token_num": 16}}})
    ranges = split_layers(cfg.num_layers, topo.num_stages)
    w = load_model_weights(cfg, synthetic_seed=1, dtype=torch.float32, layer_range=ranges[topo.stage])
    model = TransformerModel(cfg, w, TPGroup(), layer_range=ranges[topo.stage])
    if not topo.is_last:
        model.norm_w = None
    eng = LLMEngine(model, serving, num_blocks=blocks, num_host_blocks=host)
    eng.attach_control_group(dist.group.WORLD)
    eng.attach_pipeline(PipelineStage(model, topo, HiddenChannel(topo, cfg.hidden_size, torch.float32,
                                                                 torch.device("cpu"))), mbs)
    if rank == 0:
        res = _pressure_run(eng, prompts, kw, rnd)
        eng.shutdown_followers()
        out.put(res)
    else:
        eng.follow()
    dist.destroy_process_group()


@pytest.mark.parametrize("seed", [0, 1])
def test_pp2_under_memory_pressure_matches_a_roomy_single_process(seed):
    """Two pipeline stages, one to three micro-batches in flight with a random balancing strategy, a block pool that
    forces pre-emption, chunked prefill, beams and seeded sampling arriving between steps: same results as one
    process with plenty of blocks."""
    cfg = _cfg()
    prompts, kw, bs, _, _, _, _ = _pressure_case(seed)
    roomy = parse_serving_config({"setting": {"batch_scheduler": dict(bs, split_fuse_token_num=0, preempt_mode=1),
                                              "block_manager": {"block_token_num": 16}}})
    w = load_model_weights(cfg, synthetic_seed=1, dtype=torch.float32)
    want = _pressure_run(LLMEngine(TransformerModel(cfg, w), roomy, num_blocks=240, num_host_blocks=0), prompts, kw)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_pressure_worker, args=(r, 2, port, q, seed)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == want
