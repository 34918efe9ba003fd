"""Tensor-parallel engine on CPU (gloo, 2 ranks): the driver rank schedules and broadcasts step plans, the
follower executes its weight shard; generated tokens must equal the single-rank run."""
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


def _cfg():
    return model_config_from_dict(dict(model_type="llama", hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                                       num_key_value_heads=2, intermediate_size=256, vocab_size=500,
                                       torch_dtype="float32", eos_token_id=2))


def _serving(enable_async=False):
    return parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 4, "max_step_tokens": 64,
                                                                 "max_token_len": 128,
                                                                 "enable_async": enable_async}}})


PROMPTS = [[5, 9, 77, 120, 33, 4, 8], [400, 3, 3, 19, 250, 7, 7, 7, 91, 12, 13], [8, 6, 4]]


def _worker(rank, world, port, out, enable_async=False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tp = TPGroup(rank, world, dist.group.WORLD, torch.device("cpu"))
    cfg = _cfg()
    w = load_model_weights(cfg, synthetic_seed=1, tp_rank=rank, tp_size=world, dtype=torch.float32)
    model = TransformerModel(cfg, w, tp)
    eng = LLMEngine(model, _serving(enable_async), tp, num_blocks=64, num_host_blocks=0)
    eng.attach_control_group(dist.group.WORLD)
    if rank == 0:
        reqs = eng.generate(PROMPTS, SamplingParams(topk=1, max_new_tokens=6, ignore_eos=True))
        eng.shutdown_followers()
        out.put([r.output_token_ids[0] for r in reqs])
    else:
        eng.follow()
    dist.destroy_process_group()


import pytest


@pytest.mark.parametrize("enable_async", [False, True])
def test_tp2_matches_single_rank(enable_async):
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
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, enable_async)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == want


def _mm_cfg():
    return model_config_from_dict(dict(model_type="qwen2_vl", hidden_size=128, num_hidden_layers=2,
                                       num_attention_heads=4, num_key_value_heads=2, intermediate_size=256,
                                       vocab_size=500, torch_dtype="float32", eos_token_id=2,
                                       rope_scaling=dict(type="mrope", mrope_section=[4, 6, 6])))


def _mm_request():
    g = torch.Generator().manual_seed(7)
    prompt = [5, 9, 77] + [300] * 20 + [33, 4, 8]
    refit = [(3, torch.randn(20, 128, generator=g) * 0.05)]  # an "image" spanning two prefill chunks
    idx = torch.arange(20)
    img = torch.stack((torch.full((20,), 3), 3 + idx // 5, 3 + idx % 5))
    pos3 = torch.cat((torch.arange(3).expand(3, 3), img, (8 + torch.arange(3)).expand(3, 3)), dim=1)
    return prompt, refit, pos3


def _mm_run(eng):
    prompt, refit, pos3 = _mm_request()
    sp = SamplingParams(topk=1, max_new_tokens=6, ignore_eos=True)
    reqs = [eng.add_request(prompt, sp, refit=refit, mrope_positions=pos3), eng.add_request(PROMPTS[0], sp)]
    eng.run_until_done()
    return [r.output_token_ids[0] for r in reqs]


def _mm_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tp = TPGroup(rank, world, dist.group.WORLD, torch.device("cpu"))
    cfg = _mm_cfg()
    w = load_model_weights(cfg, synthetic_seed=1, tp_rank=rank, tp_size=world, dtype=torch.float32)
    serving = parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 4, "max_step_tokens": 64,
                                                                     "max_token_len": 128, "split_fuse_token_num": 16}}})
    eng = LLMEngine(TransformerModel(cfg, w, tp), serving, tp, num_blocks=64, num_host_blocks=0)
    eng.attach_control_group(dist.group.WORLD)
    if rank == 0:
        out.put(_mm_run(eng))
        eng.shutdown_followers()
    else:
        eng.follow()
    dist.destroy_process_group()


def test_tp2_multimodal_inputs_reach_the_follower():
    """Spliced embeddings and three-axis positions are part of the step plan the driver broadcasts."""
    cfg = _mm_cfg()
    w = load_model_weights(cfg, synthetic_seed=1, dtype=torch.float32)
    serving = parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 4, "max_step_tokens": 64,
                                                                     "max_token_len": 128, "split_fuse_token_num": 16}}})
    want = _mm_run(LLMEngine(TransformerModel(cfg, w), serving, num_blocks=64, num_host_blocks=0))
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_mm_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == want


MIXED = [dict(num_beams=3, num_return_sequences=2, max_new_tokens=5, ignore_eos=True),
         dict(topk=20, topp=0.9, temperature=0.8, seed=11, logprobs=3, repetition_penalty=1.2, max_new_tokens=6,
              ignore_eos=True),
         dict(topk=1, max_new_tokens=6, ignore_eos=True, num_return_sequences=1, frequency_penalty=0.5)]


def _mixed_run(eng):
    reqs = [eng.add_request(p, SamplingParams(**kw)) for p, kw in zip(PROMPTS, MIXED)]
    eng.run_until_done()
    beams = [h.tokens for h in sorted(reqs[0].beam.finished, key=lambda h: -h.score)[:2]]
    lps = [round(e["logprob"], 4) for e in reqs[1].seqs[0].logprobs]
    return beams, reqs[1].output_token_ids[0], lps, reqs[2].output_token_ids[0]


def _mixed_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tp = TPGroup(rank, world, dist.group.WORLD, torch.device("cpu"))
    cfg = _cfg()
    w = load_model_weights(cfg, synthetic_seed=1, tp_rank=rank, tp_size=world, dtype=torch.float32)
    eng = LLMEngine(TransformerModel(cfg, w, tp), _serving(), tp, num_blocks=64, num_host_blocks=0)
    eng.attach_control_group(dist.group.WORLD)
    if rank == 0:
        out.put(_mixed_run(eng))
        eng.shutdown_followers()
    else:
        eng.follow()
    dist.destroy_process_group()


def test_tp2_beam_search_sampling_logprobs_and_penalties_in_one_batch():
    """Beam search (copy-on-write forks), seeded top-k / top-p sampling with log-probs and penalties, and a greedy
    request share steps under tensor parallelism: the follower joins the full-logits path the driver picks."""
    cfg = _cfg()
    w = load_model_weights(cfg, synthetic_seed=1, dtype=torch.float32)
    want = _mixed_run(LLMEngine(TransformerModel(cfg, w), _serving(), num_blocks=64, num_host_blocks=0))
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_mixed_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0] == want[0] and got[1] == want[1] and got[3] == want[3]
    assert all(abs(a - b) < 2e-3 for a, b in zip(got[2], want[2]))


def _pressure_case(seed):
    import random
    rnd = random.Random(seed)
    g = torch.Generator().manual_seed(900 + seed)
    stem = torch.randint(3, 490, (32,), generator=g).tolist()
    prompts = [(stem if rnd.random() < 0.6 else []) + torch.randint(3, 490, (rnd.randint(2, 30),), generator=g).tolist()
               for _ in range(7)]
    kw = []
    for i in range(len(prompts)):
        n = rnd.randint(4, 24)
        kw.append([dict(topk=1, max_new_tokens=n, ignore_eos=True),
                   dict(num_beams=2, num_return_sequences=2, max_new_tokens=n, ignore_eos=True),
                   dict(topk=20, topp=0.9, seed=5 + i, max_new_tokens=n, ignore_eos=True)][i % 3])
    host = rnd.choice([0, 24])
    bs = {"max_batch_size": rnd.choice([4, 6]), "max_step_tokens": 96, "max_token_len": 200,
          "enable_auto_prefix_cache": True, "preempt_mode": rnd.choice([0, 1]) if host else 1,
          "split_fuse_token_num": rnd.choice([0, 24])}
    return prompts, kw, bs, rnd.randint(14, 22), host, rnd


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
    tp = TPGroup(rank, world, dist.group.WORLD, torch.device("cpu"))
    cfg = _cfg()
    prompts, kw, bs, blocks, host, rnd = _pressure_case(seed)
    serving = parse_serving_config({"setting": {"batch_scheduler": bs, "block_manager": {"block_token_num": 16}}})
    w = load_model_weights(cfg, synthetic_seed=1, tp_rank=rank, tp_size=world, dtype=torch.float32)
    eng = LLMEngine(TransformerModel(cfg, w, tp), serving, tp, num_blocks=blocks, num_host_blocks=host)
    eng.attach_control_group(dist.group.WORLD)
    if rank == 0:
        res = _pressure_run(eng, prompts, kw, rnd)
        st = eng.sched.stats
        eng.shutdown_followers()
        out.put((res, st.preempt_swap + st.preempt_recompute))
    else:
        eng.follow()
    dist.destroy_process_group()


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_tp2_under_memory_pressure_matches_a_roomy_single_rank(seed):
    """Followers replay the driver's swap-out / swap-in / copy-on-write block operations: with a block pool that
    forces pre-emption, chunked prefill, beams and seeded sampling arriving between steps, two ranks generate what
    one rank with plenty of blocks generates."""
    cfg = _cfg()
    prompts, kw, bs, _, _, _ = _pressure_case(seed)
    roomy = parse_serving_config({"setting": {"batch_scheduler": dict(bs, split_fuse_token_num=0, preempt_mode=1),
                                              "block_manager": {"block_token_num": 16}}})
    w = load_model_weights(cfg, synthetic_seed=1, dtype=torch.float32)
    want = _pressure_run(LLMEngine(TransformerModel(cfg, w), roomy, num_blocks=200, num_host_blocks=0), prompts, kw)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_pressure_worker, args=(r, 2, port, q, seed)) for r in range(2)]
    for p in procs:
        p.start()
    got, preemptions = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == want
