"""Attention data parallelism on CPU (gloo, 2 ranks): each rank serves its own requests with its own scheduler and
cache, the routed experts are sharded over the ranks and reached through the exchange; ranks with nothing to do run
mock steps. Outputs must equal a single-process run of the same prompts."""
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
from ksanallm_b200.parallel.attn_dp import DPCoordinator, GatherEPExchange
from ksanallm_b200.parallel.comm import TPGroup


def _cfg():
    return model_config_from_dict(dict(model_type="mixtral", hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                                       num_key_value_heads=2, intermediate_size=96, num_local_experts=4,
                                       num_experts_per_tok=2, vocab_size=300, torch_dtype="float32", eos_token_id=2))


def _serving():
    return parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 4, "max_step_tokens": 64,
                                                                 "max_token_len": 128}}})


PROMPTS = {0: [[5, 9, 77, 120, 33, 4, 8], [8, 6, 4]], 1: [[200, 3, 3, 19, 250, 7, 7, 7, 91, 12, 13, 14, 15, 16]]}
NEW = {0: 9, 1: 3}  # rank 1 finishes early and must keep stepping (mock steps) until rank 0 is done


def _worker(rank, world, port, out, eplb=""):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      EPLB_WEIGHT=eplb)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = _cfg()
    w = load_model_weights(cfg, synthetic_seed=2, dtype=torch.float32, ep_rank=rank, ep_size=world)
    tp = TPGroup()
    tp.ep_rank, tp.ep_size = rank, world
    tp.ep = GatherEPExchange(dist.group.WORLD, rank, world, cfg.num_experts_per_tok, cfg.num_experts)
    model = TransformerModel(cfg, w, tp)
    eng = LLMEngine(model, _serving(), tp, num_blocks=64, num_host_blocks=0)
    eng.attach_dp(DPCoordinator(dist.group.WORLD))
    reqs = [eng.add_request(p, SamplingParams(topk=1, max_new_tokens=NEW[rank], ignore_eos=True)) for p in PROMPTS[rank]]
    steps = eng.run_dp(max_steps=200)
    out.put((rank, [r.output_token_ids[0] for r in reqs], steps, eng.stats.get("mock_steps", 0)))
    dist.barrier()
    dist.destroy_process_group()


import pytest


@pytest.mark.parametrize("placement", [None, [1, 0, 0, 1]])
def test_attention_dp_two_ranks_match_single_process(placement, tmp_path):
    """``placement``: rank of every expert as an expert-load-balancing file gives it (experts 1 and 2 on rank 0, 0 and
    3 on rank 1); where the experts live must not change any token."""
    import json
    eplb = ""
    if placement is not None:
        eplb = str(tmp_path / "eplb.json")
        with open(eplb, "w") as f:
            json.dump({f"layer_{i}": {"rank_of_expert": placement} for i in range(2)}, f)
    cfg = _cfg()
    w = load_model_weights(cfg, synthetic_seed=2, dtype=torch.float32)
    want = {}
    for r in (0, 1):
        eng = LLMEngine(TransformerModel(cfg, w), _serving(), num_blocks=64, num_host_blocks=0)
        want[r] = [q.output_token_ids[0] for q in
                   eng.generate(PROMPTS[r], SamplingParams(topk=1, max_new_tokens=NEW[r], ignore_eos=True))]
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, eplb)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict()
    for _ in range(2):
        rank, toks, steps, mocks = q.get(timeout=120)
        got[rank] = (toks, steps, mocks)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0][0] == want[0] and got[1][0] == want[1]
    assert got[0][1] == got[1][1], "ranks must take the same number of steps"
    assert got[1][2] > 0, "the rank that finished first must have run mock steps"


def _balance_worker(rank, world, port, out, max_wait_steps):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = _cfg()
    w = load_model_weights(cfg, synthetic_seed=2, dtype=torch.float32, ep_rank=rank, ep_size=world)
    tp = TPGroup()
    tp.ep_rank, tp.ep_size = rank, world
    tp.ep = GatherEPExchange(dist.group.WORLD, rank, world, cfg.num_experts_per_tok, cfg.num_experts)
    serving = parse_serving_config({"setting": {"batch_scheduler": {
        "max_batch_size": 4, "max_step_tokens": 64, "max_token_len": 128,
        "attention_dp_lb_config": {"enable_balance": True, "max_waiting_steps": max_wait_steps,
                                   "max_waiting_time_in_ms": 600000}}}})
    eng = LLMEngine(TransformerModel(cfg, w, tp), serving, tp, num_blocks=64, num_host_blocks=0)
    eng.attach_dp(DPCoordinator(dist.group.WORLD))
    assert eng.adp_balance is not None
    sp = SamplingParams(topk=1, max_new_tokens=30, ignore_eos=True)
    eng.add_request([5 + rank, 9, 77, 120], sp)          # step 0: both ranks start a prompt together
    second_at = {0: 3, 1: 8}[rank]                        # the second prompt reaches rank 1 five steps later
    prefill_steps, cur = [], [0]
    eng.on_step = lambda info: prefill_steps.append(cur[0]) if info["prefill"] else None
    for step in range(20):
        cur[0] = step
        if step == second_at:
            eng.add_request([40 + rank, 41, 42, 43, 44, 45], sp)
        eng._step_sync()
    out.put((rank, prefill_steps, eng.adp_balance.held_steps, eng.adp_balance.released_by_timeout))
    dist.barrier()
    dist.destroy_process_group()


def _run_balance(max_wait_steps):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_balance_worker, args=(r, 2, port, q, max_wait_steps)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        rank, steps, held, by_timeout = q.get(timeout=120)
        got[rank] = (steps, held, by_timeout)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return got


def test_adp_balance_aligns_prefills_across_ranks():
    got = _run_balance(50)
    # rank 0's second prompt waits until rank 1 has one as well: both prefills run in step 8
    assert got[0][0] == [0, 8] and got[1][0] == [0, 8]
    assert got[0][1] == got[1][1] == 5 and got[0][2] == 0


def test_adp_balance_gives_up_after_max_waiting_steps():
    got = _run_balance(2)
    # held in steps 3 and 4, released by the step limit in step 5; rank 1's prompt then waits for nobody... but
    # rank 0 has nothing waiting at step 8, so rank 1 is held for two steps as well
    assert got[0][0] == [0, 5] and got[1][0] == [0, 10]
    assert got[0][2] == got[1][2] == 2


def test_expert_placement_permutation_and_routing_dump(tmp_path, monkeypatch):
    from ksanallm_b200.tools.eplb import balance_experts, permutation_from_map
    assert permutation_from_map([1, 0, 0, 1], 2) == [2, 0, 1, 3]
    assert sorted(permutation_from_map([0, 0, 0, 1], 2)) == [0, 1, 2, 3]  # an overfull rank spills, still a permutation
    # the loader stores the experts in physical order and leaves the map for the layer
    import json
    path = tmp_path / "eplb.json"
    path.write_text(json.dumps({"layer_0": {"rank_of_expert": [1, 0, 0, 1]}, "layer_1": [5.0, 1.0, 1.0, 5.0]}))
    monkeypatch.setenv("EPLB_WEIGHT", str(path))
    cfg = _cfg()
    full = load_model_weights(cfg, synthetic_seed=2, dtype=torch.float32)
    parts = [load_model_weights(cfg, synthetic_seed=2, dtype=torch.float32, ep_rank=r, ep_size=2) for r in range(2)]
    key = "model.layers.0.mlp.experts.down_proj.weight"
    assert parts[0]["model.layers.0.mlp.expert_perm"].tolist() == [2, 0, 1, 3]
    assert torch.equal(parts[0][key], full[key][[1, 2]]) and torch.equal(parts[1][key], full[key][[0, 3]])
    hot = parts[0]["model.layers.1.mlp.expert_perm"].tolist()  # counts: the two hot experts end up on different ranks
    assert hot[0] // 2 != hot[3] // 2
    assert balance_experts([5.0, 1.0, 1.0, 5.0], 2)["rank_load"] == [6.0, 6.0]
    # routing dump
    monkeypatch.setenv("EPLB_WEIGHT", "")
    monkeypatch.setenv("DUMP_EPLB_PATH", str(tmp_path / "dump"))
    from ksanallm_b200.models import layers
    layers._EPLB_LAYERS.clear()
    eng = LLMEngine(TransformerModel(cfg, full), _serving(), num_blocks=64, num_host_blocks=0)
    eng.generate(PROMPTS[0], SamplingParams(topk=1, max_new_tokens=4, ignore_eos=True))
    out = layers.dump_eplb_counts()
    counts = json.load(open(out))
    n_tok = sum(len(p) for p in PROMPTS[0]) + 2 * 3
    assert set(counts) == {"layer_0", "layer_1"} and sum(counts["layer_0"]) == 2 * n_tok
    layers._EPLB_LAYERS.clear()


def _mtp_dp_worker(rank, world, port, out, drafts=1):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      EPLB_WEIGHT="")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = _mtp_cfg()
    w = load_model_weights(cfg, synthetic_seed=4, dtype=torch.float32, ep_rank=rank, ep_size=world)
    tp = TPGroup()
    tp.ep_rank, tp.ep_size = rank, world
    tp.ep = GatherEPExchange(dist.group.WORLD, rank, world, cfg.num_experts_per_tok, cfg.num_experts)
    serving = parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 4, "max_step_tokens": 64,
                                                                     "max_token_len": 128, "mtp_step_num": drafts}}})
    eng = LLMEngine(TransformerModel(cfg, w, tp), serving, tp, num_blocks=64, num_host_blocks=0)
    eng.attach_dp(DPCoordinator(dist.group.WORLD))
    assert eng.mtp_steps == drafts
    reqs = [eng.add_request(p, SamplingParams(topk=1, max_new_tokens=NEW[rank], ignore_eos=True)) for p in PROMPTS[rank]]
    steps = eng.run_dp(max_steps=200)
    out.put((rank, [r.output_token_ids[0] for r in reqs], steps, eng.sched.stats.draft_proposed))
    dist.barrier()
    dist.destroy_process_group()


def _mtp_cfg():
    return model_config_from_dict(dict(
        model_type="deepseek_v3", hidden_size=128, num_hidden_layers=2, num_attention_heads=4, vocab_size=300,
        intermediate_size=256, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1, moe_intermediate_size=64,
        first_k_dense_replace=1, n_group=4, topk_group=2, norm_topk_prob=True, routed_scaling_factor=2.5,
        q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
        num_nextn_predict_layers=1, torch_dtype="float32", max_position_embeddings=256, eos_token_id=2))


@pytest.mark.parametrize("drafts", [1, 2, 3])
def test_mtp_drafts_under_attention_dp_keep_the_ranks_in_step(drafts):
    """Every pass of the draft module goes through the expert exchange once more per step; a rank that idles (mock
    steps), has no draft rows or ran out of reserved slots joins the others' passes with empty ones. Outputs equal
    single-process decoding without drafts."""
    cfg = _mtp_cfg()
    w = load_model_weights(cfg, synthetic_seed=4, dtype=torch.float32)
    want = {}
    for r in (0, 1):
        eng = LLMEngine(TransformerModel(cfg, w), _serving(), num_blocks=64, num_host_blocks=0)
        want[r] = [q.output_token_ids[0] for q in
                   eng.generate(PROMPTS[r], SamplingParams(topk=1, max_new_tokens=NEW[r], ignore_eos=True))]
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_mtp_dp_worker, args=(r, 2, port, q, drafts)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        rank, toks, steps, proposed = q.get(timeout=120)
        got[rank] = (toks, steps, proposed)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0][0] == want[0] and got[1][0] == want[1]
    assert got[0][1] == got[1][1] and got[0][2] > 0


def _fp8_dp_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      EPLB_WEIGHT="")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = _fp8_cfg()
    w = load_model_weights(cfg, synthetic_seed=2, dtype=torch.float32, quantize="fp8_block", ep_rank=rank, ep_size=world)
    assert w["model.layers.0.mlp.experts.down_proj.weight"].dtype == torch.float8_e4m3fn
    tp = TPGroup()
    tp.ep_rank, tp.ep_size = rank, world
    tp.ep = GatherEPExchange(dist.group.WORLD, rank, world, cfg.num_experts_per_tok, cfg.num_experts)
    eng = LLMEngine(TransformerModel(cfg, w, tp), _serving(), tp, num_blocks=64, num_host_blocks=0)
    eng.attach_dp(DPCoordinator(dist.group.WORLD))
    reqs = [eng.add_request(p, SamplingParams(topk=1, max_new_tokens=NEW[rank], ignore_eos=True)) for p in PROMPTS[rank]]
    eng.run_dp(max_steps=200)
    out.put((rank, [r.output_token_ids[0] for r in reqs]))
    dist.barrier()
    dist.destroy_process_group()


def _fp8_cfg():
    return model_config_from_dict(dict(model_type="mixtral", hidden_size=128, num_hidden_layers=2,
                                       num_attention_heads=4, num_key_value_heads=2, intermediate_size=128,
                                       num_local_experts=4, num_experts_per_tok=2, vocab_size=300,
                                       torch_dtype="float32", eos_token_id=2))


def test_fp8_experts_under_attention_dp_match_single_process():
    """Block-scaled fp8 experts sharded over two DP ranks: the gathered exchange runs each rank's experts through
    the fp8 path; tokens equal a single process holding all (equally quantised) experts."""
    cfg = _fp8_cfg()
    w = load_model_weights(cfg, synthetic_seed=2, dtype=torch.float32, quantize="fp8_block")
    want = {}
    for r in (0, 1):
        eng = LLMEngine(TransformerModel(cfg, w), _serving(), num_blocks=64, num_host_blocks=0)
        want[r] = [q.output_token_ids[0] for q in
                   eng.generate(PROMPTS[r], SamplingParams(topk=1, max_new_tokens=NEW[r], ignore_eos=True))]
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_fp8_dp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0] == want[0] and got[1] == want[1]


def _dp_pressure_case(seed, rank):
    import random
    rnd = random.Random(seed * 10 + rank)
    g = torch.Generator().manual_seed(40 + seed * 10 + rank)
    stem = torch.randint(3, 290, (32,), generator=g).tolist()
    prompts = [(stem if rnd.random() < 0.6 else []) + torch.randint(3, 290, (rnd.randint(2, 30),), generator=g).tolist()
               for _ in range(rnd.randint(2, 6))]
    news = [rnd.randint(3, 22) for _ in prompts]
    host = rnd.choice([0, 16])
    bs = {"max_batch_size": rnd.choice([3, 6]), "max_step_tokens": 96, "max_token_len": 200,
          "enable_auto_prefix_cache": True, "preempt_mode": rnd.choice([0, 1]) if host else 1,
          "split_fuse_token_num": rnd.choice([0, 24])}
    return prompts, news, bs, rnd.randint(9, 14), host, rnd


def _dp_pressure_worker(rank, world, port, out, seed):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = _cfg()
    prompts, news, bs, blocks, host, rnd = _dp_pressure_case(seed, rank)
    serving = parse_serving_config({"setting": {"batch_scheduler": bs, "block_manager": {"block_token_num": 16}}})
    w = load_model_weights(cfg, synthetic_seed=2, dtype=torch.float32, ep_rank=rank, ep_size=world)
    tp = TPGroup()
    tp.ep_rank, tp.ep_size = rank, world
    tp.ep = GatherEPExchange(dist.group.WORLD, rank, world, cfg.num_experts_per_tok, cfg.num_experts)
    eng = LLMEngine(TransformerModel(cfg, w, tp), serving, tp, num_blocks=blocks, num_host_blocks=host)
    eng.attach_dp(DPCoordinator(dist.group.WORLD))
    reqs, order = {}, list(range(len(prompts)))
    for _ in range(8):  # both ranks take the same number of steps; arrivals fall between them
        for _ in range(rnd.randint(0, 2)):
            if order:
                i = order.pop(0)
                reqs[i] = eng.add_request(prompts[i], SamplingParams(topk=1, max_new_tokens=news[i], ignore_eos=True))
        eng._step_sync()
    for i in order:
        reqs[i] = eng.add_request(prompts[i], SamplingParams(topk=1, max_new_tokens=news[i], ignore_eos=True))
    eng.run_dp(max_steps=2000)
    st = eng.sched.stats
    out.put((rank, [reqs[i].output_token_ids[0] for i in range(len(prompts))], st.preempt_swap + st.preempt_recompute))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("seed", [0, 1])
def test_attention_dp_ranks_under_their_own_memory_pressure(seed):
    """Each DP rank has its own small block pool, chunking, pre-emption mode and arrival times; the lock-step exchange
    must keep working while one rank pre-empts, idles or prefills, and every request equals a single-process run."""
    cfg = _cfg()
    w = load_model_weights(cfg, synthetic_seed=2, dtype=torch.float32)
    want = {}
    for r in range(2):
        prompts, news, _, _, _, _ = _dp_pressure_case(seed, r)
        eng = LLMEngine(TransformerModel(cfg, w), _serving(), num_blocks=128, num_host_blocks=0)
        want[r] = [eng.generate([p], SamplingParams(topk=1, max_new_tokens=n, ignore_eos=True))[0].output_token_ids[0]
                   for p, n in zip(prompts, news)]
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_dp_pressure_worker, args=(r, 2, port, q, seed)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        rank, toks, pre = q.get(timeout=240)
        got[rank] = toks
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0] == want[0] and got[1] == want[1]
