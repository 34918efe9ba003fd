"""Speculative decoding through the engine is lossless: with MTP draft layers (DeepSeek next-n) or the n-gram trie the
greedy outputs equal plain decoding token for token, and drafts are really proposed / verified."""
import pytest
import torch

from ksanallm_b200.config.model_config import model_config_from_dict, tiny_llama_config
from ksanallm_b200.config.schema import parse_serving_config
from ksanallm_b200.engine.llm_engine import LLMEngine
from ksanallm_b200.engine.sampling_params import SamplingParams
from ksanallm_b200.models.loader import load_model_weights
from ksanallm_b200.models.transformer import TransformerModel


def _serving(**bs):
    return parse_serving_config({"setting": {"batch_scheduler": dict(
        {"max_batch_size": 4, "max_step_tokens": 64, "max_token_len": 160}, **bs),
        "block_manager": {"block_token_num": 16}}})


def _run(cfg, weights, prompts, n, **bs):
    eng = LLMEngine(TransformerModel(cfg, weights), _serving(**bs), num_blocks=64, num_host_blocks=0)
    reqs = eng.generate(prompts, SamplingParams(topk=1, max_new_tokens=n, ignore_eos=True))
    return [r.output_token_ids[0] for r in reqs], eng


def test_mtp_draft_layer_is_lossless():
    cfg = model_config_from_dict(dict(
        model_type="deepseek_v3", hidden_size=128, num_hidden_layers=2, num_attention_heads=4, vocab_size=300,
        intermediate_size=256, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1, moe_intermediate_size=64,
        first_k_dense_replace=1, n_group=4, topk_group=2, norm_topk_prob=True, routed_scaling_factor=2.5,
        q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
        num_nextn_predict_layers=1, torch_dtype="float32", max_position_embeddings=256))
    w = load_model_weights(cfg, synthetic_seed=4, dtype=torch.float32)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 290, (n,), generator=g).tolist() for n in (7, 19, 33)]
    plain, _ = _run(cfg, w, prompts, 12)
    spec, eng = _run(cfg, w, prompts, 12, mtp_step_num=1, enable_speculative_decoding=True)
    assert eng.mtp_steps == 1 and spec == plain
    st = eng.sched.stats
    assert st.draft_proposed > 0 and 0 <= st.draft_accepted <= st.draft_proposed


def test_trie_drafts_are_lossless_and_get_accepted_on_repetitive_text():
    cfg = tiny_llama_config()
    w = load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, dtype=torch.float32)
    prompts = [[11, 12, 13, 14, 15] * 6, [21, 22, 23] * 8 + [21]]
    plain, _ = _run(cfg, w, prompts, 20)
    spec, eng = _run(cfg, w, prompts, 20, enable_speculative_decoding=True)
    assert eng.trie_drafts > 0 and spec == plain
    assert eng.sched.stats.draft_proposed > 0


def test_mtp_drafts_equal_a_plain_forward_of_the_draft_module():
    """The drafts the engine proposes (chunked prefill, then decode steps with verification) equal what the next-n
    module yields when main model and module are simply run over the whole sequence so far."""
    from ksanallm_b200.engine.step_input import make_step_input
    from ksanallm_b200 import ops
    cfg = model_config_from_dict(dict(
        model_type="deepseek_v3", hidden_size=128, num_hidden_layers=2, num_attention_heads=4, vocab_size=300,
        intermediate_size=256, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1, moe_intermediate_size=64,
        first_k_dense_replace=1, n_group=4, topk_group=2, norm_topk_prob=True, routed_scaling_factor=2.5,
        q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
        num_nextn_predict_layers=1, torch_dtype="float32", max_position_embeddings=256))
    w = load_model_weights(cfg, synthetic_seed=4, dtype=torch.float32)
    model = TransformerModel(cfg, w)

    def oracle(tokens):
        """(next token, draft after it) for the sequence ``tokens``."""
        T = len(tokens)
        caches = model.allocate_kv_cache(4, 64)
        meta = make_step_input(tokens, list(range(T)), list(range(T)), [0, T], [T], [[0, 1, 2, 3]], device="cpu")
        h = model.forward(meta, caches)
        nxt_tok = int(model.compute_logits(h, meta.logits_idx)[0].argmax())
        nxt = torch.tensor(tokens[1:] + [nxt_tok], dtype=torch.int32)
        hp = model.mtp_layers[0].forward(ops.embedding(nxt, model.embed, cfg.emb_scale), h, meta, caches[len(model.layers)])
        return nxt_tok, int(model.compute_logits(hp[-1:])[0].argmax())

    eng = LLMEngine(model, _serving(mtp_step_num=1, split_fuse_token_num=8), num_blocks=64, num_host_blocks=0)
    seen = []
    orig = eng._mtp_forward

    def spy(*a):
        d = orig(*a)
        if d is not None:
            seen.append(d.tolist())
        return d

    eng._mtp_forward = spy
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(3, 290, (21,), generator=g).tolist()
    req = eng.add_request(prompt, SamplingParams(topk=1, max_new_tokens=5, ignore_eos=True))
    eng.run_until_done()
    out = req.output_token_ids[0]
    # first draft: after the prompt's last chunk
    t1, d1 = oracle(prompt)
    assert out[0] == t1 and seen[0] == [d1]
    # every later draft follows the tokens accepted so far
    ctx, k = list(prompt), 0
    for drafts in seen:
        nxt_tok, d = oracle(ctx + out[:k])
        while out[k] != nxt_tok:  # (a step that accepted its draft advanced by two tokens)
            k += 1
            nxt_tok, d = oracle(ctx + out[:k])
        assert drafts == [d]
        k += 1
        if k >= len(out):
            break


def _ds_cfg():
    return model_config_from_dict(dict(
        model_type="deepseek_v3", hidden_size=128, num_hidden_layers=2, num_attention_heads=4, vocab_size=300,
        intermediate_size=256, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1, moe_intermediate_size=64,
        first_k_dense_replace=1, n_group=4, topk_group=2, norm_topk_prob=True, routed_scaling_factor=2.5,
        q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
        num_nextn_predict_layers=1, torch_dtype="float32", max_position_embeddings=256))


TP_PROMPTS = [[5, 9, 77, 120, 33, 4, 8], [200, 3, 3, 19, 250, 7, 7, 7, 91, 12, 13], [8, 6, 4]]


def _tp_worker(rank, world, port, out, steps=1):
    import os
    import torch.distributed as dist
    from ksanallm_b200.parallel.comm import TPGroup
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    tp = TPGroup(rank, world, dist.group.WORLD, torch.device("cpu"))
    cfg = _ds_cfg()
    w = load_model_weights(cfg, synthetic_seed=4, tp_rank=rank, tp_size=world, dtype=torch.float32)
    eng = LLMEngine(TransformerModel(cfg, w, tp), _serving(mtp_step_num=steps), tp, num_blocks=64, num_host_blocks=0)
    eng.attach_control_group(dist.group.WORLD)
    if rank == 0:
        reqs = eng.generate(TP_PROMPTS, SamplingParams(topk=1, max_new_tokens=8, ignore_eos=True))
        eng.shutdown_followers()
        out.put(([r.output_token_ids[0] for r in reqs], eng.sched.stats.draft_proposed))
    else:
        eng.follow()
    dist.destroy_process_group()


@pytest.mark.parametrize("steps", [1, 2])
def test_mtp_under_tensor_parallelism_matches_plain_decoding(steps):
    """One draft per step, and two (the second pass's rows reach the follower from the driver)."""
    import socket
    import torch.multiprocessing as mp
    cfg = _ds_cfg()
    w = load_model_weights(cfg, synthetic_seed=4, dtype=torch.float32)
    want, _ = _run(cfg, w, TP_PROMPTS, 8)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q, steps)) for r in range(2)]
    for p in procs:
        p.start()
    got, proposed = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == want and proposed > 0


def test_two_draft_steps_are_lossless_and_the_second_draft_follows_the_chain_rule():
    """mtp_step_num = 2: the module is applied a second time one position further, fed with its own un-normalised
    output and the token it just drafted. Decoding stays exact; the first proposal after the prompt equals a
    hand-written two-step chain."""
    from ksanallm_b200.engine.step_input import make_step_input
    from ksanallm_b200 import ops
    cfg = _ds_cfg()
    w = load_model_weights(cfg, synthetic_seed=4, dtype=torch.float32)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 290, (n,), generator=g).tolist() for n in (7, 19, 33)]
    plain, _ = _run(cfg, w, prompts, 12)
    spec, eng = _run(cfg, w, prompts, 12, mtp_step_num=2)
    assert eng.mtp_steps == 2 and eng.sched_cfg.lookahead_slots == 1 and spec == plain
    assert eng.sched.stats.draft_proposed >= 2 * 3  # two drafts per sequence and step

    model = TransformerModel(cfg, w)
    tokens = prompts[1]
    T = len(tokens)
    caches = model.allocate_kv_cache(4, 64)
    meta = make_step_input(tokens, list(range(T)), list(range(T)), [0, T], [T], [[0, 1, 2, 3]], device="cpu")
    h = model.forward(meta, caches)
    t1 = int(model.compute_logits(h, meta.logits_idx)[0].argmax())
    mtp, mc = model.mtp_layers[0], caches[len(model.layers)]
    nxt = torch.tensor(tokens[1:] + [t1], dtype=torch.int32)
    hp, res = mtp.forward(ops.embedding(nxt, model.embed, cfg.emb_scale), h, meta, mc, return_residual=True)
    d1 = int(model.compute_logits(hp[-1:])[0].argmax())
    m2 = make_step_input([d1], [T], [T], [0, 1], [T + 1], [[0, 1, 2, 3]], device="cpu")
    hp2 = mtp.forward(ops.embedding(m2.input_ids, model.embed, cfg.emb_scale), res[-1:], m2, mc)
    d2 = int(model.compute_logits(hp2)[0].argmax())

    eng2 = LLMEngine(model, _serving(mtp_step_num=2), num_blocks=64, num_host_blocks=0)
    seen = []
    orig = eng2._mtp_chain

    def spy(mtp_, seqs, positions, chains, rows):
        orig(mtp_, seqs, positions, chains, rows)
        seen.append([list(c) for c in chains])

    eng2._mtp_chain = spy
    req = eng2.add_request(tokens, SamplingParams(topk=1, max_new_tokens=3, ignore_eos=True))
    eng2.run_until_done()
    assert req.output_token_ids[0][0] == t1 and seen[0] == [[d1, d2]]


@pytest.mark.parametrize("seed", list(range(int(__import__("os").environ.get("KSANA_FUZZ_SEEDS", "8")))))
def test_mtp_under_memory_pressure_and_staggered_arrivals_is_lossless(seed):
    """One or two MTP drafts per step while the block pool is too small for the batch (recompute or swap
    pre-emption, chunked prefill, look-ahead slots for the second draft), requests arriving between steps: the
    greedy outputs still equal plain decoding, and every block returns to the pool."""
    import random
    rnd = random.Random(seed)
    cfg = _ds_cfg()
    w = load_model_weights(cfg, synthetic_seed=4, dtype=torch.float32)
    g = torch.Generator().manual_seed(50 + seed)
    stem = torch.randint(3, 290, (rnd.choice([16, 24, 32]),), generator=g).tolist()
    prompts = [(stem if rnd.random() < 0.6 else []) + torch.randint(3, 290, (rnd.randint(2, 30),), generator=g).tolist()
               for _ in range(6)]
    params = [SamplingParams(topk=1, max_new_tokens=rnd.randint(4, 30), ignore_eos=True) for _ in prompts]
    model = TransformerModel(cfg, w)
    roomy = LLMEngine(model, _serving(), num_blocks=96, num_host_blocks=0)
    want = [roomy.generate([p], sp)[0].output_token_ids[0] for p, sp in zip(prompts, params)]
    host_blocks = rnd.choice([0, 16])
    eng = LLMEngine(model, _serving(mtp_step_num=rnd.choice([1, 2]), max_batch_size=rnd.choice([3, 6]),
                                    preempt_mode=rnd.choice([0, 1]) if host_blocks else 1,
                                    split_fuse_token_num=rnd.choice([0, 16]),
                                    enable_auto_prefix_cache=rnd.random() < 0.7),
                    num_blocks=rnd.randint(10, 18), num_host_blocks=host_blocks)
    reqs, order = [], list(range(len(prompts)))
    rnd.shuffle(order)
    while order:
        for _ in range(rnd.randint(1, 3)):
            if order:
                i = order.pop()
                reqs.append((i, eng.add_request(prompts[i], params[i])))
        for _ in range(rnd.randint(0, 4)):
            eng.step()
    eng.run_until_done()
    for i, r in reqs:
        assert r.output_token_ids[0] == want[i], (seed, i)
    assert eng.sched.stats.draft_proposed > 0
    assert eng.cache.num_free_blocks + eng.cache.num_cached_blocks == eng.cache.num_device_blocks
