"""Checkpoint naming conventions of the model families: a synthetic Llama-named checkpoint is re-expressed in each
family's own tensor names / packings and must load into the SAME model (identical hidden states), or - where the
architecture itself differs (GPT-2, ChatGLM) - load and run."""
import torch

from ksanallm_b200.config.model_config import model_config_from_dict
from ksanallm_b200.engine.step_input import make_step_input
from ksanallm_b200.models.loader import WeightLoader, synthetic_checkpoint
from ksanallm_b200.models.transformer import TransformerModel

BASE = dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=256,
            vocab_size=300, torch_dtype="float32", max_position_embeddings=64)


def _hidden(cfg, sd):
    w = WeightLoader(cfg, dtype=torch.float32).load(sd)
    model = TransformerModel(cfg, w, max_positions=64)
    T = 11
    meta = make_step_input(list(range(5, 5 + T)), list(range(T)), list(range(T)), [0, T], [T], [[0, 1]], device="cpu")
    h = model.forward(meta, model.allocate_kv_cache(2, 16))
    logits = model.compute_logits(h, meta.logits_idx)
    assert torch.isfinite(logits).all()
    return h


def _llama_reference(**over):
    cfg = model_config_from_dict(dict(BASE, model_type="llama", **over))
    sd = list(synthetic_checkpoint(cfg, seed=3, dtype=torch.float32))
    return cfg, sd, _hidden(cfg, sd)


def test_baichuan_w_pack():
    cfg, sd, want = _llama_reference(num_key_value_heads=4)
    d = dict(sd)
    out = []
    for k, v in sd:
        if ".q_proj." in k:
            p = k.replace("q_proj", "{}")
            out.append((k.replace("q_proj", "W_pack"), torch.cat([d[p.format(n)] for n in ("q_proj", "k_proj", "v_proj")], 0)))
        elif ".k_proj." in k or ".v_proj." in k:
            continue
        else:
            out.append((k, v))
    got = _hidden(model_config_from_dict(dict(BASE, model_type="baichuan", num_key_value_heads=4)), out)
    assert torch.equal(got, want)


def test_internlm2_wqkv_and_names():
    cfg, sd, want = _llama_reference()
    d = dict(sd)
    hq, hk, hd = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    g = hq // hk
    out = []
    for k, v in sd:
        k2 = (k.replace("model.embed_tokens.", "model.tok_embeddings.").replace("lm_head.", "output.")
              .replace(".self_attn.o_proj.", ".attention.wo.").replace(".mlp.gate_proj.", ".feed_forward.w1.")
              .replace(".mlp.up_proj.", ".feed_forward.w3.").replace(".mlp.down_proj.", ".feed_forward.w2.")
              .replace(".input_layernorm.", ".attention_norm.").replace(".post_attention_layernorm.", ".ffn_norm."))
        if ".q_proj." in k:
            q = d[k].view(hk, g, hd, -1)
            kk = d[k.replace("q_proj", "k_proj")].view(hk, 1, hd, -1)
            vv = d[k.replace("q_proj", "v_proj")].view(hk, 1, hd, -1)
            out.append((k.replace(".self_attn.q_proj.", ".attention.wqkv."),
                        torch.cat((q, kk, vv), 1).reshape((g + 2) * hk * hd, -1)))
        elif ".k_proj." in k or ".v_proj." in k:
            continue
        else:
            out.append((k2, v))
    got = _hidden(model_config_from_dict(dict(BASE, model_type="internlm2")), out)
    assert torch.equal(got, want)


def test_qwen3_and_mixtral_style_renames_are_exact():
    cfg = model_config_from_dict(dict(BASE, model_type="qwen3", head_dim=32))
    sd = list(synthetic_checkpoint(cfg, seed=3, dtype=torch.float32))
    want = _hidden(cfg, sd)
    hf = [(k.replace("query_layernorm", "q_norm").replace("key_layernorm", "k_norm"), v) for k, v in sd]
    assert torch.equal(_hidden(cfg, hf), want)


def test_gpt2_conv1d_learned_positions_layernorm():
    cfg = model_config_from_dict(dict(model_type="gpt2", n_embd=64, n_layer=2, n_head=4, n_positions=64, vocab_size=200,
                                      torch_dtype="float32"))
    assert cfg.position_encoding == "learned" and cfg.norm_type == "layernorm" and not cfg.gated_mlp
    H, I = 64, 256
    g = torch.Generator().manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.05  # noqa: E731
    sd = [("wte.weight", rnd(200, H)), ("wpe.weight", rnd(64, H)), ("ln_f.weight", torch.ones(H)), ("ln_f.bias", torch.zeros(H))]
    for i in range(2):
        p = f"h.{i}."
        sd += [(p + "ln_1.weight", torch.ones(H)), (p + "ln_1.bias", torch.zeros(H)),
               (p + "ln_2.weight", torch.ones(H)), (p + "ln_2.bias", torch.zeros(H)),
               (p + "attn.c_attn.weight", rnd(H, 3 * H)), (p + "attn.c_attn.bias", rnd(3 * H)),
               (p + "attn.c_proj.weight", rnd(H, H)), (p + "attn.c_proj.bias", rnd(H)),
               (p + "mlp.c_fc.weight", rnd(H, I)), (p + "mlp.c_fc.bias", rnd(I)),
               (p + "mlp.c_proj.weight", rnd(I, H)), (p + "mlp.c_proj.bias", rnd(H))]
    h = _hidden(cfg, sd)
    assert h.shape == (11, H)


def test_chatglm_packed_qkv_multi_query_partial_rotary():
    cfg = model_config_from_dict(dict(model_type="chatglm", hidden_size=128, num_layers=2, num_attention_heads=4,
                                      multi_query_attention=True, multi_query_group_num=2, kv_channels=32,
                                      ffn_hidden_size=256, padded_vocab_size=300, seq_length=64, layernorm_epsilon=1e-5,
                                      rmsnorm=True, add_qkv_bias=True, torch_dtype="float32"))
    assert cfg.num_kv_heads == 2 and cfg.rotary_dim == 16 and cfg.rope_interleaved
    H, d, hq, hk, I = 128, 32, 4, 2, 256
    g = torch.Generator().manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g) * 0.05  # noqa: E731
    sd = [("transformer.embedding.word_embeddings.weight", rnd(300, H)),
          ("transformer.encoder.final_layernorm.weight", torch.ones(H)), ("transformer.output_layer.weight", rnd(300, H))]
    for i in range(2):
        p = f"transformer.encoder.layers.{i}."
        sd += [(p + "input_layernorm.weight", torch.ones(H)), (p + "post_attention_layernorm.weight", torch.ones(H)),
               (p + "self_attention.query_key_value.weight", rnd((hq + 2 * hk) * d, H)),
               (p + "self_attention.query_key_value.bias", rnd((hq + 2 * hk) * d)),
               (p + "self_attention.dense.weight", rnd(H, hq * d)),
               (p + "mlp.dense_h_to_4h.weight", rnd(2 * I, H)), (p + "mlp.dense_4h_to_h.weight", rnd(H, I))]
    h = _hidden(cfg, sd)
    assert h.shape == (11, H)


def test_minicpm_scaling_factors():
    cfg = model_config_from_dict(dict(BASE, model_type="minicpm", scale_emb=12, scale_depth=1.4, dim_model_base=64))
    assert cfg.emb_scale == 12 and abs(cfg.residual_scale - 1.4 / (2 ** 0.5)) < 1e-6
    assert abs(cfg.logit_scale - 64 / 128) < 1e-9
    sd = list(synthetic_checkpoint(cfg, seed=3, dtype=torch.float32))
    h = _hidden(cfg, sd)
    plain = _hidden(model_config_from_dict(dict(BASE, model_type="llama")), sd)
    assert not torch.allclose(h, plain)


def test_cross_layer_attention_shares_kv_projections():
    """Hunyuan-Large style CLA: with a share factor of 2 the odd layers have no K / V projections."""
    import dataclasses
    from ksanallm_b200.config.model_config import tiny_llama_config
    from ksanallm_b200.config.schema import parse_serving_config
    from ksanallm_b200.engine.llm_engine import LLMEngine
    from ksanallm_b200.engine.sampling_params import SamplingParams
    from test_tiny_llama_oracle import plain_forward_all
    parsed = model_config_from_dict(dict(BASE, model_type="hunyuan_v1_dense", use_cla=True, cla_share_factor=2))
    assert parsed.cla_share_factor == 2
    cfg = dataclasses.replace(tiny_llama_config(), num_layers=4, cla_share_factor=2)
    sd = dict(synthetic_checkpoint(cfg, seed=5, std=0.02, dtype=torch.float32))
    assert "model.layers.1.self_attn.k_proj.weight" not in sd and "model.layers.2.self_attn.k_proj.weight" in sd
    model = TransformerModel(cfg, WeightLoader(cfg, dtype=torch.float32).load(sd.items()))
    serving = parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 4, "max_step_tokens": 64,
                                                                     "max_token_len": 128, "split_fuse_token_num": 16},
                                                "block_manager": {"block_token_num": 16}}})
    eng = LLMEngine(model, serving, num_blocks=32, num_host_blocks=0)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(3, 31000, (n,), generator=g).tolist() for n in (9, 37)]
    reqs = eng.generate(prompts, SamplingParams(topk=1, max_new_tokens=8, ignore_eos=True))
    for prompt, req in zip(prompts, reqs):
        toks = list(prompt)
        for _ in range(8):
            toks.append(int(plain_forward_all(sd, cfg, toks, cla=2)[-1].argmax()))
        assert req.output_token_ids[0] == toks[len(prompt):]


def test_xd_rope_four_axes():
    """Arc-Hunyuan-Video XD-RoPE: four position axes over quarter sections of the alpha-scaled NTK table."""
    from ksanallm_b200.ops import reference as ref
    cfg = model_config_from_dict(dict(BASE, model_type="hunyuan_v1_dense", use_qk_norm=False,
                                      rope_scaling={"type": "dynamic", "alpha": 1000.0, "factor": 1.0},
                                      xdrope_section=[0.25, 0.25, 0.25, 0.25]))
    assert cfg.rope_scaling.mrope_section == [4, 4, 4, 4] and cfg.rope_scaling.alpha == 1000.0
    rd, T = cfg.head_dim, 9
    table = ref.build_rope_cache(rd, 64, cfg.rope_theta, cfg.rope_scaling)
    pos4 = torch.tensor([[0, 1, 2, 3, 3, 3, 3, 4, 5], [0, 1, 2, 0, 0, 0, 0, 4, 5],
                         [0, 1, 2, 3, 3, 4, 4, 4, 5], [0, 1, 2, 3, 4, 3, 4, 4, 5]])
    rows = ref.mrope_rows(table, pos4, cfg.rope_scaling.mrope_section)
    base = cfg.rope_theta * 1000.0 ** (rd / (rd - 2))
    inv = 1.0 / base ** (torch.arange(rd // 2, dtype=torch.float64) * 2 / rd)
    axis = torch.arange(rd // 2) // 4
    ang = pos4[axis].t().double() * inv  # [T, rd / 2]
    assert torch.allclose(rows, torch.cat((ang.cos(), ang.sin()), -1).float(), atol=1e-6)
    # identical positions on all four axes are ordinary RoPE
    sd = list(synthetic_checkpoint(cfg, seed=3, dtype=torch.float32))
    model = TransformerModel(cfg, WeightLoader(cfg, dtype=torch.float32).load(sd), max_positions=64)
    ids, p = list(range(5, 5 + T)), list(range(T))
    outs = []
    for with_axes in (False, True):
        meta = make_step_input(ids, p, p, [0, T], [T], [[0, 1]], device="cpu")
        if with_axes:
            meta.mrope_positions = torch.tensor([p] * 4)
        outs.append(model.forward(meta, model.allocate_kv_cache(2, 16)))
    assert torch.allclose(outs[0], outs[1], atol=1e-6)
    meta = make_step_input(ids, p, p, [0, T], [T], [[0, 1]], device="cpu")
    meta.mrope_positions = pos4
    assert not torch.allclose(model.forward(meta, model.allocate_kv_cache(2, 16)), outs[0], atol=1e-4)


def test_deepseek_v32_config_enables_the_sparse_attention_indexer():
    cfg = model_config_from_dict(dict(
        model_type="deepseek_v32", hidden_size=128, num_hidden_layers=2, num_attention_heads=4, vocab_size=300,
        intermediate_size=256, q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
        n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, first_k_dense_replace=1,
        index_topk=4, index_n_heads=4, index_head_dim=16, torch_dtype="float32", max_position_embeddings=64))
    assert (cfg.index_topk, cfg.index_n_heads, cfg.index_head_dim) == (4, 4, 16) and cfg.rope_interleaved
    sd = list(synthetic_checkpoint(cfg, seed=3, dtype=torch.float32))
    assert any(k.endswith("indexer.weights_proj.weight") for k, _ in sd)
    w = WeightLoader(cfg, dtype=torch.float32).load(sd)
    model = TransformerModel(cfg, w, max_positions=64)
    assert model.layers[0].attn.index_topk == 4
    cache = model.allocate_kv_cache(2, 16)
    assert cache[0].shape[-1] == 32 + 8 + 16  # latent | rope key | indexer key
    T = 11
    meta = make_step_input(list(range(5, 5 + T)), list(range(T)), list(range(T)), [0, T], [T], [[0, 1]], device="cpu")
    sparse = model.forward(meta, cache)
    for layer in model.layers:
        layer.attn.index_topk = 64  # every key selected: dense attention through the same code path
    dense = model.forward(meta, model.allocate_kv_cache(2, 16))
    assert torch.isfinite(sparse).all() and torch.allclose(sparse[:4], dense[:4], atol=1e-6)  # <= 4 keys: identical
    assert not torch.allclose(sparse[-1], dense[-1], atol=1e-6)


def test_layerwise_reranker_head_through_the_engine():
    """bge-reranker-v2-minicpm-layerwise: the lm_head probe stops after `cutoff_layer` layers, applies the final norm
    and the scoring head of that depth to every prompt row."""
    import base64
    import numpy as np
    from ksanallm_b200.config.schema import parse_serving_config
    from ksanallm_b200.engine.llm_engine import LLMEngine
    from ksanallm_b200.engine.forward_probe import validate_targets
    from ksanallm_b200.engine.sampling_params import SamplingParams
    cfg = model_config_from_dict(dict(BASE, model_type="minicpm", num_hidden_layers=3, scale_emb=2.0, scale_depth=1.4,
                                      dim_model_base=64, start_layer=1, tie_word_embeddings=True))
    assert cfg.reranker_start_layer == 1
    sd = [(k, v) for k, v in synthetic_checkpoint(cfg, seed=3, dtype=torch.float32) if k != "lm_head.weight"]
    g = torch.Generator().manual_seed(0)
    heads = [torch.randn(1, 128, generator=g) for _ in range(3)]
    sd += [(f"lm_head.{i}.linear_head.weight", h) for i, h in enumerate(heads)]
    model = TransformerModel(cfg, WeightLoader(cfg, dtype=torch.float32).load(sd), max_positions=64)
    serving = parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 2, "max_step_tokens": 64,
                                                                     "max_token_len": 64}}})
    eng = LLMEngine(model, serving, num_blocks=8, num_host_blocks=0)
    ids = list(range(5, 16))
    targets = [{"target_name": "lm_head", "cutoff_layer": [2], "token_reduce_mode": "GATHER_ALL"}]
    validate_targets(targets, len(ids))
    req = eng.add_request(ids, SamplingParams(topk=1, max_new_tokens=1, ignore_eos=True), probe=targets)
    eng.run_until_done()
    t = req.probe_result[0]["tensor"]
    got = torch.from_numpy(np.frombuffer(base64.b64decode(t["data"]), dtype=np.float32).reshape(t["shape"]).copy())
    T = len(ids)
    meta = make_step_input(ids, list(range(T)), list(range(T)), [0, T], [T], [[0, 1]], device="cpu")
    h2 = model.forward(meta, model.allocate_kv_cache(2, 64), cutoff_layer=2)
    assert got.shape == (T, 1) and torch.allclose(got, h2 @ heads[1].t(), atol=1e-5)
    h3 = model.forward(meta, model.allocate_kv_cache(2, 64))
    assert not torch.allclose(h2, h3, atol=1e-4)
