"""Auxiliary subsystems: GGUF round trip, model cache, memory checker, checksums, EPLB, tracing, config parsing,
weight loaders for several families, registry."""
import json
import os

import torch

from ksanallm_b200.config.model_config import model_config_from_dict
from ksanallm_b200.config.schema import parse_serving_config
from ksanallm_b200.models import gguf_reader, model_cache, registry
from ksanallm_b200.models.loader import WeightLoader, load_model_weights, synthetic_checkpoint
from ksanallm_b200.models.transformer import TransformerModel
from ksanallm_b200.tools.eplb import balance_experts
from ksanallm_b200.utils.memory_checker import BlockChecksumTracker, GuardedBuffer
from ksanallm_b200.utils.tracing import ScheduleEventTracer, summarise_trace


def test_gguf_round_trip(tmp_path):
    t = {"token_embd.weight": torch.randn(8, 4), "blk.0.attn_q.weight": torch.randn(4, 4).to(torch.bfloat16),
         "blk.0.ffn_down.weight": torch.randn(4, 6).half()}
    p = str(tmp_path / "m.gguf")
    gguf_reader.write_gguf(p, t, {"general.architecture": "llama", "llama.block_count": 1})
    meta, back = gguf_reader.read_gguf(p)
    assert meta["general.architecture"] == "llama"
    for k in t:
        assert torch.equal(back[k], t[k])
    names = dict(gguf_reader.iter_gguf(p))
    assert "model.embed_tokens.weight" in names and "model.layers.0.self_attn.q_proj.weight" in names


def test_model_cache_round_trip(tmp_path, monkeypatch):
    monkeypatch.setenv("ENABLE_MODEL_CACHE", "1")
    monkeypatch.setenv("MODEL_CACHE_PATH", str(tmp_path))
    path = model_cache.cache_file("", 0, 2)
    w = {"a.weight": torch.randn(3, 4).to(torch.bfloat16), "b.weight": torch.randn(4, 128).to(torch.float8_e4m3fn)}
    model_cache.save_weights(path, w)
    back = model_cache.load_weights(path)
    assert torch.equal(back["a.weight"], w["a.weight"])
    assert back["b.weight"].dtype == torch.float8_e4m3fn and torch.equal(back["b.weight"].view(torch.uint8), w["b.weight"].view(torch.uint8))


def test_guard_bands_and_checksums():
    g = GuardedBuffer((4, 8), torch.float32)
    g.tensor.fill_(1.0)
    assert g.check()
    g.raw[3] = 0  # an out-of-bounds write in front of the tensor
    assert not g.check()
    kv = torch.randn(6, 2, 1, 4, 8, generator=torch.Generator().manual_seed(0))
    tr = BlockChecksumTracker()
    tr.remember(kv, [1, 3])
    assert tr.verify(kv) == []
    kv[3, 0, 0, 0, 0] += 1.0
    assert tr.verify(kv) == [3]


def test_eplb_balances():
    load = [100, 1, 1, 1, 50, 50, 1, 1]
    r = balance_experts(load, 4)
    assert max(r["rank_load"]) <= 101 and sorted(set(r["rank_of_expert"])) == [0, 1, 2, 3]
    r2 = balance_experts(load, 4, redundant=4)
    assert max(r2["rank_load"]) < max(r["rank_load"]) and "0" in r2["replicas"]


def test_schedule_event_tracer(tmp_path):
    tr = ScheduleEventTracer(rank=0, level=1, directory=str(tmp_path))
    for step in range(3):
        with tr.span("Schedule", step, 4, 128):
            pass
        with tr.span("ForwardingLayers", step, 4, 128):
            pass
    tr.close()
    s = summarise_trace(tr.path, str(tmp_path / "trace.json"))
    assert s["Schedule"]["count"] == 3 and s["ForwardingLayers"]["count"] == 3
    assert len(json.load(open(tmp_path / "trace.json"))["traceEvents"]) == 6


def test_yaml_schema_keeps_reference_keys():
    cfg = parse_serving_config({"setting": {"global": {"tensor_para_size": 8, "attn_data_para_size": 2, "future_key": 1},
                                            "batch_scheduler": {"split_fuse_token_num": 256, "mtp_step_num": 1},
                                            "quantization_config": {"kv_cache": {"dtype": "fp8_e4m3"}}},
                                "model_spec": {"base_model": {"model_dir": "/nope"}}})
    assert cfg.tp == 8 and cfg.attn_dp == 2 and cfg.setting.global_.extra["future_key"] == 1
    assert cfg.setting.batch_scheduler.enable_auto_prefix_cache  # implied by split-fuse
    assert cfg.setting.quantization_config.kv_cache.dtype == "fp8_e4m3"


def _run_family(cfg_dict, rename=None, quantize=None):
    cfg = model_config_from_dict(cfg_dict)
    sd = list(synthetic_checkpoint(cfg, seed=1, dtype=torch.float32))
    if rename:
        sd = [(rename(k), v) for k, v in sd]
    w = WeightLoader(cfg, dtype=torch.float32, quantize=quantize).load(sd)
    from ksanallm_b200.engine.step_input import make_step_input
    model = TransformerModel(cfg, w, max_positions=64)
    T = 9
    meta = make_step_input(list(range(5, 5 + T)), list(range(T)), list(range(T)), [0, T], [T], [[0, 1]], device="cpu")
    bs = 64 if cfg.use_mla else 16
    kv = model.allocate_kv_cache(2, bs)
    h = model.forward(meta, kv)
    logits = model.compute_logits(h, meta.logits_idx)
    assert torch.isfinite(logits).all() and logits.shape == (1, cfg.vocab_size)
    return model, w


def test_model_families_load_and_run():
    base = dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=256,
                vocab_size=300, torch_dtype="float32", max_position_embeddings=64)
    _run_family(dict(base, model_type="llama"))
    _run_family(dict(base, model_type="qwen2"))
    _run_family(dict(base, model_type="qwen3", head_dim=32),
                rename=lambda k: k.replace("query_layernorm", "q_norm").replace("key_layernorm", "k_norm"))
    _run_family(dict(base, model_type="mixtral", num_local_experts=4, num_experts_per_tok=2),
                rename=lambda k: k.replace(".mlp.experts", ".block_sparse_moe.experts").replace(".mlp.gate.", ".block_sparse_moe.gate.")
                .replace("gate_proj", "w1").replace("down_proj", "w2").replace("up_proj", "w3"))
    _run_family(dict(base, model_type="qwen2_moe", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64,
                     shared_expert_intermediate_size=128))
    m, w = _run_family(dict(base, model_type="deepseek_v3", n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1,
                            moe_intermediate_size=64, first_k_dense_replace=1, n_group=4, topk_group=2,
                            scoring_func="sigmoid", topk_method="noaux_tc", norm_topk_prob=True, routed_scaling_factor=2.5,
                            q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                            num_nextn_predict_layers=1),
                       rename=lambda k: k.replace("shared_expert.", "shared_experts."))
    assert "model.layers.0.self_attn.w_uk_t" in w and len(m.mtp_layers) == 1
    # load-time quantisation keeps the model runnable
    _run_family(dict(base, model_type="llama", hidden_size=128, intermediate_size=256), quantize="fp8_block")
    _run_family(dict(base, model_type="llama", hidden_size=128, intermediate_size=256), quantize="int4")


def test_registry():
    assert registry.resolve_family("deepseek_v3") == "deepseek_v3"
    assert registry.resolve_family("Qwen3_MoE".lower()) == "qwen3_moe"
    assert registry.resolve_family("fairseq-transformer") == "gpt2"
    assert registry.resolve_family("totally_unknown") is None


def test_kv_cache_scales_file(tmp_path):
    import json

    import pytest
    import torch

    from ksanallm_b200.config.model_config import model_config_from_dict
    from ksanallm_b200.models.kv_scales import apply_kv_scales, find_kv_scales_file, load_kv_cache_scales
    from ksanallm_b200.models.loader import load_model_weights
    from ksanallm_b200.models.transformer import TransformerModel

    doc = {"model_type": "llama", "kv_cache": {"dtype": "float8_e4m3fn",
                                               "scaling_factor": {"0": {"0": 0.5, "1": 0.25}}}}
    (tmp_path / "kv_cache_scales.json").write_text(json.dumps(doc))
    path = find_kv_scales_file(str(tmp_path))
    assert path is not None
    assert load_kv_cache_scales(path, 1, 3) == [0.5, 0.25, 1.0]  # rank 1 falls back to the rank-0 table
    with pytest.raises(ValueError):
        load_kv_cache_scales(path, 0, 2, expect_model_type="qwen2")
    cfg = model_config_from_dict(dict(model_type="llama", hidden_size=64, num_hidden_layers=2, num_attention_heads=2,
                                      num_key_value_heads=2, intermediate_size=128, vocab_size=100,
                                      torch_dtype="float32"))
    m = TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, dtype=torch.float32))
    apply_kv_scales(m, [0.5, 0.25])
    assert m.layers[0].attn.k_scale == 0.5 and m.layers[1].attn.v_scale == 0.25


def test_gemm_tuning_map(tmp_path):
    from ksanallm_b200.ops import gemm_tune
    p = tmp_path / "map.yaml"
    p.write_text("gemm_bf16:\n  - {n: 4096, k: 4096, m_max: 64, bn: 128, splits: 4}\n"
                 "  - {n: 4096, k: 4096, m_max: 1024, bn: 256, splits: 0}\n")
    assert gemm_tune.load_map(str(p)) == 2
    assert gemm_tune.lookup(16, 4096, 4096) == (128, 4)
    assert gemm_tune.lookup(512, 4096, 4096) == (256, 0)
    assert gemm_tune.lookup(4096, 4096, 4096) == (0, 0) and gemm_tune.lookup(16, 11008, 4096) == (0, 0)
    gemm_tune.clear()
    assert gemm_tune.lookup(16, 4096, 4096) == (0, 0)


def test_logging_levels_categories_and_state_lines(tmp_path):
    import json
    import logging
    from ksanallm_b200.config.model_config import tiny_llama_config
    from ksanallm_b200.config.schema import parse_serving_config
    from ksanallm_b200.engine.llm_engine import LLMEngine
    from ksanallm_b200.engine.sampling_params import SamplingParams
    from ksanallm_b200.models.loader import load_model_weights
    from ksanallm_b200.models.transformer import TransformerModel
    from ksanallm_b200.utils import logger as kl
    kl._configured = False
    logf = tmp_path / "log" / "k.log"
    main = kl.setup_logging("WARNING,SCHEDULER", str(logf))
    assert main.getEffectiveLevel() == logging.WARNING
    assert kl.get_logger("SCHEDULER").getEffectiveLevel() == logging.DEBUG
    assert kl.get_logger("MOE").getEffectiveLevel() == logging.WARNING
    cfg = tiny_llama_config()
    eng = LLMEngine(TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, dtype=torch.float32)),
                    parse_serving_config({"setting": {"batch_scheduler": {"max_token_len": 64}}}), num_blocks=16,
                    num_host_blocks=0)
    eng.generate([[5, 6, 7]], SamplingParams(topk=1, max_new_tokens=3, ignore_eos=True))
    rep = kl.StateReporter(eng, stat_file=str(tmp_path / "stat.jsonl"))
    s = rep.report_once()
    assert s["generated_tokens"] == 3 and s["running"] == 0 and s["blocks_total"] == 16
    assert json.loads((tmp_path / "stat.jsonl").read_text().splitlines()[0])["prompt_tokens"] == 3
    for h in logging.getLogger("ksanallm").handlers:
        h.flush()
    assert "state step=" in logf.read_text()
    logging.getLogger("ksanallm").handlers.clear()
    kl._configured = False


def test_engine_writes_schedule_events(tmp_path, monkeypatch):
    """KLLM_SCHED_TRACE_LEVEL=2: every step's phases and every request's steps appear as Begin / End pairs."""
    from ksanallm_b200.config.model_config import tiny_llama_config
    from ksanallm_b200.config.schema import parse_serving_config
    from ksanallm_b200.engine.llm_engine import LLMEngine
    from ksanallm_b200.engine.sampling_params import SamplingParams
    from ksanallm_b200.models.loader import load_model_weights
    from ksanallm_b200.models.transformer import TransformerModel
    from ksanallm_b200.utils.tracing import summarise_trace
    monkeypatch.setenv("KLLM_SCHED_TRACE_LEVEL", "2")
    monkeypatch.setenv("KLLM_SCHED_TRACE_DIR", str(tmp_path))
    cfg = tiny_llama_config()
    eng = LLMEngine(TransformerModel(cfg, load_model_weights(cfg, synthetic_seed=0, dtype=torch.float32)),
                    parse_serving_config({"setting": {"batch_scheduler": {"max_token_len": 64}}}), num_blocks=16,
                    num_host_blocks=0)
    eng.generate([[5, 6, 7], [8, 9]], SamplingParams(topk=1, max_new_tokens=4, ignore_eos=True))
    eng.tracer.close()
    path = tmp_path / "sched_events_node_0.csv"
    rows = path.read_text().splitlines()
    assert rows[0].startswith("time_ns,node_rank,event,phase")
    events = [r.split(",") for r in rows[1:]]
    names = {e[2] for e in events}
    assert {"Schedule", "PrepareForwarding", "ForwardingLayers", "LmHeadSampling", "UpdateResults",
            "ForwardRequest"} <= names
    for n in names:
        assert sum(e[3] == "B" for e in events if e[2] == n) == sum(e[3] == "E" for e in events if e[2] == n)
    summary = summarise_trace(str(path), str(tmp_path / "trace.json"))
    assert summary["ForwardingLayers"]["count"] == eng.stats["steps"] and (tmp_path / "trace.json").exists()
