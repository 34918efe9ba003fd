"""Logit parity with the Hugging Face transformers implementations: a tiny randomly initialised HF model's state dict
goes through this repo's config parser, weight loader and paged-KV forward; the last-token logits must agree to fp32
round-off. Covers checkpoint naming (per-expert and stacked expert tensors, packed projections), RoPE flavours,
QK-norm placement, routing rules (softmax / renormalised / DeepSeek grouped sigmoid / Llama-4 input scaling), shared
experts, MLA with absorbed projections and position-free layers."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from ksanallm_b200.config.model_config import model_config_from_dict  # noqa: E402
from ksanallm_b200.engine.step_input import make_step_input  # noqa: E402
from ksanallm_b200.models.loader import WeightLoader  # noqa: E402
from ksanallm_b200.models.transformer import TransformerModel  # noqa: E402

BASE = dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, intermediate_size=256,
            vocab_size=300, max_position_embeddings=64)
DS = dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, intermediate_size=256,
          vocab_size=300, max_position_embeddings=64, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=1,
          moe_intermediate_size=64, first_k_dense_replace=1, n_group=4, topk_group=2, norm_topk_prob=True,
          routed_scaling_factor=2.5, q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8,
          v_head_dim=16)
L4 = dict(hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=32, intermediate_size=64,
          intermediate_size_mlp=256, vocab_size=300, max_position_embeddings=64, num_local_experts=4,
          attention_chunk_size=64)

CASES = {
    "llama": ("LlamaConfig", "LlamaForCausalLM", BASE),
    "llama3_rope": ("LlamaConfig", "LlamaForCausalLM", dict(BASE, rope_scaling=dict(
        rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=32))),
    "llama_linear_rope": ("LlamaConfig", "LlamaForCausalLM", dict(BASE, rope_scaling=dict(rope_type="linear", factor=4.0))),
    "llama_yarn": ("LlamaConfig", "LlamaForCausalLM", dict(BASE, rope_scaling=dict(
        rope_type="yarn", factor=4.0, original_max_position_embeddings=16))),
    "deepseek_v3_yarn": ("DeepseekV3Config", "DeepseekV3ForCausalLM", dict(DS, rope_scaling=dict(
        rope_type="yarn", factor=4.0, original_max_position_embeddings=16, beta_fast=32.0, beta_slow=1.0, mscale=1.0,
        mscale_all_dim=1.0))),
    "qwen2": ("Qwen2Config", "Qwen2ForCausalLM", BASE),
    "qwen3": ("Qwen3Config", "Qwen3ForCausalLM", dict(BASE, head_dim=32)),
    "mistral": ("MistralConfig", "MistralForCausalLM", dict(BASE, sliding_window=None)),
    "mistral_sliding_window": ("MistralConfig", "MistralForCausalLM", dict(BASE, sliding_window=4)),
    "qwen2_mixed_window_layers": ("Qwen2Config", "Qwen2ForCausalLM", dict(
        BASE, num_hidden_layers=3, use_sliding_window=True, sliding_window=5, max_window_layers=1)),
    "mixtral": ("MixtralConfig", "MixtralForCausalLM", dict(BASE, num_local_experts=4, num_experts_per_tok=2)),
    "qwen2_moe": ("Qwen2MoeConfig", "Qwen2MoeForCausalLM", dict(
        BASE, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, shared_expert_intermediate_size=128,
        decoder_sparse_step=1, mlp_only_layers=[])),
    "qwen3_moe": ("Qwen3MoeConfig", "Qwen3MoeForCausalLM", dict(
        BASE, head_dim=32, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=64, decoder_sparse_step=1,
        mlp_only_layers=[], norm_topk_prob=True)),
    "deepseek_v3": ("DeepseekV3Config", "DeepseekV3ForCausalLM", DS),
    "deepseek_v3_rope_halves": ("DeepseekV3Config", "DeepseekV3ForCausalLM", dict(DS, rope_interleave=False,
                                                                                 q_lora_rank=None)),
    "gpt2": ("GPT2Config", "GPT2LMHeadModel", dict(n_embd=64, n_layer=2, n_head=4, n_positions=64, vocab_size=200)),
    "glm4": ("GlmConfig", "GlmForCausalLM", dict(BASE, head_dim=32, pad_token_id=0)),
    "hunyuan_dense": ("HunYuanDenseV1Config", "HunYuanDenseV1ForCausalLM", dict(BASE, head_dim=32)),
    "hunyuan_moe": ("HunYuanMoEV1Config", "HunYuanMoEV1ForCausalLM", dict(
        BASE, head_dim=32, num_experts=4, moe_topk=2, moe_intermediate_size=64)),
    "llama4": ("Llama4TextConfig", "Llama4ForCausalLM", dict(
        L4, num_hidden_layers=4, num_experts_per_tok=1, interleave_moe_layer_step=2, use_qk_norm=True,
        attn_temperature_tuning=True, floor_scale=4, attn_scale=0.3, no_rope_layers=[1, 1, 1, 0])),
    "llama4_top2": ("Llama4TextConfig", "Llama4ForCausalLM", dict(
        L4, num_hidden_layers=2, num_experts_per_tok=2, interleave_moe_layer_step=1, use_qk_norm=False,
        attn_temperature_tuning=False)),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_logits_match_transformers(name):
    cfg_cls, model_cls, kw = CASES[name]
    if not hasattr(transformers, cfg_cls) or not hasattr(transformers, model_cls):
        pytest.skip(f"transformers {transformers.__version__} has no {model_cls}")
    cfg = getattr(transformers, cfg_cls)(**kw)
    torch.manual_seed(0)
    hf = getattr(transformers, model_cls)(cfg).eval().float()
    with torch.no_grad():
        for n, p in hf.named_parameters():  # non-trivial norm weights and biases
            if "norm" in n or n.endswith("bias"):
                p.add_(torch.randn_like(p) * 0.05)
    T = 11
    ids = list(range(5, 5 + T))
    with torch.no_grad():
        want = hf(torch.tensor([ids])).logits[0, -1]
    c = model_config_from_dict(cfg.to_dict())
    w = WeightLoader(c, dtype=torch.float32).load(list(hf.state_dict().items()))
    model = TransformerModel(c, w, max_positions=64)
    meta = make_step_input(ids, list(range(T)), list(range(T)), [0, T], [T], [[0, 1]], device="cpu")
    h = model.forward(meta, model.allocate_kv_cache(2, 64 if c.use_mla else 16))
    got = model.compute_logits(h, meta.logits_idx)[0]
    assert (got - want).abs().max().item() < 1e-4


@pytest.mark.parametrize("name", ["llama", "deepseek_v3", "qwen3_moe", "mistral_sliding_window"])
def test_engine_greedy_generation_matches_transformers(name):
    """Continuous batching over the paged cache (prefill + decode steps, several requests at once) against
    ``generate(do_sample=False)`` of the transformers model, request by request."""
    from ksanallm_b200.config.schema import parse_serving_config
    from ksanallm_b200.engine.llm_engine import LLMEngine
    from ksanallm_b200.engine.sampling_params import SamplingParams
    cfg_cls, model_cls, kw = CASES[name]
    cfg = getattr(transformers, cfg_cls)(**kw)
    torch.manual_seed(1)
    hf = getattr(transformers, model_cls)(cfg).eval().float()
    prompts = [[5, 9, 77, 120, 33, 4, 8], [200, 3, 3, 19, 250, 7, 7, 7, 91, 12, 13, 14, 15, 16, 17, 18, 19, 20], [8, 6]]
    new = 7
    want = []
    for p in prompts:
        with torch.no_grad():
            out = hf.generate(torch.tensor([p]), max_new_tokens=new, do_sample=False, pad_token_id=0, eos_token_id=None)
        want.append(out[0, len(p):].tolist())
    c = model_config_from_dict(cfg.to_dict())
    c.eos_token_ids = []
    w = WeightLoader(c, dtype=torch.float32).load(list(hf.state_dict().items()))
    model = TransformerModel(c, w, max_positions=64)
    serving = parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 4, "max_step_tokens": 16,
                                                                     "max_token_len": 64, "split_fuse_token_num": 16}}})
    eng = LLMEngine(model, serving, num_blocks=32, num_host_blocks=0)
    got = [r.output_token_ids[0] for r in
           eng.generate(prompts, SamplingParams(topk=1, max_new_tokens=new, ignore_eos=True))]
    assert got == want
