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
    "deepseek_v2": ("DeepseekV2Config", "DeepseekV2ForCausalLM", dict(
        hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, intermediate_size=256,
        vocab_size=300, max_position_embeddings=64, n_routed_experts=8, num_experts_per_tok=2, n_shared_experts=2,
        moe_intermediate_size=64, first_k_dense_replace=1, topk_method="greedy", norm_topk_prob=False,
        routed_scaling_factor=16.0, q_lora_rank=48, kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8,
        v_head_dim=16)),
    "gpt2": ("GPT2Config", "GPT2LMHeadModel", dict(n_embd=64, n_layer=2, n_head=4, n_positions=64, vocab_size=200)),
    "glm4": ("GlmConfig", "GlmForCausalLM", dict(BASE, head_dim=32, pad_token_id=0)),
    "hunyuan_dense": ("HunYuanDenseV1Config", "HunYuanDenseV1ForCausalLM", dict(BASE, head_dim=32)),
    "hunyuan_moe": ("HunYuanMoEV1Config", "HunYuanMoEV1ForCausalLM", dict(
        BASE, head_dim=32, num_experts=4, moe_topk=2, moe_intermediate_size=64)),
    "llama4": ("Llama4TextConfig", "Llama4ForCausalLM", dict(
        L4, num_hidden_layers=4, num_experts_per_tok=1, interleave_moe_layer_step=2, use_qk_norm=True,
        attn_temperature_tuning=True, floor_scale=4, attn_scale=0.3, no_rope_layers=[1, 1, 1, 0])),
    "glm_moe_dsa_sparse_attention": ("GlmMoeDsaConfig", "GlmMoeDsaForCausalLM", dict(
        DS, mlp_layer_types=["dense", "sparse"], index_topk=4, index_head_dim=16, index_n_heads=4)),
    "llama4_chunked_attention": ("Llama4TextConfig", "Llama4ForCausalLM", dict(
        L4, num_hidden_layers=4, num_experts_per_tok=1, interleave_moe_layer_step=2, use_qk_norm=True,
        attn_temperature_tuning=False, no_rope_layers=[1, 1, 1, 0], attention_chunk_size=4)),
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
    if name.startswith("glm_moe_dsa"):
        # with the fused-kernel attention back-ends this transformers model receives no materialised causal mask and
        # its indexer mask alone would let queries see later keys; the eager path carries the causal mask explicitly
        cfg._attn_implementation = "eager"
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


@pytest.mark.parametrize("name", ["llama", "deepseek_v3", "qwen3_moe", "mistral_sliding_window",
                                  "glm_moe_dsa_sparse_attention"])
def test_engine_greedy_generation_matches_transformers(name):
    """Continuous batching over the paged cache (prefill + decode steps, several requests at once) against
    ``generate(do_sample=False)`` of the transformers model, request by request."""
    from ksanallm_b200.config.schema import parse_serving_config
    from ksanallm_b200.engine.llm_engine import LLMEngine
    from ksanallm_b200.engine.sampling_params import SamplingParams
    cfg_cls, model_cls, kw = CASES[name]
    cfg = getattr(transformers, cfg_cls)(**kw)
    if name.startswith("glm_moe_dsa"):
        cfg._attn_implementation = "eager"  # see test_logits_match_transformers
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


def test_multimodal_rope_matches_qwen2_vl_text_model():
    if not hasattr(transformers, "Qwen2VLTextModel"):
        pytest.skip("no Qwen2VLTextModel in this transformers")
    cfg = transformers.Qwen2VLTextConfig(**dict(BASE, rope_scaling=dict(type="mrope", mrope_section=[4, 6, 6])))
    torch.manual_seed(0)
    hf = transformers.Qwen2VLTextModel(cfg).eval().float()
    T = 11
    ids = list(range(5, 5 + T))
    # an "image" in the middle: temporal position frozen, height / width walking a 2 x 2 grid
    pos3 = torch.tensor([[0, 1, 2, 3, 3, 3, 3, 5, 6, 7, 8],
                         [0, 1, 2, 3, 3, 4, 4, 5, 6, 7, 8],
                         [0, 1, 2, 3, 4, 3, 4, 5, 6, 7, 8]])
    with torch.no_grad():
        want = hf(input_ids=torch.tensor([ids]), position_ids=pos3.unsqueeze(1)).last_hidden_state[0]
    d = cfg.to_dict()
    d["model_type"] = "qwen2_vl"
    c = model_config_from_dict(d)
    assert c.rope_scaling.mrope_section == [4, 6, 6] and c.qkv_bias
    sd = [("model." + k, v) for k, v in hf.state_dict().items()] + [("lm_head.weight", torch.zeros(300, 128))]
    model = TransformerModel(c, WeightLoader(c, dtype=torch.float32).load(sd), max_positions=64)
    meta = make_step_input(ids, list(range(T)), list(range(T)), [0, T], [T], [[0, 1]], device="cpu")
    meta.mrope_positions = pos3
    got = model.forward(meta, model.allocate_kv_cache(2, 16))
    assert (got - want).abs().max().item() < 1e-4


def test_engine_generation_with_multimodal_positions():
    """Prompt with image-like 3-d positions, then greedy decoding: generated tokens continue from max + 1 on all
    three axes (the transformers rule), over chunked prefill and the paged cache."""
    if not hasattr(transformers, "Qwen2VLTextModel"):
        pytest.skip("no Qwen2VLTextModel in this transformers")
    from ksanallm_b200.config.schema import parse_serving_config
    from ksanallm_b200.engine.llm_engine import LLMEngine
    from ksanallm_b200.engine.sampling_params import SamplingParams
    cfg = transformers.Qwen2VLTextConfig(**dict(BASE, rope_scaling=dict(type="mrope", mrope_section=[4, 6, 6])))
    torch.manual_seed(0)
    hf = transformers.Qwen2VLTextModel(cfg).eval().float()
    head = torch.randn(300, 128) * 0.1
    ids = list(range(5, 16))
    pos3 = torch.tensor([[0, 1, 2, 3, 3, 3, 3, 5, 6, 7, 8], [0, 1, 2, 3, 3, 4, 4, 5, 6, 7, 8],
                         [0, 1, 2, 3, 4, 3, 4, 5, 6, 7, 8]])
    # reference: re-run the full sequence every step with explicit positions
    want, seq, p3 = [], list(ids), pos3.clone()
    for _ in range(5):
        with torch.no_grad():
            h = hf(input_ids=torch.tensor([seq]), position_ids=p3.unsqueeze(1)).last_hidden_state[0, -1]
        tok = int((h @ head.t()).argmax())
        want.append(tok)
        seq.append(tok)
        p3 = torch.cat((p3, (p3.max() + 1).view(1, 1).expand(3, 1)), dim=1)
    d = cfg.to_dict()
    d["model_type"] = "qwen2_vl"
    c = model_config_from_dict(d)
    c.eos_token_ids = []
    sd = [("model." + k, v) for k, v in hf.state_dict().items()] + [("lm_head.weight", head)]
    model = TransformerModel(c, WeightLoader(c, dtype=torch.float32).load(sd), max_positions=64)
    serving = parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 2, "max_step_tokens": 16,
                                                                     "max_token_len": 64, "split_fuse_token_num": 4}}})
    eng = LLMEngine(model, serving, num_blocks=16, num_host_blocks=0)
    req = eng.add_request(ids, SamplingParams(topk=1, max_new_tokens=5, ignore_eos=True), mrope_positions=pos3)
    eng.run_until_done()
    assert req.output_token_ids[0] == want


def test_beam_search_matches_transformers():
    """Three beams over a fixed budget without EOS: the hypotheses returned (best first) must equal transformers'
    beam search - the per-step expansion / pruning and the copy-on-write forks keep the right KV for every beam."""
    from ksanallm_b200.config.schema import parse_serving_config
    from ksanallm_b200.engine.llm_engine import LLMEngine
    from ksanallm_b200.engine.sampling_params import SamplingParams
    cfg = transformers.LlamaConfig(**BASE)
    torch.manual_seed(3)
    hf = transformers.LlamaForCausalLM(cfg).eval().float()
    with torch.no_grad():
        hf.lm_head.weight.mul_(8.0)  # sharper distributions: beams differ from greedy and from each other
    prompt = [5, 9, 77, 120, 33, 4, 8, 200, 3]
    new = 6
    with torch.no_grad():
        out = hf.generate(torch.tensor([prompt]), max_new_tokens=new, num_beams=3, num_return_sequences=2,
                          do_sample=False, eos_token_id=None, pad_token_id=0, length_penalty=1.0, early_stopping=False)
        greedy = hf.generate(torch.tensor([prompt]), max_new_tokens=new, do_sample=False, eos_token_id=None,
                             pad_token_id=0)[0, len(prompt):].tolist()
    want = [o[len(prompt):].tolist() for o in out]
    c = model_config_from_dict(cfg.to_dict())
    c.eos_token_ids = []
    model = TransformerModel(c, WeightLoader(c, dtype=torch.float32).load(list(hf.state_dict().items())),
                             max_positions=64)
    serving = parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 8, "max_step_tokens": 32,
                                                                     "max_token_len": 64}}})
    eng = LLMEngine(model, serving, num_blocks=64, num_host_blocks=0)
    req = eng.add_request(prompt, SamplingParams(num_beams=3, num_return_sequences=2, max_new_tokens=new,
                                                 ignore_eos=True, length_penalty=1.0))
    eng.run_until_done()
    got = [h.tokens for h in sorted(req.beam.finished, key=lambda h: -h.score)[:2]]
    assert got == want
    assert want[0] != greedy or want[1] != greedy
