"""Token-for-token check of the engine (continuous batching over the paged KV cache) against a plain
PyTorch forward of the same tiny Llama: 2 layers, hidden 256, 4 heads, FFN 688, vocab 32000, fp32."""
import math

import torch

from ksanallm_b200.config.model_config import tiny_llama_config
from ksanallm_b200.config.schema import parse_serving_config
from ksanallm_b200.engine.llm_engine import LLMEngine
from ksanallm_b200.engine.sampling_params import SamplingParams
from ksanallm_b200.models.loader import load_model_weights, synthetic_checkpoint
from ksanallm_b200.models.transformer import TransformerModel


def plain_forward(sd, cfg, tokens):
    """Dense causal forward with HF-named weights; returns logits of the last position."""
    return plain_forward_all(sd, cfg, tokens)[-1]


def plain_forward_all(sd, cfg, tokens, cla=0):
    """Dense causal forward with HF-named weights; returns the logits of every position. ``cla``: cross-layer
    attention, layers with ``i % cla != 0`` attend over the K / V projections of the last layer that has them."""
    H, nh, d = cfg.hidden_size, cfg.num_heads, cfg.head_dim
    x = sd["model.embed_tokens.weight"][tokens]
    T = len(tokens)
    pos = torch.arange(T, dtype=torch.float32)
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    fr = torch.outer(pos, inv)
    cos, sin = fr.cos()[:, None, :], fr.sin()[:, None, :]

    def norm(v, w):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w

    def rope(v):
        a, b = v[..., : d // 2], v[..., d // 2:]
        return torch.cat((a * cos - b * sin, b * cos + a * sin), -1)

    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        h = norm(x, sd[p + "input_layernorm.weight"])
        q = (h @ sd[p + "self_attn.q_proj.weight"].t()).view(T, nh, d)
        if not (cla and i % cla):
            k_raw = (h @ sd[p + "self_attn.k_proj.weight"].t()).view(T, nh, d)
            v = (h @ sd[p + "self_attn.v_proj.weight"].t()).view(T, nh, d)
        q, k = rope(q), rope(k_raw)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(d)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        a = torch.einsum("hqk,khd->qhd", s.softmax(-1), v).reshape(T, H)
        x = x + a @ sd[p + "self_attn.o_proj.weight"].t()
        h = norm(x, sd[p + "post_attention_layernorm.weight"])
        g = torch.nn.functional.silu(h @ sd[p + "mlp.gate_proj.weight"].t()) * (h @ sd[p + "mlp.up_proj.weight"].t())
        x = x + g @ sd[p + "mlp.down_proj.weight"].t()
    x = norm(x, sd["model.norm.weight"])
    return x @ sd["lm_head.weight"].t()


def test_tiny_llama_greedy_matches_plain_forward():
    cfg = tiny_llama_config()
    sd = dict(synthetic_checkpoint(cfg, seed=0, std=0.02, dtype=torch.float32))
    weights = load_model_weights(cfg, synthetic_seed=0, synthetic_std=0.02, dtype=torch.float32)
    model = TransformerModel(cfg, weights)
    serving = parse_serving_config({"setting": {"batch_scheduler": {"max_batch_size": 4, "max_step_tokens": 96,
                                                                     "max_token_len": 256},
                                                "block_manager": {"block_token_num": 16}}})
    eng = LLMEngine(model, serving, num_blocks=64, num_host_blocks=0)
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(16, 65, (4,), generator=g).tolist()
    prompts = [torch.randint(3, 32000, (n,), generator=g).tolist() for n in lens]
    sp = SamplingParams(topk=1, max_new_tokens=32, ignore_eos=True)
    reqs = eng.generate(prompts, sp)
    for prompt, req in zip(prompts, reqs):
        toks = list(prompt)
        for _ in range(32):
            toks.append(int(plain_forward(sd, cfg, toks).argmax()))
        assert req.output_token_ids[0] == toks[len(prompt):]
    # continuous batching really interleaved requests: fewer steps than sequential decoding would need
    assert eng.stats["steps"] < 4 * 32
