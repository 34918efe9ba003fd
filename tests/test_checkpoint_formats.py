"""One tiny Llama written to disk as (a) one safetensors file, (b) sharded safetensors, (c) a PyTorch ``.bin``,
(d) safetensors under foreign tensor names plus a ``<model_type>_weight_map.json``: every directory, loaded through
the same entry point, yields the same logits."""
import json
import os

import torch
from safetensors.torch import save_file

from ksanallm_b200.config.model_config import load_model_config
from ksanallm_b200.engine.step_input import make_step_input
from ksanallm_b200.models.loader import load_model_weights, synthetic_checkpoint
from ksanallm_b200.models.transformer import TransformerModel

CONFIG = dict(model_type="llama", hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              intermediate_size=128, vocab_size=300, torch_dtype="float32", max_position_embeddings=64,
              rms_norm_eps=1e-5, rope_theta=10000.0)


def _logits(model_dir):
    cfg = load_model_config(model_dir)
    model = TransformerModel(cfg, load_model_weights(cfg, model_dir, dtype=torch.float32), max_positions=64)
    T = 9
    meta = make_step_input(list(range(5, 5 + T)), list(range(T)), list(range(T)), [0, T], [T], [[0]], device="cpu")
    return model.compute_logits(model.forward(meta, model.allocate_kv_cache(1, 16)), meta.logits_idx)[0]


def _dir(tmp_path, name, config=CONFIG):
    d = tmp_path / name
    d.mkdir()
    (d / "config.json").write_text(json.dumps(config))
    return str(d)


def test_all_formats_load_to_the_same_model(tmp_path):
    cfg = load_model_config(_dir(tmp_path, "cfg_only"))
    sd = {k: v.contiguous() for k, v in synthetic_checkpoint(cfg, seed=7, dtype=torch.float32)}
    a = _dir(tmp_path, "single")
    save_file(sd, os.path.join(a, "model.safetensors"))
    want = _logits(a)

    b = _dir(tmp_path, "sharded")
    keys = sorted(sd)
    for i in range(3):
        part = {k: sd[k] for k in keys[i::3]}
        save_file(part, os.path.join(b, f"model-{i + 1:05d}-of-00003.safetensors"))
    assert torch.equal(_logits(b), want)

    c = _dir(tmp_path, "bin")
    torch.save(sd, os.path.join(c, "pytorch_model.bin"))
    assert torch.equal(_logits(c), want)

    # foreign names + a weight map (regex -> replacement) next to the checkpoint
    d = _dir(tmp_path, "mapped", dict(CONFIG, model_type="mymodel"))
    foreign = {k.replace("model.layers.", "decoder.blocks.").replace("self_attn.", "attn.")
               .replace("model.embed_tokens", "decoder.wte").replace("model.norm", "decoder.ln_out"): v
               for k, v in sd.items()}
    save_file(foreign, os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "mymodel_weight_map.json"), "w") as f:
        json.dump({r"^decoder\.blocks\.": "model.layers.", r"\.attn\.": ".self_attn.",
                   r"^decoder\.wte": "model.embed_tokens", r"^decoder\.ln_out": "model.norm"}, f)
    assert torch.equal(_logits(d), want)


def test_processed_weight_cache_is_written_and_reused(tmp_path, monkeypatch):
    cfg = load_model_config(_dir(tmp_path, "cfg_only"))
    sd = {k: v.contiguous() for k, v in synthetic_checkpoint(cfg, seed=7, dtype=torch.float32)}
    d = _dir(tmp_path, "cached")
    save_file(sd, os.path.join(d, "model.safetensors"))
    want = _logits(d)
    monkeypatch.setenv("ENABLE_MODEL_CACHE", "1")
    monkeypatch.setenv("MODEL_CACHE_PATH", str(tmp_path / "cache"))
    assert torch.equal(_logits(d), want)
    files = os.listdir(tmp_path / "cache")
    assert len(files) == 1 and files[0].startswith("rank0of1")
    os.remove(os.path.join(d, "model.safetensors"))  # the second start never opens the checkpoint
    assert torch.equal(_logits(d), want)


def test_gguf_llama_checkpoint_with_converter_row_order(tmp_path):
    """A GGUF file as llama.cpp's converter writes it for Llama-architecture models (q / k rows reordered for its
    rotary kernel, llama.cpp tensor names) loads to the same logits as the original safetensors."""
    from ksanallm_b200.models import gguf_reader
    cfg = load_model_config(_dir(tmp_path, "cfg_only"))
    sd = {k: v.contiguous() for k, v in synthetic_checkpoint(cfg, seed=7, dtype=torch.float32)}
    a = _dir(tmp_path, "st")
    save_file(sd, os.path.join(a, "model.safetensors"))
    want = _logits(a)

    def permute(w, n_head):  # the converter's reordering
        return w.reshape(n_head, 2, w.shape[0] // n_head // 2, *w.shape[1:]).swapaxes(1, 2).reshape(w.shape)

    names = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
             "lm_head.weight": "output.weight"}
    per_layer = {"input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm", "self_attn.q_proj": "attn_q",
                 "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v", "self_attn.o_proj": "attn_output",
                 "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down"}
    g = {}
    for k, v in sd.items():
        if k in names:
            g[names[k]] = v
            continue
        _, _, li, rest = k.split(".", 3)
        stem = rest[:-len(".weight")]
        t = v
        if stem == "self_attn.q_proj":
            t = permute(v, cfg.num_heads)
        elif stem == "self_attn.k_proj":
            t = permute(v, cfg.num_kv_heads)
        g[f"blk.{li}.{per_layer[stem]}.weight"] = t.contiguous()
    d = _dir(tmp_path, "gguf")
    gguf_reader.write_gguf(os.path.join(d, "model.gguf"), g, {
        "general.architecture": "llama", "llama.block_count": cfg.num_layers,
        "llama.attention.head_count": cfg.num_heads, "llama.attention.head_count_kv": cfg.num_kv_heads})
    assert torch.allclose(_logits(d), want, atol=1e-6)


def test_generation_config_adds_end_of_sequence_ids(tmp_path):
    d = _dir(tmp_path, "gen", dict(CONFIG, eos_token_id=2))
    with open(os.path.join(d, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": [2, 7]}, f)
    assert load_model_config(d).eos_token_ids == [2, 7]


def test_reference_package_names_and_bundled_plugin_lookup(tmp_path):
    import ksana_llm
    from ksanallm_b200.serving.plugin import search_plugin_path
    assert ksana_llm.KsanaLLMEngine is not None and ksana_llm.PluginConfig(plugin_name="qwen2_vl").plugin_name == "qwen2_vl"
    tok = ksana_llm.TokenizerProcessorOpBase(str(tmp_path), None, None)
    assert tok.decode(tok.encode("hi", add_special_tokens=False)) == "hi"
    assert search_plugin_path(str(tmp_path), {"plugin_name": "qwen2_vl"}).endswith("plugins/qwen2_vl.py")
    assert search_plugin_path(str(tmp_path), {"plugin_name": "internvl_chat"}).endswith("plugins/internvl.py")
    assert search_plugin_path(str(tmp_path), {}) is None
    own = tmp_path / "ksana_plugin.py"
    own.write_text("class KsanaPlugin:\n    pass\n")
    assert search_plugin_path(str(tmp_path), {"plugin_name": "qwen2_vl"}) == str(own)
