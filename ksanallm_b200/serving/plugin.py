"""Per-model plugin hook: a ``ksana_plugin.py`` inside the model directory (or the path given by
``model_spec.plugin_model.plugin_path``) may define a class ``KsanaPlugin`` with ``init_plugin(**kwargs)``,
``preprocess(**kwargs)`` and ``postprocess(**kwargs)``. Typical use: a vision / audio tower that turns
``messages`` into ``input_refit_embedding`` (positions + embedding rows spliced into the token embeddings).
Reference: src/ksana_llm/python/ksana_llm/ksana_plugin.py:36-205 and ksana_plugin/<model>/ksana_plugin.py.
"""
from __future__ import annotations

import importlib.util
import os
from typing import Any, Dict, List, Optional


class RefitEmbedding:
    """Mutable stand-in for the reference's ``ksana_python_input.input_refit_embedding``: a plugin writes the splice
    positions, one embedding tensor per position and optional extra tensors (multimodal RoPE: [positions, delta])."""

    def __init__(self):
        self.pos: List[int] = []
        self.embeddings: List[Any] = []
        self.embedding_tensors: List[Any] = []
        self.additional_tensors: List[Any] = []


class PluginInput:
    """What a plugin sees as ``ksana_python_input`` (reference: KsanaPythonInput in torch_op/serving_op.cpp)."""

    def __init__(self, tokens: List[int]):
        self.input_tokens: List[int] = list(tokens)
        self.input_refit_embedding = RefitEmbedding()


class PluginHost:
    def __init__(self, impl, engine):
        self.impl = impl
        self.engine = engine

    def preprocess(self, request_dict: Dict[str, Any], tokens: List[int]) -> Optional[Dict[str, Any]]:
        """Runs the plugin's ``preprocess``. Both contracts are understood: the reference's (the plugin mutates
        ``ksana_python_input``: input_tokens, input_refit_embedding.pos / embedding_tensors / additional_tensors)
        and a returned dict with ``input_tokens``, ``input_refit_embedding`` {pos, embeddings}, ``mrope_positions``."""
        fn = getattr(self.impl, "preprocess", None)
        if fn is None:
            return None
        import torch
        pin = PluginInput(tokens)
        res = fn(ksana_python_input=pin, request_dict=request_dict, input_tokens=tokens,
                 tokenizer=self.engine.tokenizer.tokenizer, messages=request_dict.get("messages"),
                 additional_params=request_dict.get("additional_params") or {}) or {}
        out: Dict[str, Any] = {}
        hs = self.engine.model_config.hidden_size
        if "input_tokens" in res:
            out["input_tokens"] = list(res["input_tokens"])
        elif list(pin.input_tokens) != list(tokens):
            out["input_tokens"] = list(pin.input_tokens)
        emb = res.get("input_refit_embedding")
        pos, vals = (emb["pos"], emb["embeddings"]) if emb else \
            (pin.input_refit_embedding.pos,
             pin.input_refit_embedding.embedding_tensors or pin.input_refit_embedding.embeddings)
        if pos and vals:
            out["refit"] = [(int(p), torch.as_tensor(e, dtype=torch.float32).view(-1, hs)) for p, e in zip(pos, vals)]
        extra = pin.input_refit_embedding.additional_tensors
        if res.get("mrope_positions") is not None:
            out["mrope_positions"] = res["mrope_positions"]
        elif extra:
            out["mrope_positions"] = extra[0]  # [axes, prompt_len]; the delta follows from it
        return out or None

    def postprocess(self, request_dict: Dict[str, Any], output) -> None:
        fn = getattr(self.impl, "postprocess", None)
        if fn is not None:
            fn(ksana_python_input=None, ksana_python_output=output, request_dict=request_dict)


BUNDLED = {"qwen2_vl": "qwen2_vl", "qwen2_5_vl": "qwen2_vl", "internvl": "internvl", "internvl_chat": "internvl",
           "qwen_vl": "qwen_vl", "qwenvl": "qwen_vl", "internlmxcomposer2": "internlmxcomposer2",
           "internlm_xcomposer2": "internlmxcomposer2"}


def search_plugin_path(model_dir: str, plugin_cfg: Dict[str, Any]) -> Optional[str]:
    """An explicit ``plugin_path``, else ``ksana_plugin.py`` in the model directory, else the bundled plugin named
    by ``model_spec.plugin_model.plugin_name`` (reference: KsanaPlugin.search_plugin_path, ksana_plugin.py)."""
    cfg = plugin_cfg or {}
    for cand in (cfg.get("plugin_path"), os.path.join(model_dir or "", "ksana_plugin.py")):
        if cand and os.path.isfile(cand):
            return cand
    name = BUNDLED.get(str(cfg.get("plugin_name", "") or "").lower())
    if name:
        return os.path.join(os.path.dirname(os.path.abspath(__file__)), "plugins", name + ".py")
    return None


def load_plugin(model_dir: str, plugin_cfg: Dict[str, Any], engine) -> Optional[PluginHost]:
    path = search_plugin_path(model_dir, plugin_cfg)
    if not path:
        return None
    if os.path.dirname(path) == os.path.join(os.path.dirname(os.path.abspath(__file__)), "plugins"):
        from importlib import import_module
        mod = import_module(f"{__package__}.plugins.{os.path.basename(path)[:-3]}")
        impl = mod.KsanaPlugin()
        impl.init_plugin(python_plugin_path=path, model_path=model_dir, preprocess=True, postprocess=True,
                         **{k: v for k, v in (plugin_cfg or {}).items() if k not in ("plugin_path", "plugin_name")})
        return PluginHost(impl, engine)
    spec = importlib.util.spec_from_file_location("ksana_plugin", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    cls = getattr(mod, "KsanaPlugin", None)
    if cls is None:
        return None
    impl = cls()
    init = getattr(impl, "init_plugin", None)
    if init is not None:
        init(python_plugin_path=path, model_path=model_dir, preprocess=True, postprocess=True,
             **{k: v for k, v in (plugin_cfg or {}).items() if k != "plugin_path"})
    return PluginHost(impl, engine)
