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


class PluginHost:
    def __init__(self, impl, engine):
        self.impl = impl
        self.engine = engine

    def preprocess(self, request_dict: Dict[str, Any], tokens: List[int]) -> Optional[Dict[str, Any]]:
        fn = getattr(self.impl, "preprocess", None)
        if fn is None:
            return None
        res = fn(ksana_python_input=None, request_dict=request_dict, input_tokens=tokens,
                 tokenizer=self.engine.tokenizer.tokenizer, messages=request_dict.get("messages"))
        if not res:
            return None
        out: Dict[str, Any] = {}
        if "input_tokens" in res:
            out["input_tokens"] = list(res["input_tokens"])
        emb = res.get("input_refit_embedding")
        if emb:
            import torch
            hs = self.engine.model_config.hidden_size
            out["refit"] = [(int(p), torch.as_tensor(e, dtype=torch.float32).view(-1, hs))
                            for p, e in zip(emb["pos"], emb["embeddings"])]
        return out

    def postprocess(self, request_dict: Dict[str, Any], output) -> None:
        fn = getattr(self.impl, "postprocess", None)
        if fn is not None:
            fn(ksana_python_input=None, ksana_python_output=output, request_dict=request_dict)


def load_plugin(model_dir: str, plugin_cfg: Dict[str, Any], engine) -> Optional[PluginHost]:
    path = (plugin_cfg or {}).get("plugin_path") or os.path.join(model_dir or "", "ksana_plugin.py")
    if not path or not os.path.isfile(path):
        return None
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
