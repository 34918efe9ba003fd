"""Bundled vision plugin for Qwen-VL (the first generation, ``model_type: qwen`` with a ``visual`` block).

Qwen-VL's tokenizer turns ``<img>URL</img>`` into ``image_start_id``, the URL's bytes as token ids padded with
``image_start_id + 2`` to 256 positions, ``image_start_id + 1``. The plugin reads the URLs back out of the token ids,
runs the checkpoint's vision tower (ViT + resampler -> 256 rows of the language model's width per image) and has
those rows spliced over the 256 positions. The tower is the checkpoint's own code
(``transformers`` remote code: ``<model>.transformer.visual`` with its ``encode(urls)``), loaded from the model
directory; ``init_plugin(tower=...)`` takes any object with that method instead. Behaviour of the reference:
src/ksana_llm/python/ksana_plugin/qwen_vl/ksana_plugin.py:46-75 (its TensorRT engine path is not reproduced; the
tower runs in PyTorch).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional

import torch


def image_urls(tokens: List[int], image_start_id: int) -> (List[int], List[str]):
    """-> (position of the first of the 256 image slots, URL) for every ``<img>...</img>`` span in ``tokens``."""
    end_id, pad_id = image_start_id + 1, image_start_id + 2
    starts = [i + 1 for i, t in enumerate(tokens) if t == image_start_id]
    ends = [i for i, t in enumerate(tokens) if t == end_id]
    if len(starts) != len(ends):
        raise ValueError("unbalanced <img> ... </img> markers in the prompt")
    pos, urls = [], []
    for a, b in zip(starts, ends):
        if b < a:
            raise ValueError("</img> before <img>")
        span = tokens[a:b]
        if pad_id in span:
            span = span[:span.index(pad_id)]
        if any(not 0 <= t < 256 for t in span):
            raise ValueError("an image span holds something else than URL bytes")
        pos.append(a)
        urls.append(bytes(span).decode("utf-8"))
    return pos, urls


class KsanaPlugin:
    def init_plugin(self, **kwargs) -> Optional[Dict[str, Any]]:
        model_path = kwargs.get("model_path") or ""
        self.device = torch.device(kwargs.get("device") or ("cuda" if torch.cuda.is_available() else "cpu"))
        visual: Dict[str, Any] = dict(kwargs.get("visual") or {})
        cfg_file = os.path.join(model_path, "config.json")
        if not visual and os.path.isfile(cfg_file):
            with open(cfg_file, "r", encoding="utf-8") as f:
                visual = dict(json.load(f).get("visual") or {})
        if "image_start_id" not in visual:
            raise ValueError("Qwen-VL plugin: config.json has no visual.image_start_id")
        self.image_start_id = int(visual["image_start_id"])
        self.tower = kwargs.get("tower")
        if self.tower is None:
            from transformers import AutoModelForCausalLM
            full = AutoModelForCausalLM.from_pretrained(model_path, trust_remote_code=True, torch_dtype=torch.float16)
            self.tower = full.transformer.visual.to(self.device).eval()
            del full
        return {"plugin_trt": False}

    @torch.no_grad()
    def preprocess(self, **kwargs) -> Optional[Dict[str, Any]]:
        tokens = list(kwargs.get("input_tokens") or getattr(kwargs.get("ksana_python_input"), "input_tokens", []) or [])
        pos, urls = image_urls(tokens, self.image_start_id)
        if not urls:
            return None
        emb = self.tower.encode(urls)  # [images, 256, hidden]
        rows = [e.detach().float().cpu() for e in torch.unbind(emb, 0)]
        pin = kwargs.get("ksana_python_input")
        if pin is not None:
            pin.input_refit_embedding.pos = list(pos)
            pin.input_refit_embedding.embedding_tensors = rows
        return {"input_refit_embedding": {"pos": list(pos), "embeddings": rows}}

    def postprocess(self, **kwargs) -> None:
        return None
