"""Bundled vision plugin for InternLM-XComposer2.

OpenAI-style ``messages`` (text parts plus ``image_url`` / ``zip_url`` parts) become the model's chat prompt
``[UNUSED_TOKEN_146]user\\n...[UNUSED_TOKEN_145]\\n[UNUSED_TOKEN_146]assistant\\n`` with one ``<ImageHere>`` per
image (a single image without a marker goes in front). The text between the markers is tokenised piece by piece
(only the first piece gets the BOS token), every image is encoded by the checkpoint's own vision side
(``encode_img``: ViT + projector -> rows of the language model's width) and takes that many placeholder positions
(token id 0), over which its rows are spliced. The prompt is cut at the model's ``max_length``. The vision side is the
checkpoint's remote code loaded through ``transformers``; ``init_plugin(model=..., tokenizer=...)`` takes stand-ins.
Behaviour of the reference: src/ksana_llm/python/ksana_plugin/internlmxcomposer2/ksana_plugin.py:55-107, 164-184
(its TensorRT engine path is not reproduced).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Tuple

import torch

MARK = "<ImageHere>"


def convert_openai_messages(messages) -> Tuple[Optional[str], List[str]]:
    """The last text part is the prompt; every image_url / zip_url part is an image, in order."""
    text, images = None, []
    for m in messages or []:
        content = m.get("content")
        if isinstance(content, str):
            text = content
            continue
        for part in content or []:
            if "text" in part:
                text = part["text"]
            for key in ("zip_url", "image_url"):
                if key in part:
                    url = part[key]
                    images.append(url["url"] if isinstance(url, dict) else url)
    return text, images


class KsanaPlugin:
    def init_plugin(self, **kwargs) -> Optional[Dict[str, Any]]:
        model_path = kwargs.get("model_path") or ""
        self.device = torch.device(kwargs.get("device") or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.max_length = int(kwargs.get("max_length") or 0)
        cfg_file = os.path.join(model_path, "config.json")
        if not self.max_length and os.path.isfile(cfg_file):
            with open(cfg_file, "r", encoding="utf-8") as f:
                self.max_length = int(json.load(f).get("max_length") or 0)
        self.max_length = self.max_length or 4096
        self.tokenizer = kwargs.get("tokenizer")
        self.model = kwargs.get("model")
        if self.tokenizer is None:
            from transformers import AutoTokenizer
            self.tokenizer = AutoTokenizer.from_pretrained(model_path, trust_remote_code=True)
        if self.model is None:
            from transformers import AutoModel
            self.model = AutoModel.from_pretrained(model_path, trust_remote_code=True, torch_dtype=torch.float16)
            self.model = self.model.to(self.device).eval()
            self.model.tokenizer = self.tokenizer
        return {"plugin_trt": False}

    @torch.no_grad()
    def preprocess(self, **kwargs) -> Optional[Dict[str, Any]]:
        messages = kwargs.get("messages")
        if messages is None:
            return None
        prompt, images = convert_openai_messages(messages)
        if not images:
            return None
        prompt = f"[UNUSED_TOKEN_146]user\n{prompt or ''}[UNUSED_TOKEN_145]\n[UNUSED_TOKEN_146]assistant\n"
        if len(images) == 1 and MARK not in prompt:
            prompt = MARK + prompt
        parts = prompt.split(MARK)
        tokens: List[int] = []
        pos: List[int] = []
        rows: List[torch.Tensor] = []
        need_bos = True
        for idx, part in enumerate(parts):
            if part:
                tokens.extend(self.tokenizer(part, add_special_tokens=need_bos).input_ids)
                need_bos = False
            if idx < len(images):
                img = self.model.encode_img(images[idx])  # [1, rows, hidden]
                img = img.reshape(-1, img.shape[-1]).detach().float().cpu()
                pos.append(len(tokens))
                rows.append(img)
                tokens.extend([0] * img.shape[0])
        # the prompt is cut at max_length; an image the cut would split is dropped together with what follows it
        cut, keep = min(len(tokens), self.max_length), 0
        for p, r in zip(pos, rows):
            if p + r.shape[0] > cut:
                cut = min(cut, p)
                break
            keep += 1
        tokens, pos, rows = tokens[:cut], pos[:keep], rows[:keep]
        pin = kwargs.get("ksana_python_input")
        if pin is not None:
            pin.input_tokens = tokens
            pin.input_refit_embedding.pos = pos
            pin.input_refit_embedding.embedding_tensors = rows
        return {"input_tokens": tokens, "input_refit_embedding": {"pos": pos, "embeddings": rows}}

    def postprocess(self, **kwargs) -> None:
        return None
