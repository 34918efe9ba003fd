"""Vision plugin for Qwen2-VL: images in the request become embedding rows spliced over the prompt's image
placeholders, plus the three-axis (temporal, height, width) RoPE positions of every prompt token.

What the reference's plugin does (src/ksana_llm/python/ksana_plugin/qwen2_vl/ksana_plugin.py:69-134,
ksana_plugin_model.py): chat template -> processor -> ViT -> ``input_refit_embedding`` (pos = first placeholder of each
image, one tensor per image) + ``additional_tensors`` = [positions [3, T], delta]. Here:

* the vision tower is the transformers module (``Qwen2VisionTransformerPretrainedModel``) loaded from the
  checkpoint's ``visual.*`` / ``model.visual.*`` tensors; it runs in PyTorch on the engine's device,
* pixels come from ``Qwen2VLImageProcessor`` (the checkpoint's preprocessor_config.json when present),
* the prompt is either ``input_tokens`` with ONE image placeholder token per image, or ``messages`` rendered through
  the tokenizer's chat template; every placeholder is widened to the image's number of merged patches,
* positions follow the published rule: text advances all three axes together; an image keeps its temporal index and
  walks its (height, width) grid; what follows continues from the largest index used so far + 1.

Images: PIL images, file paths, ``file://`` URLs and base64 ``data:`` URLs (there is no network access for http).
"""
from __future__ import annotations

import base64
import io
import json
import os
from typing import Any, Dict, List, Optional, Tuple

import torch


def _load_image(src):
    from PIL import Image
    if hasattr(src, "convert"):
        return src.convert("RGB")
    if isinstance(src, dict):
        src = src.get("url") or src.get("image") or src.get("path")
    if not isinstance(src, str):
        raise ValueError("unsupported image reference")
    if src.startswith("data:"):
        return Image.open(io.BytesIO(base64.b64decode(src.split(",", 1)[1]))).convert("RGB")
    if src.startswith("file://"):
        src = src[7:]
    if src.startswith("http://") or src.startswith("https://"):
        raise ValueError("remote images are not fetched; pass a file path or a data: URL")
    return Image.open(src).convert("RGB")


def images_of(messages) -> List[Any]:
    out = []
    for m in messages or []:
        c = m.get("content") if isinstance(m, dict) else None
        if not isinstance(c, list):
            continue
        for part in c:
            if not isinstance(part, dict):
                continue
            if part.get("type") == "image_url":
                out.append(_load_image(part["image_url"]))
            elif part.get("type") == "image":
                out.append(_load_image(part.get("image", part)))
    return out


def mrope_positions(tokens: List[int], grids: List[Tuple[int, int, int]], image_token: int, merge: int) -> torch.Tensor:
    """[3, len(tokens)] positions. ``grids``: (t, h, w) in patches for every image, in prompt order; an image
    occupies t * (h / merge) * (w / merge) consecutive ``image_token`` entries."""
    pos = torch.zeros(3, len(tokens), dtype=torch.long)
    nxt, i, g = 0, 0, 0
    while i < len(tokens):
        if tokens[i] == image_token and g < len(grids):
            t, h, w = grids[g]
            h, w = h // merge, w // merge
            n = t * h * w
            idx = torch.arange(n)
            pos[0, i:i + n] = nxt + idx // (h * w)
            pos[1, i:i + n] = nxt + (idx // w) % h
            pos[2, i:i + n] = nxt + idx % w
            nxt += max(t, h, w)
            i += n
            g += 1
        else:
            pos[:, i] = nxt
            nxt += 1
            i += 1
    return pos


class KsanaPlugin:
    def init_plugin(self, **kwargs) -> None:
        from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLVisionConfig
        from transformers.models.qwen2_vl.image_processing_qwen2_vl import Qwen2VLImageProcessor
        from transformers.models.qwen2_vl.modeling_qwen2_vl import Qwen2VisionTransformerPretrainedModel
        model_path = kwargs.get("model_path") or ""
        with open(os.path.join(model_path, "config.json"), "r", encoding="utf-8") as f:
            raw = json.load(f)
        self.image_token = int(raw.get("image_token_id", 151655))
        self.vision_start = int(raw.get("vision_start_token_id", 151652))
        vcfg = Qwen2VLVisionConfig(**{k: v for k, v in (raw.get("vision_config") or {}).items() if k != "model_type"})
        self.merge = int(vcfg.spatial_merge_size)
        self.device = torch.device(kwargs.get("device") or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.visual = Qwen2VisionTransformerPretrainedModel(vcfg).eval()
        self._load_visual(model_path)
        self.visual.to(self.device)
        pre = os.path.join(model_path, "preprocessor_config.json")
        kw = {}
        if os.path.isfile(pre):
            with open(pre, "r", encoding="utf-8") as f:
                pc = json.load(f)
            kw = {k: pc[k] for k in ("min_pixels", "max_pixels", "patch_size", "temporal_patch_size", "merge_size",
                                     "image_mean", "image_std", "size") if k in pc}
        kw.setdefault("patch_size", int(vcfg.patch_size))
        kw.setdefault("merge_size", self.merge)
        kw.setdefault("temporal_patch_size", int(vcfg.temporal_patch_size))
        self.image_processor = Qwen2VLImageProcessor(**kw)

    def _load_visual(self, model_path: str) -> None:
        from ...models.loader import iter_checkpoint
        sd = {}
        for name, t in iter_checkpoint(model_path):
            for prefix in ("model.visual.", "visual."):
                if name.startswith(prefix):
                    sd[name[len(prefix):]] = t
                    break
        missing, unexpected = self.visual.load_state_dict(sd, strict=False)
        if missing:
            raise RuntimeError(f"vision tower: {len(missing)} tensors missing from the checkpoint, e.g. {missing[:3]}")

    @torch.inference_mode()
    def embed_images(self, images) -> Tuple[List[torch.Tensor], List[Tuple[int, int, int]]]:
        feats = self.image_processor(images=images, return_tensors="pt")
        grid = feats["image_grid_thw"]
        pixels = feats["pixel_values"].to(self.device, dtype=self.visual.dtype)
        out = self.visual(pixels, grid_thw=grid.to(self.device))
        rows = out.pooler_output if hasattr(out, "pooler_output") else out
        sizes = (grid.prod(-1) // self.merge ** 2).tolist()
        return [r.float().cpu() for r in torch.split(rows, sizes)], [tuple(int(x) for x in g) for g in grid.tolist()]

    def preprocess(self, **kwargs) -> Optional[Dict[str, Any]]:
        images = images_of(kwargs.get("messages"))
        req = kwargs.get("request_dict") or {}
        images += [_load_image(i) for i in (req.get("images") or [])]
        if not images:
            return None
        tokens = list(kwargs.get("input_tokens") or [])
        if not tokens and kwargs.get("messages") is not None:
            tok = kwargs["tokenizer"]
            tokens = list(tok.apply_chat_template(kwargs["messages"], tokenize=True, add_generation_prompt=True))
        embeds, grids = self.embed_images(images)
        # widen each single placeholder to the image's number of merged patches
        wide, starts, g = [], [], 0
        i = 0
        while i < len(tokens):
            if tokens[i] == self.image_token and g < len(embeds):
                starts.append(len(wide))
                wide.extend([self.image_token] * embeds[g].shape[0])
                g += 1
                while i < len(tokens) and tokens[i] == self.image_token:
                    i += 1  # a prompt that already carries the widened run
                continue
            wide.append(tokens[i])
            i += 1
        if g != len(embeds):
            raise ValueError(f"{len(embeds)} images but {g} image placeholders in the prompt")
        pin = kwargs.get("ksana_python_input")
        if pin is not None:  # the reference's contract: results are written into the input object
            pin.input_tokens = wide
            pin.input_refit_embedding.pos = starts
            pin.input_refit_embedding.embedding_tensors = embeds
        pos3 = mrope_positions(wide, grids, self.image_token, self.merge)
        if pin is not None:
            delta = int(pos3.max()) + 1 - len(wide)
            pin.input_refit_embedding.additional_tensors = [pos3, torch.tensor([delta])]
        return {"input_tokens": wide, "input_refit_embedding": {"pos": starts, "embeddings": embeds},
                "mrope_positions": pos3}

    def postprocess(self, **kwargs) -> None:
        return None
