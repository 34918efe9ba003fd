"""Vision plugin for InternVL (transformers layout: ``model.vision_tower``, ``model.multi_modal_projector``,
``model.language_model``): every image becomes ``(image_size / patch)^2 * downsample_ratio^2`` embedding rows per
tile, spliced over the prompt's image-context tokens. Positions stay one-dimensional.

What the reference's plugin does (src/ksana_llm/python/ksana_plugin/internvl_chat/ksana_plugin.py): dynamic tiling of
the picture into up to ``max_dynamic_patch`` square tiles plus a thumbnail, ViT, pixel shuffle, MLP projector,
``input_refit_embedding`` at the ``<IMG_CONTEXT>`` runs. Here the ViT / projector are the transformers modules; tiling
follows the published rule (closest aspect ratio among the grids with at most ``max_tiles`` tiles, thumbnail when
more than one tile).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Tuple

import torch

from .qwen2_vl import _load_image, images_of

MEAN, STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)


def tile_grid(width: int, height: int, tile: int, max_tiles: int) -> Tuple[int, int]:
    """(columns, rows) of the tiling whose aspect ratio is closest to the picture's; ties go to the larger grid when
    the picture has more than half of its pixels."""
    ratio = width / height
    best, best_diff = (1, 1), float("inf")
    grids = sorted({(c, r) for n in range(1, max_tiles + 1) for c in range(1, n + 1) for r in range(1, n + 1)
                    if c * r <= max_tiles}, key=lambda g: g[0] * g[1])
    for c, r in grids:
        diff = abs(ratio - c / r)
        if diff < best_diff:
            best, best_diff = (c, r), diff
        elif diff == best_diff and width * height > 0.5 * tile * tile * c * r:
            best = (c, r)
    return best


class _VisionSide(torch.nn.Module):
    def __init__(self, cfg):
        super().__init__()
        from transformers.models.internvl.modeling_internvl import InternVLMultiModalProjector, InternVLVisionModel
        self.config = cfg
        self.vision_tower = InternVLVisionModel(cfg.vision_config)
        self.multi_modal_projector = InternVLMultiModalProjector(cfg)

    @torch.inference_mode()
    def features(self, pixels: torch.Tensor) -> torch.Tensor:
        """pixels [tiles, 3, S, S] -> [tiles, tokens per tile, hidden of the language model]."""
        cfg = self.config
        layer = cfg.vision_feature_layer
        out = self.vision_tower(pixel_values=pixels, return_dict=True, output_hidden_states=layer != -1)
        f = out.last_hidden_state if layer == -1 else out.hidden_states[layer]
        if cfg.vision_feature_select_strategy == "default":
            f = f[:, 1:, :]  # drop the class token
        b, n, _ = f.shape
        side = int(n ** 0.5)
        f = f.reshape(b, side, side, -1)
        s = cfg.downsample_ratio  # pixel shuffle: (w, h, c) -> (w * s, h * s, c / s^2)
        f = f.view(b, side, int(side * s), int(f.shape[-1] / s)).permute(0, 2, 1, 3).contiguous()
        f = f.view(b, int(side * s), int(side * s), int(f.shape[-1] / s)).permute(0, 2, 1, 3).contiguous()
        return self.multi_modal_projector(f.reshape(b, -1, f.shape[-1]))


class KsanaPlugin:
    def init_plugin(self, **kwargs) -> None:
        from transformers.models.internvl.configuration_internvl import InternVLConfig
        model_path = kwargs.get("model_path") or ""
        with open(os.path.join(model_path, "config.json"), "r", encoding="utf-8") as f:
            raw = json.load(f)
        raw.pop("model_type", None)
        raw.pop("architectures", None)
        self.config = InternVLConfig(**raw)
        self.image_token = int(self.config.image_token_id)
        self.tile = int(self.config.vision_config.image_size[0])
        self.max_tiles = int(kwargs.get("max_tiles", kwargs.get("max_dynamic_patch", 1)) or 1)
        self.device = torch.device(kwargs.get("device") or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.side = _VisionSide(self.config).eval()
        from ...models.loader import iter_checkpoint
        sd = {}
        for name, t in iter_checkpoint(model_path):
            for prefix in ("model.", ""):
                for part in ("vision_tower.", "multi_modal_projector."):
                    if name.startswith(prefix + part):
                        sd[name[len(prefix):]] = t
        missing, _ = self.side.load_state_dict(sd, strict=False)
        if missing:
            raise RuntimeError(f"vision side: {len(missing)} tensors missing from the checkpoint, e.g. {missing[:3]}")
        self.side.to(self.device)

    def tiles_of(self, img) -> torch.Tensor:
        import numpy as np
        from PIL import Image
        cols, rows = tile_grid(img.width, img.height, self.tile, self.max_tiles)
        big = img.resize((cols * self.tile, rows * self.tile), Image.BICUBIC)
        parts = [big.crop((c * self.tile, r * self.tile, (c + 1) * self.tile, (r + 1) * self.tile))
                 for r in range(rows) for c in range(cols)]
        if len(parts) > 1:
            parts.append(img.resize((self.tile, self.tile), Image.BICUBIC))  # thumbnail of the whole picture
        arr = np.stack([np.asarray(p, dtype=np.float32) / 255.0 for p in parts])
        x = torch.from_numpy(arr).permute(0, 3, 1, 2)
        return (x - torch.tensor(MEAN).view(1, 3, 1, 1)) / torch.tensor(STD).view(1, 3, 1, 1)

    def embed_images(self, images) -> List[torch.Tensor]:
        out = []
        for img in images:
            px = self.tiles_of(img).to(self.device, dtype=next(self.side.parameters()).dtype)
            out.append(self.side.features(px).reshape(-1, self.config.text_config.hidden_size).float().cpu())
        return out

    def preprocess(self, **kwargs) -> Optional[Dict[str, Any]]:
        images = images_of(kwargs.get("messages"))
        req = kwargs.get("request_dict") or {}
        images += [_load_image(i) for i in (req.get("images") or [])]
        if not images:
            return None
        tokens = list(kwargs.get("input_tokens") or [])
        embeds = self.embed_images(images)
        wide, starts, g, i = [], [], 0, 0
        while i < len(tokens):
            if tokens[i] == self.image_token and g < len(embeds):
                starts.append(len(wide))
                wide.extend([self.image_token] * embeds[g].shape[0])
                g += 1
                while i < len(tokens) and tokens[i] == self.image_token:
                    i += 1
                continue
            wide.append(tokens[i])
            i += 1
        if g != len(embeds):
            raise ValueError(f"{len(embeds)} images but {g} image placeholders in the prompt")
        pin = kwargs.get("ksana_python_input")
        if pin is not None:
            pin.input_tokens = wide
            pin.input_refit_embedding.pos = starts
            pin.input_refit_embedding.embedding_tensors = embeds
        return {"input_tokens": wide, "input_refit_embedding": {"pos": starts, "embeddings": embeds}}

    def postprocess(self, **kwargs) -> None:
        return None
