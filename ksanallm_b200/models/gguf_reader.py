"""Minimal GGUF reader for unquantised tensors (F32 / F16 / BF16) plus llama.cpp -> HF name mapping.

The reference loads ``*.gguf`` through its own file loader (src/ksana_llm/utils/gguf_file_tensor_loader.cpp) with
the renames of python/weight_map/llama_gguf_weight_map.json. Quantised GGML block types are not decoded here: a
file containing them raises, it is never silently mis-read.
"""
from __future__ import annotations

import mmap
import re
import struct
from typing import Any, Dict, Iterator, Tuple

import numpy as np
import torch

GGUF_MAGIC = 0x46554747
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_GGML_DTYPES = {0: (np.float32, torch.float32), 1: (np.float16, torch.float16), 30: (np.uint16, torch.bfloat16)}

_NAME_MAP = [
    (r"^token_embd\.", "model.embed_tokens."), (r"^output_norm\.", "model.norm."), (r"^output\.", "lm_head."),
    (r"^blk\.(\d+)\.attn_norm\.", r"model.layers.\1.input_layernorm."),
    (r"^blk\.(\d+)\.ffn_norm\.", r"model.layers.\1.post_attention_layernorm."),
    (r"^blk\.(\d+)\.attn_q\.", r"model.layers.\1.self_attn.q_proj."),
    (r"^blk\.(\d+)\.attn_k\.", r"model.layers.\1.self_attn.k_proj."),
    (r"^blk\.(\d+)\.attn_v\.", r"model.layers.\1.self_attn.v_proj."),
    (r"^blk\.(\d+)\.attn_output\.", r"model.layers.\1.self_attn.o_proj."),
    (r"^blk\.(\d+)\.ffn_gate\.", r"model.layers.\1.mlp.gate_proj."),
    (r"^blk\.(\d+)\.ffn_up\.", r"model.layers.\1.mlp.up_proj."),
    (r"^blk\.(\d+)\.ffn_down\.", r"model.layers.\1.mlp.down_proj."),
]


class _Reader:
    def __init__(self, buf):
        self.buf, self.off = buf, 0

    def scalar(self, fmt):
        v = struct.unpack_from(fmt, self.buf, self.off)[0]
        self.off += struct.calcsize(fmt)
        return v

    def string(self):
        n = self.scalar("<Q")
        s = bytes(self.buf[self.off:self.off + n]).decode("utf-8", errors="replace")
        self.off += n
        return s

    def value(self, typ):
        if typ in _SCALARS:
            return self.scalar(_SCALARS[typ])
        if typ == 8:
            return self.string()
        if typ == 9:
            et = self.scalar("<I")
            n = self.scalar("<Q")
            return [self.value(et) for _ in range(n)]
        raise ValueError(f"unknown GGUF value type {typ}")


def read_gguf(path: str) -> Tuple[Dict[str, Any], Dict[str, torch.Tensor]]:
    f = open(path, "rb")
    mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    r = _Reader(mm)
    if r.scalar("<I") != GGUF_MAGIC:
        raise ValueError("not a GGUF file")
    version = r.scalar("<I")
    n_tensors, n_kv = r.scalar("<Q"), r.scalar("<Q")
    meta: Dict[str, Any] = {"gguf.version": version}
    for _ in range(n_kv):
        k = r.string()
        meta[k] = r.value(r.scalar("<I"))
    infos = []
    for _ in range(n_tensors):
        name = r.string()
        nd = r.scalar("<I")
        dims = [r.scalar("<Q") for _ in range(nd)]
        gtype = r.scalar("<I")
        off = r.scalar("<Q")
        infos.append((name, dims, gtype, off))
    align = int(meta.get("general.alignment", 32))
    base = (r.off + align - 1) // align * align
    tensors: Dict[str, torch.Tensor] = {}
    for name, dims, gtype, off in infos:
        if gtype not in _GGML_DTYPES:
            raise ValueError(f"GGUF tensor {name} uses quantised ggml type {gtype}: not supported")
        npdt, tdt = _GGML_DTYPES[gtype]
        shape = list(reversed(dims))  # ggml stores the fastest dimension first
        count = int(np.prod(shape)) if shape else 1
        arr = np.frombuffer(mm, dtype=npdt, count=count, offset=base + off).reshape(shape)
        t = torch.from_numpy(arr.copy())
        tensors[name] = t.view(torch.bfloat16) if tdt == torch.bfloat16 else t
    return meta, tensors


def unpermute_rope_rows(w: torch.Tensor, n_head: int) -> torch.Tensor:
    """llama.cpp's converter reorders the rows of q / k projections of Llama-architecture models so that its
    adjacent-pair rotary kernel matches the half-split convention of the original weights (rows [head][2][d/2] ->
    [head][d/2][2]); this is the inverse, giving back the Hugging Face row order."""
    rows = w.shape[0]
    return w.reshape(n_head, rows // n_head // 2, 2, *w.shape[1:]).swapaxes(1, 2).reshape(w.shape)


def iter_gguf(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    meta, tensors = read_gguf(path)
    arch = str(meta.get("general.architecture", ""))
    n_head = int(meta.get(f"{arch}.attention.head_count", 0) or 0)
    n_kv = int(meta.get(f"{arch}.attention.head_count_kv", n_head) or n_head)
    for name, t in tensors.items():
        if arch == "llama" and n_head and t.dim() == 2:
            if name.endswith("attn_q.weight"):
                t = unpermute_rope_rows(t, n_head)
            elif name.endswith("attn_k.weight"):
                t = unpermute_rope_rows(t, n_kv)
        hf = name
        for pat, rep in _NAME_MAP:
            hf = re.sub(pat, rep, hf)
        yield hf, t


def write_gguf(path: str, tensors: Dict[str, torch.Tensor], meta: Dict[str, Any] = None) -> None:
    """Writer for F32 / F16 / BF16 tensors (used by tests and by small conversions)."""
    meta = dict(meta or {})
    inv = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 30}
    out = bytearray()
    out += struct.pack("<IIQQ", GGUF_MAGIC, 3, len(tensors), len(meta))

    def wstr(s):
        b = s.encode()
        return struct.pack("<Q", len(b)) + b

    for k, v in meta.items():
        out += wstr(k)
        if isinstance(v, str):
            out += struct.pack("<I", 8) + wstr(v)
        elif isinstance(v, int):
            out += struct.pack("<Iq", 11, v)
        else:
            out += struct.pack("<If", 6, float(v))
    blobs, off = [], 0
    for name, t in tensors.items():
        t = t.contiguous()
        out += wstr(name) + struct.pack("<I", t.dim())
        for d in reversed(t.shape):
            out += struct.pack("<Q", d)
        out += struct.pack("<IQ", inv[t.dtype], off)
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        pad = (-len(raw)) % 32
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    out += b"\0" * ((-len(out)) % 32)
    with open(path, "wb") as f:
        f.write(bytes(out))
        for b in blobs:
            f.write(b)
