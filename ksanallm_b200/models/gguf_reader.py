"""GGUF reader (F32 / F16 / BF16 tensors and the common quantised GGML block types, dequantised at load) plus the
llama.cpp -> HF name mapping.

The reference loads ``*.gguf`` through its own file loader (src/ksana_llm/utils/gguf_file_tensor_loader.cpp) with
the renames of python/weight_map/llama_gguf_weight_map.json. Quantised tensors (Q4_0, Q4_1, Q5_0, Q5_1, Q8_0 and
the 256-element super-block types Q4_K, Q5_K, Q6_K: what Q8_0 / Q4_0 / Q4_K_M / Q5_K_M files contain) are expanded
to fp16 here; the loader then treats them like any 16-bit checkpoint (and can re-quantise them to this engine's own
fp8 / int4 formats). Other block types raise: a file is never silently mis-read.
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


# ---- quantised GGML block types -> fp32 ---------------------------------------------------------------------------
def _f16(b: np.ndarray) -> np.ndarray:
    """[n, 2] bytes -> [n, 1] fp32"""
    return np.ascontiguousarray(b).view(np.float16).astype(np.float32)


def _deq_q4_0(b):  # 32 weights: fp16 d | 16 bytes, low nibbles = weights 0..15, high nibbles = 16..31
    d, qs = _f16(b[:, 0:2]), b[:, 2:18]
    q = np.concatenate([qs & 0xF, qs >> 4], 1).astype(np.float32) - 8.0
    return d * q


def _deq_q4_1(b):  # fp16 d | fp16 m | 16 bytes: w = d * q + m
    d, m, qs = _f16(b[:, 0:2]), _f16(b[:, 2:4]), b[:, 4:20]
    return d * np.concatenate([qs & 0xF, qs >> 4], 1).astype(np.float32) + m


def _fifth_bits(qh_bytes):
    """[n, 4] bytes holding 32 bits -> [n, 32] array of 0 / 16 (the fifth bit of each weight)"""
    qh = np.ascontiguousarray(qh_bytes).view(np.uint32)  # [n, 1]
    return (((qh >> np.arange(32, dtype=np.uint32)[None, :]) & 1) << 4).astype(np.uint8)


def _deq_q5_0(b):  # fp16 d | 32 high bits | 16 bytes of low nibbles
    d, hi, qs = _f16(b[:, 0:2]), _fifth_bits(b[:, 2:6]), b[:, 6:22]
    q = (np.concatenate([qs & 0xF, qs >> 4], 1) | hi).astype(np.float32) - 16.0
    return d * q


def _deq_q5_1(b):  # fp16 d | fp16 m | 32 high bits | 16 bytes
    d, m, hi, qs = _f16(b[:, 0:2]), _f16(b[:, 2:4]), _fifth_bits(b[:, 4:8]), b[:, 8:24]
    return d * (np.concatenate([qs & 0xF, qs >> 4], 1) | hi).astype(np.float32) + m


def _deq_q8_0(b):  # fp16 d | 32 int8
    return _f16(b[:, 0:2]) * b[:, 2:34].view(np.int8).astype(np.float32)


def _k_scales(sc):
    """12 bytes -> (8 six-bit scales, 8 six-bit mins) of the K super-blocks: entries 0..3 sit in the low 6 bits of
    bytes 0..3 (scales) and 4..7 (mins); entries 4..7 take their low 4 bits from bytes 8..11 (scale: low nibble,
    min: high nibble) and their top 2 bits from the top 2 bits of bytes 0..3 / 4..7."""
    sc = sc.astype(np.uint8)
    s_lo, m_lo = sc[:, 0:4] & 63, sc[:, 4:8] & 63
    s_hi = (sc[:, 8:12] & 0xF) | ((sc[:, 0:4] >> 6) << 4)
    m_hi = (sc[:, 8:12] >> 4) | ((sc[:, 4:8] >> 6) << 4)
    return (np.concatenate([s_lo, s_hi], 1).astype(np.float32), np.concatenate([m_lo, m_hi], 1).astype(np.float32))


def _deq_q4_k(b):  # 256 weights: fp16 d | fp16 dmin | 12 scale bytes | 128 bytes; sub-blocks of 32: w = d sc q - dmin m
    d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
    sc, mn = _k_scales(b[:, 4:16])
    qs = b[:, 16:144].reshape(-1, 4, 32)                      # 4 chunks of 64 weights: low nibbles, then high nibbles
    q = np.stack([qs & 0xF, qs >> 4], 2).reshape(-1, 8, 32).astype(np.float32)
    return ((d * sc)[:, :, None] * q - (dmin * mn)[:, :, None]).reshape(-1, 256)


def _deq_q5_k(b):  # fp16 d | fp16 dmin | 12 scale bytes | 32 bytes of fifth bits | 128 bytes of nibbles
    d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
    sc, mn = _k_scales(b[:, 4:16])
    qh = b[:, 16:48]                                          # bit j of byte l: fifth bit of weight l of sub-block j
    qs = b[:, 48:176].reshape(-1, 4, 32)
    q = np.stack([qs & 0xF, qs >> 4], 2).reshape(-1, 8, 32)
    hi = ((qh[:, None, :] >> np.arange(8, dtype=np.uint8)[None, :, None]) & 1) << 4
    q = (q | hi).astype(np.float32)
    return ((d * sc)[:, :, None] * q - (dmin * mn)[:, :, None]).reshape(-1, 256)


def _deq_q6_k(b):  # 128 bytes of low nibbles | 64 bytes of 2-bit tops | 16 int8 scales | fp16 d; w = d sc (q - 32)
    ql = b[:, 0:128].reshape(-1, 2, 64)
    qh = b[:, 128:192].reshape(-1, 2, 32)
    sc = b[:, 192:208].view(np.int8).astype(np.float32).reshape(-1, 2, 8)
    d = _f16(b[:, 208:210])
    lo = np.stack([ql[:, :, 0:32] & 0xF, ql[:, :, 32:64] & 0xF, ql[:, :, 0:32] >> 4, ql[:, :, 32:64] >> 4], 2)
    top = np.stack([(qh >> s) & 3 for s in (0, 2, 4, 6)], 2)              # [n, 2, 4, 32]
    q = (lo | (top << 4)).astype(np.float32) - 32.0
    # scales: one per 16 weights; quarter k of half h uses scales h * 8 + 2 k + (0 or 1)
    scale = np.repeat(sc.reshape(-1, 2, 4, 2), 16, axis=3)
    return (d[:, :, None, None] * scale * q).reshape(-1, 256)


# ggml type id -> (weights per block, bytes per block, decoder)
_GGML_QUANT = {2: (32, 18, _deq_q4_0), 3: (32, 20, _deq_q4_1), 6: (32, 22, _deq_q5_0), 7: (32, 24, _deq_q5_1),
               8: (32, 34, _deq_q8_0), 12: (256, 144, _deq_q4_k), 13: (256, 176, _deq_q5_k), 14: (256, 210, _deq_q6_k)}


def dequantize_ggml(raw: np.ndarray, gtype: int, shape) -> np.ndarray:
    """Raw bytes of a quantised tensor -> fp32 array of ``shape`` (row-major, rows are whole numbers of blocks)."""
    per, nbytes, fn = _GGML_QUANT[gtype]
    blocks = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1, nbytes)
    return fn(blocks).reshape(shape)

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
        shape = list(reversed(dims))  # ggml stores the fastest dimension first
        count = int(np.prod(shape)) if shape else 1
        if gtype in _GGML_QUANT:
            per, nbytes, _ = _GGML_QUANT[gtype]
            if not shape or shape[-1] % per:
                raise ValueError(f"GGUF tensor {name}: row length {shape[-1:]} is not a multiple of the block size {per}")
            raw = np.frombuffer(mm, dtype=np.uint8, count=count // per * nbytes, offset=base + off)
            tensors[name] = torch.from_numpy(dequantize_ggml(raw, gtype, shape)).to(torch.float16)
            continue
        if gtype not in _GGML_DTYPES:
            raise ValueError(f"GGUF tensor {name} uses ggml type {gtype}: not supported")
        npdt, tdt = _GGML_DTYPES[gtype]
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
    """Writer for F32 / F16 / BF16 tensors (used by tests and by small conversions). A value may also be a tuple
    ``(ggml type id, shape, raw block bytes)`` of an already quantised tensor."""
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
        if isinstance(t, tuple):
            gtype, shape, raw = t
            out += wstr(name) + struct.pack("<I", len(shape))
            for d in reversed(shape):
                out += struct.pack("<Q", d)
            out += struct.pack("<IQ", int(gtype), off)
            raw = bytes(raw)
            pad = (-len(raw)) % 32
            blobs.append(raw + b"\0" * pad)
            off += len(raw) + pad
            continue
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
