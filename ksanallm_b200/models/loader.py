"""Checkpoint -> per-rank canonical weights.

Input: an iterator of ``(hf_name, tensor)`` pairs from ``*.safetensors`` (mmap), ``pytorch_model*.bin``
or a synthetic generator. Output: a dict with the canonical internal names
(``model.layers.N.self_attn.query_key_value.weight`` fused per rank, ``...mlp.gate_up_proj.weight``,
``...mlp.experts.up_gate_proj.weight`` stacked, MLA ``fused_lora_a_proj / w_uk_t / w_uv`` ...),
tensor-parallel slices taken, expert-parallel experts selected and optional load-time quantisation
(bf16 -> fp8 128x128 block-scaled, bf16 -> int4 group-128) applied.

Reference: model_weight_loader.cpp:25-120, llama_model_weight_loader.cpp:91-280 (TP slicing, fused qkv),
new_deepseek_v3_weight_loader.cpp:154-186, 268-320, 383-497 (fp8 scale_inv, lora-a fusion, kv_b split for
absorption, expert stacking), python/weight_map/*.json (regex renames to Llama names).
"""
from __future__ import annotations

import glob
import json
import os
import re
from collections import defaultdict
from typing import Dict, Iterable, Iterator, List, Optional, Tuple

import torch

from ..config.model_config import ModelConfig
from ..ops import reference as ref

# Block-scaled e4m3 linear weights are kept with power-of-two scales (KSANA_FP8_POW2_SCALES=0: the checkpoint's own
# fp32 scales, which only the kernel with per-K-block promotion can take).
FP8_POW2_SCALES = os.environ.get("KSANA_FP8_POW2_SCALES", "1") != "0"

# ---------------------------------------------------------------------------------------------------
# name normalisation: architecture-specific HF names -> Llama-style names
# ---------------------------------------------------------------------------------------------------

_RENAMES: Dict[str, List[Tuple[str, str]]] = {
    "qwen3": [(r"\.q_norm\.", ".query_layernorm."), (r"\.k_norm\.", ".key_layernorm.")],
    "qwen3_moe": [(r"\.q_norm\.", ".query_layernorm."), (r"\.k_norm\.", ".key_layernorm.")],
    "mixtral": [(r"\.block_sparse_moe\.", ".mlp."), (r"\.w1\.", ".gate_proj."), (r"\.w2\.", ".down_proj."),
                (r"\.w3\.", ".up_proj.")],
    "deepseek_v2": [(r"\.shared_experts\.", ".shared_expert.")],
    "deepseek_v3": [(r"\.shared_experts\.", ".shared_expert.")],
    "kimi_k2": [(r"\.shared_experts\.", ".shared_expert.")],
    "qwen2_moe": [],
    "internlm2": [(r"^model\.tok_embeddings\.", "model.embed_tokens."), (r"^output\.", "lm_head."),
                  (r"\.attention\.wqkv\.", ".self_attn.wqkv."), (r"\.attention\.wo\.", ".self_attn.o_proj."),
                  (r"\.feed_forward\.w1\.", ".mlp.gate_proj."), (r"\.feed_forward\.w3\.", ".mlp.up_proj."),
                  (r"\.feed_forward\.w2\.", ".mlp.down_proj."), (r"\.attention_norm\.", ".input_layernorm."),
                  (r"\.ffn_norm\.", ".post_attention_layernorm.")],
    "baichuan": [(r"\.W_pack\.", ".wpack.")],
    "chatglm": [(r"^transformer\.embedding\.word_embeddings\.", "model.embed_tokens."),
                (r"^transformer\.encoder\.layers\.", "model.layers."),
                (r"^transformer\.encoder\.final_layernorm\.", "model.norm."),
                (r"^transformer\.output_layer\.", "lm_head."),
                (r"\.self_attention\.query_key_value\.", ".self_attn.wpack."),
                (r"\.self_attention\.dense\.", ".self_attn.o_proj."),
                (r"\.mlp\.dense_h_to_4h\.", ".mlp.gate_up_proj."), (r"\.mlp\.dense_4h_to_h\.", ".mlp.down_proj.")],
    "gpt2": [(r"^(transformer\.)?wte\.", "model.embed_tokens."), (r"^(transformer\.)?wpe\.", "model.embed_positions."),
             (r"^(transformer\.)?h\.", "model.layers."), (r"^(transformer\.)?ln_f\.", "model.norm."),
             (r"\.ln_1\.", ".input_layernorm."), (r"\.ln_2\.", ".post_attention_layernorm."),
             (r"\.attn\.c_attn\.", ".self_attn.wpack_t."), (r"\.attn\.c_proj\.", ".self_attn.o_proj_t."),
             (r"\.mlp\.c_fc\.", ".mlp.up_proj_t."), (r"\.mlp\.c_proj\.", ".mlp.down_proj_t.")],
    "hunyuan": [(r"\.mlp\.shared_mlp\.", ".mlp.shared_expert."), (r"\.query_layernorm\.", ".query_layernorm."),
                (r"\.mlp\.gate\.wg\.", ".mlp.gate.")],
}
# multimodal checkpoints: the language tower sits under model.language_model (transformers >= 4.52) or model.
_RENAMES["qwen2_vl"] = [(r"^model\.language_model\.", "model.")]
_RENAMES["internvl_chat"] = [(r"^language_model\.", "")] + _RENAMES["internlm2"]
_RENAMES["internvl"] = [(r"^model\.language_model\.", "model.")]  # transformers layout: qwen2 / llama tower
_RENAMES["internlmxcomposer2"] = _RENAMES["internlm2"]
_RENAMES["llama4"] = [(r"^language_model\.", ""), (r"\.feed_forward\.", ".mlp."), (r"\.router\.", ".gate.")]


def load_weight_map(model_dir: str, model_type: str) -> List[Tuple[str, str]]:
    """Optional ``<model_type>_weight_map.json`` in the model directory: {regex: replacement}."""
    path = os.path.join(model_dir or "", f"{model_type}_weight_map.json")
    if model_dir and os.path.isfile(path):
        with open(path, "r", encoding="utf-8") as f:
            return [(k, v) for k, v in json.load(f).items()]
    return []


def normalise_name(name: str, rules: List[Tuple[str, str]]) -> str:
    for pat, rep in rules:
        name = re.sub(pat, rep, name)
    return name


# ---------------------------------------------------------------------------------------------------
# checkpoint readers
# ---------------------------------------------------------------------------------------------------

def iter_checkpoint(model_dir: str) -> Iterator[Tuple[str, torch.Tensor]]:
    st = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if st:
        from safetensors import safe_open
        for path in st:
            with safe_open(path, framework="pt", device="cpu") as f:
                for k in f.keys():
                    yield k, f.get_tensor(k)
        return
    bins = sorted(glob.glob(os.path.join(model_dir, "pytorch_model*.bin"))) or \
        sorted(glob.glob(os.path.join(model_dir, "*.bin"))) or sorted(glob.glob(os.path.join(model_dir, "*.pt")))
    if bins:
        for path in bins:
            sd = torch.load(path, map_location="cpu", weights_only=True, mmap=True)
            for k, v in sd.items():
                yield k, v
        return
    ggufs = sorted(glob.glob(os.path.join(model_dir, "*.gguf")))
    if ggufs:
        from .gguf_reader import iter_gguf
        for path in ggufs:
            yield from iter_gguf(path)
        return
    raise FileNotFoundError(f"no *.safetensors / *.bin / *.gguf under {model_dir}")


def synthetic_checkpoint(cfg: ModelConfig, seed: int = 0, std: float = 0.02, device="cpu",
                         dtype: Optional[torch.dtype] = None,
                         expert_filter=None) -> Iterator[Tuple[str, torch.Tensor]]:
    """Random-init N(0, std) weights under plain HF Llama-style names (norm weights = 1). Every rank
    that iterates with the same seed sees identical tensors, so TP slices are consistent. Routed experts draw from a
    generator of their own per (layer, expert), so ``expert_filter(layer index, expert) -> bool`` can leave out the
    experts another rank owns without changing any other tensor: an expert-parallel rank of a 256-expert model
    generates 1/ep_size of the expert weights instead of all of them."""
    dtype = dtype or getattr(torch, cfg.torch_dtype, torch.bfloat16)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    cur = [gen]

    def rnd(*shape):
        return (torch.randn(*shape, generator=cur[0], device=device, dtype=torch.float32) * std).to(dtype)

    def ones(n):
        return torch.ones(n, device=device, dtype=dtype)

    H, d = cfg.hidden_size, cfg.head_dim
    yield "model.embed_tokens.weight", rnd(cfg.vocab_size, H)
    n_total = cfg.num_layers + cfg.num_nextn_predict_layers
    for i in range(n_total):
        p = f"model.layers.{i}"
        yield p + ".input_layernorm.weight", ones(H)
        yield p + ".post_attention_layernorm.weight", ones(H)
        a = p + ".self_attn"
        if cfg.use_mla:
            if cfg.q_lora_rank:
                yield a + ".q_a_proj.weight", rnd(cfg.q_lora_rank, H)
                yield a + ".q_a_layernorm.weight", ones(cfg.q_lora_rank)
                yield a + ".q_b_proj.weight", rnd(cfg.num_heads * cfg.q_head_dim, cfg.q_lora_rank)
            else:
                yield a + ".q_proj.weight", rnd(cfg.num_heads * cfg.q_head_dim, H)
            yield a + ".kv_a_proj_with_mqa.weight", rnd(cfg.kv_lora_rank + cfg.qk_rope_head_dim, H)
            yield a + ".kv_a_layernorm.weight", ones(cfg.kv_lora_rank)
            if cfg.index_topk:
                yield a + ".indexer.wq_b.weight", rnd(cfg.index_n_heads * cfg.index_head_dim, cfg.q_lora_rank)
                yield a + ".indexer.wk.weight", rnd(cfg.index_head_dim, H)
                yield a + ".indexer.k_norm.weight", ones(cfg.index_head_dim)
                yield a + ".indexer.k_norm.bias", rnd(cfg.index_head_dim)
                yield a + ".indexer.weights_proj.weight", rnd(cfg.index_n_heads, H)
            yield a + ".kv_b_proj.weight", rnd(cfg.num_heads * (cfg.qk_nope_head_dim + cfg.v_head_dim), cfg.kv_lora_rank)
            yield a + ".o_proj.weight", rnd(H, cfg.num_heads * cfg.v_head_dim)
        else:
            yield a + ".q_proj.weight", rnd(cfg.num_heads * d, H)
            if not (cfg.cla_share_factor and i % cfg.cla_share_factor):
                yield a + ".k_proj.weight", rnd(cfg.num_kv_heads * d, H)
                yield a + ".v_proj.weight", rnd(cfg.num_kv_heads * d, H)
            if cfg.qkv_bias:
                yield a + ".q_proj.bias", rnd(cfg.num_heads * d)
                yield a + ".k_proj.bias", rnd(cfg.num_kv_heads * d)
                yield a + ".v_proj.bias", rnd(cfg.num_kv_heads * d)
            if cfg.qk_norm:
                yield a + ".query_layernorm.weight", ones(d)
                yield a + ".key_layernorm.weight", ones(d)
            yield a + ".o_proj.weight", rnd(H, cfg.num_heads * d)
        m = p + ".mlp"
        if cfg.is_moe_layer(i) or (cfg.is_moe and i >= cfg.num_layers):
            I = cfg.moe_intermediate_size
            yield m + ".gate.weight", rnd(cfg.num_experts, H).float() if cfg.scoring_func == "sigmoid" else rnd(cfg.num_experts, H)
            if cfg.topk_method == "noaux_tc":
                yield m + ".gate.e_score_correction_bias", torch.zeros(cfg.num_experts, device=device, dtype=torch.float32)
            for e in range(cfg.num_experts):
                if expert_filter is not None and not expert_filter(i, e):
                    continue
                ge = torch.Generator(device=device)
                ge.manual_seed((seed * 1000003 + i * 65537 + e + 1) & 0x7FFFFFFFFFFF)
                cur[0] = ge
                yield f"{m}.experts.{e}.gate_proj.weight", rnd(I, H)
                yield f"{m}.experts.{e}.up_proj.weight", rnd(I, H)
                yield f"{m}.experts.{e}.down_proj.weight", rnd(H, I)
                cur[0] = gen
            if cfg.num_shared_experts:
                S = cfg.shared_expert_intermediate_size
                yield m + ".shared_expert.gate_proj.weight", rnd(S, H)
                yield m + ".shared_expert.up_proj.weight", rnd(S, H)
                yield m + ".shared_expert.down_proj.weight", rnd(H, S)
                if cfg.shared_expert_gate:
                    yield m + ".shared_expert_gate.weight", rnd(1, H)
        else:
            I = cfg.intermediate_size
            if cfg.gated_mlp:
                yield m + ".gate_proj.weight", rnd(I, H)
            yield m + ".up_proj.weight", rnd(I, H)
            yield m + ".down_proj.weight", rnd(H, I)
        if i >= cfg.num_layers:
            yield p + ".enorm.weight", ones(H)
            yield p + ".hnorm.weight", ones(H)
            yield p + ".eh_proj.weight", rnd(H, 2 * H)
            yield p + ".shared_head.norm.weight", ones(H)
    yield "model.norm.weight", ones(H)
    if not cfg.tie_word_embeddings:
        yield "lm_head.weight", rnd(cfg.vocab_size, H)


# ---------------------------------------------------------------------------------------------------
# sharding helpers
# ---------------------------------------------------------------------------------------------------

class QuantW:
    """A 4-bit group-quantised linear weight travelling through the loader in place of a dense tensor:
    ``q`` [N, K] uint8 values 0..15, ``scales`` / ``zeros`` [N, K / group] fp32, w = (q - zero) * scale.
    Supports exactly the operations the loader applies to weights (row / column slices, row concatenation), so
    tensor-parallel slicing and projection fusing keep the checkpoint's quantisation grid bit for bit.

    ``perm`` (act-order GPTQ): the stored columns are input channels ``perm[0], perm[1], ...`` (sorted by group, so
    groups are contiguous again); the layer then gathers its input the same way, y = W[:, perm] x[perm]. Row slices
    and concatenation of weights with the same permutation keep it; a K slice (row-parallel shards) cannot, because
    a rank's channels no longer form whole groups, and returns the dense weight."""

    dtype = torch.uint8

    def __init__(self, q: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, group: int,
                 perm: Optional[torch.Tensor] = None):
        self.q, self.scales, self.zeros, self.group, self.perm = q, scales, zeros, group, perm

    @property
    def shape(self):
        return self.q.shape

    def dim(self) -> int:
        return 2

    def rows(self, a: int, b: int) -> "QuantW":
        return QuantW(self.q[a:b], self.scales[a:b], self.zeros[a:b], self.group, self.perm)

    def cols(self, a: int, b: int):
        if a == 0 and b == self.q.shape[1]:
            return self
        if self.perm is not None:
            return self.dequant()[:, a:b]
        g = self.group
        if a % g or b % g:
            raise ValueError(f"a K slice [{a}, {b}) must fall on group boundaries (group {g})")
        return QuantW(self.q[:, a:b], self.scales[:, a // g:b // g], self.zeros[:, a // g:b // g], g)

    @staticmethod
    def cat0(parts):
        perms = [p.perm for p in parts]
        same = all(x is None for x in perms) or (all(x is not None for x in perms) and
                                                 all(torch.equal(perms[0], x) for x in perms[1:]))
        if not same:  # projections quantised with different channel orders cannot share one input gather
            return torch.cat([p.dequant() for p in parts], 0)
        return QuantW(torch.cat([p.q for p in parts], 0), torch.cat([p.scales for p in parts], 0),
                      torch.cat([p.zeros for p in parts], 0), parts[0].group, perms[0])

    def dequant(self) -> torch.Tensor:
        """The dense weight in the checkpoint's own input-channel order."""
        N, K = self.q.shape
        qf = self.q.float().view(N, K // self.group, self.group)
        w = ((qf - self.zeros.unsqueeze(-1)) * self.scales.unsqueeze(-1)).view(N, K)
        if self.perm is None:
            return w
        out = torch.empty_like(w)
        out[:, self.perm.long()] = w
        return out


_AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)  # nibble i of an AutoAWQ word holds column 8 * word + _AWQ_ORDER[i]


def _unpack_nibbles(packed: torch.Tensor, dim: int, order=None) -> torch.Tensor:
    """int32 words -> uint8 values 0..15, eight per word laid out along ``dim`` (nibble i -> position order[i])."""
    p = packed.to(torch.int64) & 0xFFFFFFFF
    parts = [((p >> (4 * i)) & 0xF).to(torch.uint8) for i in range(8)]
    if order is not None:
        inv = [0] * 8
        for i, o in enumerate(order):
            inv[o] = i
        parts = [parts[inv[c]] for c in range(8)]
    st = torch.stack(parts, dim=dim + 1)
    shape = list(packed.shape)
    shape[dim] *= 8
    return st.reshape(shape)


def unpack_gptq(qweight, qzeros, scales, g_idx, group: int, v1_zero_offset: bool):
    """AutoGPTQ layout: qweight [K/8, N] (packed along K), qzeros [K/g, N/8] (packed along N; the v1 format stores
    zero - 1), scales [K/g, N], g_idx [K]. Returns (QuantW or None, dense fp32 weight or None). Act-order checkpoints
    (``g_idx`` not ascending: channels were quantised in order of importance) keep their grid with the columns
    gathered group by group and the gather recorded in ``QuantW.perm``; only a ``g_idx`` whose groups are not all of
    the nominal size is returned dense. Reference: the g_idx handling of src/ksana_llm/models/quant/quant_weight.cpp
    and the act-order path of 3rdparty/LLM_kernels/csrc/kernels/nvidia/gptq_marlin/marlin_template.h:54-110, which
    permutes the activations on the way into the kernel; here the layer gathers them before the 4-bit GEMM."""
    q = _unpack_nibbles(qweight, 0).t().contiguous()                 # [N, K]
    z = _unpack_nibbles(qzeros, 1).t().contiguous().float()          # [N, K/g]
    if v1_zero_offset:
        z = z + 1.0
    sc = scales.float().t().contiguous()                             # [N, K/g]
    K = q.shape[1]
    if g_idx is not None:
        gi = g_idx.to(torch.int64)
        trivial = torch.equal(gi, torch.arange(K, device=gi.device) // group)
        if not trivial:
            perm = torch.argsort(gi, stable=True)
            if torch.equal(gi[perm], torch.arange(K, device=gi.device) // group):
                return QuantW(q[:, perm].contiguous(), sc, z, group, perm.to(torch.int32)), None
            w = (q.float() - z[:, gi]) * sc[:, gi]
            return None, w
    return QuantW(q, sc, z, group), None


def unpack_w4a8(packed: torch.Tensor, weight_scale: torch.Tensor) -> "QuantW":
    """ModelOpt / TensorRT-LLM W4A8_AWQ layout: ``weight`` [N / 2, K] bytes, two signed 4-bit values per byte along
    N (low nibble = even output row), ``weight_scale`` [N, K / group]; w = nibble * weight_scale. Re-expressed on
    the unsigned grid with zero point 8. Reference: models/weight_method/w4a8_awq_method.cpp:19-31, 154-196."""
    b = packed.view(torch.uint8)
    q = torch.stack((b & 0xF, b >> 4), 1).reshape(2 * b.shape[0], b.shape[1]) ^ 8  # two's complement -> offset 8
    sc = weight_scale.float()
    return QuantW(q, sc, torch.full_like(sc, 8.0), b.shape[1] // sc.shape[1])


def unpack_awq(qweight, qzeros, scales, group: int):
    """AutoAWQ GEMM layout: qweight [K, N/8], qzeros [K/g, N/8] (both packed along N in the AWQ nibble order),
    scales [K/g, N]."""
    q = _unpack_nibbles(qweight, 1, _AWQ_ORDER).t().contiguous()     # [N, K]
    z = _unpack_nibbles(qzeros, 1, _AWQ_ORDER).t().contiguous().float()
    return QuantW(q, scales.float().t().contiguous(), z, group)


def _rows(t, rank: int, size: int):
    n = t.shape[0] // size
    if isinstance(t, QuantW):
        return t.rows(rank * n, (rank + 1) * n)
    return t[rank * n:(rank + 1) * n]


def _cols(t, rank: int, size: int):
    n = t.shape[1] // size
    if isinstance(t, QuantW):
        return t.cols(rank * n, (rank + 1) * n)
    return t[:, rank * n:(rank + 1) * n]


def _cat0(parts):
    if any(isinstance(p, QuantW) for p in parts):
        if not all(isinstance(p, QuantW) for p in parts):
            parts = [p.dequant() if isinstance(p, QuantW) else p.float() for p in parts]
            return torch.cat(parts, 0)
        return QuantW.cat0(parts)
    return torch.cat(parts, 0)


def _kv_rows(t: torch.Tensor, rank: int, size: int, num_kv_heads: int, d: int) -> torch.Tensor:
    """KV heads are split across ranks; with fewer KV heads than ranks each head is replicated."""
    if num_kv_heads >= size:
        return _rows(t, rank, size)
    rep = size // num_kv_heads
    hidx = rank // rep
    if isinstance(t, QuantW):
        return t.rows(hidx * d, (hidx + 1) * d)
    return t[hidx * d:(hidx + 1) * d]


class WeightLoader:
    def __init__(self, cfg: ModelConfig, tp_rank: int = 0, tp_size: int = 1, device="cpu",
                 dtype: Optional[torch.dtype] = None, quantize: Optional[str] = None,
                 ep_rank: Optional[int] = None, ep_size: Optional[int] = None, model_dir: str = "",
                 layer_range: Optional[range] = None):
        self.cfg = cfg
        self.rank, self.size = tp_rank, tp_size
        self.ep_rank = tp_rank if ep_rank is None else ep_rank
        self.ep_size = tp_size if ep_size is None else ep_size
        self.device = torch.device(device)
        self.dtype = dtype or getattr(torch, cfg.torch_dtype, torch.bfloat16)
        self.quantize = quantize  # None | "fp8_block" | "int4"
        from .registry import resolve_family
        fam = resolve_family(cfg.model_type, model_dir) or cfg.model_type
        # multimodal wrappers keep the language tower under model.language_model.* / language_model.*
        generic = [(r"^model\.language_model\.model\.", "model."), (r"^model\.language_model\.lm_head\.", "lm_head."),
                   (r"^model\.language_model\.", "model."), (r"^language_model\.model\.", "model."),
                   (r"^language_model\.lm_head\.", "lm_head.")]
        self.rules = load_weight_map(model_dir, cfg.model_type) + generic + \
            (_RENAMES.get(cfg.model_type) or _RENAMES.get(fam, []))
        self.family = fam
        self.layer_range = layer_range
        # expert-parallel load balancing: EPLB_WEIGHT names a placement (or routing-count) file; experts are stored
        # in "physical" order (rank r hosts slots [r * E / ranks, ...)), the layer keeps the logical -> physical map
        # and applies it to the router's choices (reference: moe_layer.cpp:124-129, 416-422 expert map, tools/eplb)
        self.expert_perm: Dict[int, List[int]] = {}
        eplb = os.environ.get("EPLB_WEIGHT", "")
        if eplb and cfg.num_experts and self.ep_size > 1 and os.path.isfile(eplb):
            from ..tools.eplb import load_expert_permutations
            self.expert_perm = load_expert_permutations(eplb, cfg.num_experts, self.ep_size)
        self.out: Dict[str, torch.Tensor] = {}
        self._pending: Dict[str, Dict[str, torch.Tensor]] = defaultdict(dict)
        self._experts: Dict[str, Dict[Tuple[int, str], torch.Tensor]] = defaultdict(dict)
        self._qparts: Dict[str, Dict[str, torch.Tensor]] = defaultdict(dict)  # GPTQ / AWQ tensors of one linear
        self._expert_pqs: Dict[str, Dict[Tuple[int, str], torch.Tensor]] = defaultdict(dict)

    # ---- placement --------------------------------------------------------------------------------
    def _own(self, t: torch.Tensor) -> torch.Tensor:
        """Device-resident, contiguous and not a view into a larger storage (a TP slice must not keep
        the full tensor alive)."""
        t = t.to(self.device).contiguous()
        if t.untyped_storage().nbytes() > t.numel() * t.element_size():
            t = t.clone()
        return t

    def _put(self, name: str, t: torch.Tensor, keep_dtype: bool = False) -> None:
        if not keep_dtype and t.is_floating_point() and t.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
            t = t.to(self.dtype)
        self.out[name] = self._own(t)

    def _put_linear(self, prefix: str, w: torch.Tensor, scale_inv: Optional[torch.Tensor] = None) -> None:
        """Stores a linear weight, quantising at load time when requested. Norms, embeddings, the router
        and lm_head stay in the model dtype."""
        if isinstance(w, QuantW):
            # a GPTQ / AWQ checkpoint: keep its grid, only re-pack into this engine's word layout
            self.out[prefix + ".qweight"] = self._own(ref.pack_int4(w.q.to(torch.int32)))
            self.out[prefix + ".scales"] = self._own(w.scales.to(self.dtype))
            self.out[prefix + ".zeros"] = self._own(w.zeros.to(self.dtype))
            if w.perm is not None:
                self.out[prefix + ".perm"] = self._own(w.perm.to(torch.int32))
            return
        if scale_inv is not None:
            if FP8_POW2_SCALES and w.dim() == 2 and w.dtype == torch.float8_e4m3fn:
                # power-of-two block scales let the tensor core apply them (ops/cuda_fp8.py): one re-rounding at load
                w, scale_inv = ref.requant_fp8_block_ue8m0(w.to(self.device), scale_inv.to(self.device))
            self.out[prefix + ".weight"] = self._own(w)
            self.out[prefix + ".weight_scale_inv"] = self._own(scale_inv.float())
            return
        if self.quantize == "fp8_block" and w.dim() == 2 and w.shape[1] % 128 == 0:
            q, s = ref.quant_fp8_block_weight(w.to(self.device).float(), ue8m0=FP8_POW2_SCALES)
            self.out[prefix + ".weight"] = q.contiguous()
            self.out[prefix + ".weight_scale_inv"] = s.contiguous()
            return
        if self.quantize == "int4" and w.dim() == 2 and w.shape[1] % 128 == 0:
            p, s, z = ref.quant_int4_group(w.to(self.device).float())
            self.out[prefix + ".qweight"] = p.contiguous()
            self.out[prefix + ".scales"] = s.to(self.dtype).contiguous()
            self.out[prefix + ".zeros"] = z.to(self.dtype).contiguous()
            return
        self._put(prefix + ".weight", w)

    def owns_expert(self, layer_idx: int, logical_expert: int) -> bool:
        """Whether this rank keeps routed expert ``logical_expert`` of layer ``layer_idx`` (expert parallelism)."""
        if self.ep_size <= 1:
            return True
        if self.layer_range is not None and layer_idx not in self.layer_range and layer_idx < self.cfg.num_layers:
            return False
        perm = self._perm_of(f"model.layers.{layer_idx}")
        e = perm[logical_expert] if perm else logical_expert
        per = max(self.cfg.num_experts // self.ep_size, 1)
        return self.ep_rank * per <= e < (self.ep_rank + 1) * per

    def _perm_of(self, layer_name: str) -> Optional[List[int]]:
        """Logical -> physical expert permutation of ``model.layers.N`` (None: identity); also leaves the map in the
        weight dict for the MoE block."""
        if not self.expert_perm:
            return None
        li = int(layer_name.rsplit(".", 1)[1])
        perm = self.expert_perm.get(li)
        if perm is not None and f"{layer_name}.mlp.expert_perm" not in self.out:
            self.out[f"{layer_name}.mlp.expert_perm"] = torch.tensor(perm, dtype=torch.int32, device=self.device)
        return perm

    def _layer_of(self, name: str) -> Optional[int]:
        m = re.match(r"model\.layers\.(\d+)\.", name)
        return int(m.group(1)) if m else None

    # ---- main entry -------------------------------------------------------------------------------
    def _fp8_scalar_scales(self, tensors: Iterable[Tuple[str, torch.Tensor]]) -> Iterator[Tuple[str, torch.Tensor]]:
        """fp8 checkpoints with ONE scale per weight (``quant_method: fp8`` without ``weight_block_size``, and the
        compressed-tensors / FBGEMM layouts: ``X.weight`` e4m3 + ``X.weight_scale`` scalar, or one scale per output
        row, + an optional static ``X.input_scale``) are re-expressed for the rest of the loader: a per-tensor scale
        becomes a block-scale array holding that value in every 128 x 128 block, so the weight stays e4m3 and runs on
        the block-scaled GEMMs; row-wise scales do not fit the block grid and are folded into a 16-bit weight.
        Activations are quantised dynamically here, so ``input_scale`` is dropped. The reference's per-tensor path is
        src/ksana_llm/layers/nvidia/fp8_matmul_layer.cpp."""
        held: Dict[str, Dict[str, torch.Tensor]] = defaultdict(dict)

        def ready(stem):
            w, sc = held[stem]["weight"], held.pop(stem)["weight_scale"].float().reshape(-1)
            n, k = w.shape[-2], w.shape[-1]
            per_matrix = sc.numel() == 1 or (w.dim() == 3 and sc.numel() == w.shape[0])  # one scale per (expert) matrix
            if per_matrix:
                nb, kb = (n + 127) // 128, (k + 127) // 128
                if w.dim() == 3:
                    blocks = sc.expand(w.shape[0]).reshape(-1, 1, 1).expand(-1, nb, kb).contiguous()
                else:
                    blocks = torch.full((nb, kb), float(sc.item()), dtype=torch.float32)
                yield stem + ".weight", w
                yield stem + ".weight_scale_inv", blocks
            else:  # one scale per output row (of every expert)
                yield stem + ".weight", (w.float() * sc.to(w.device).reshape(*w.shape[:-1], 1)).to(self.dtype)

        for name, t in tensors:
            if name.endswith(".input_scale") or name.endswith(".activation_scale"):
                continue
            if name.endswith(".weight_scale") and not name.endswith("weight_scale_inv"):
                stem = name[:-len(".weight_scale")]
                held[stem]["weight_scale"] = t
            elif name.endswith(".weight") and self._fp8(t) and t.dim() >= 2:
                stem = name[:-len(".weight")]
                held[stem]["weight"] = t
            else:
                yield name, t
                continue
            if {"weight", "weight_scale"} <= set(held[stem]):
                yield from ready(stem)
        for stem, parts in held.items():
            if "weight" in parts:
                raise ValueError(f"fp8 weight {stem}.weight has no weight_scale in the checkpoint")

    def load(self, tensors: Iterable[Tuple[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
        if self.cfg.quant.method in ("fp8", "compressed-tensors", "fbgemm_fp8"):
            tensors = self._fp8_scalar_scales(tensors)
        for raw_name, t in tensors:
            if re.match(r"(model\.)?(visual|vision_tower|vision_model|vit|multi_modal_projector|mlp1)\.", raw_name):
                continue  # vision towers belong to the serving plugin, not to the language model
            name = normalise_name(raw_name, self.rules)
            li = self._layer_of(name)
            if li is not None and self.layer_range is not None and li not in self.layer_range \
                    and li < self.cfg.num_layers:
                continue
            self._consume(name, t)
        self._finish()
        return self.out

    def _consume(self, name: str, t: torch.Tensor) -> None:
        cfg, r, n = self.cfg, self.rank, self.size
        d = cfg.head_dim
        if name.endswith("rotary_emb.inv_freq"):
            return
        if name == "model.embed_tokens.weight":
            self._put(name, t)  # replicated: no collective on the embedding path
            return
        if name == "model.embed_positions.weight":
            self._put(name, t)
            return
        if name == "lm_head.weight":
            V = t.shape[0]
            if n > 1:
                pad = (-V) % n
                if pad:
                    t = torch.cat((t, torch.zeros(pad, t.shape[1], dtype=t.dtype, device=t.device)), 0)
                t = _rows(t, r, n)
            self._put(name, t)
            return
        if name.startswith("model.norm.") or "layernorm" in name or name.endswith("norm.weight") \
                or name.endswith("norm.bias") or ".enorm." in name or ".hnorm." in name:
            self._put(name, t)
            return
        if ".self_attn.indexer." in name:
            # sparse-attention indexer (DeepSeek-V3.2 / GLM DSA): small replicated projections; block-scaled fp8
            # tensors are dequantised once their scale has arrived
            stem, part = name.rsplit(".", 1)
            if part == "weight_scale_inv" or self._fp8(t):
                got = self._qparts["indexer:" + stem]
                got[part] = t
                if {"weight", "weight_scale_inv"} <= set(got):
                    del self._qparts["indexer:" + stem]
                    self._put(stem + ".weight", ref.dequant_fp8_block_weight(
                        got["weight"].to(self.device), got["weight_scale_inv"].to(self.device)).to(self.dtype))
            else:
                self._put(name, t)
            return
        m = re.match(r"(model\.layers\.\d+)\.(self_attn|mlp)\.(.*)$", name)
        if not m:
            mm = re.match(r"(model\.layers\.\d+)\.(eh_proj)\.(weight|weight_scale_inv)$", name)
            if mm:
                self._pending[mm.group(1) + ".eh_proj"][mm.group(3)] = t
            else:
                self._put(name, t)
            return
        layer, block, rest = m.groups()
        key = f"{layer}.{block}"
        # stacked experts (transformers >= 5 state dicts, fused-expert checkpoints):
        # experts.gate_up_proj [E, 2I, H] (gate rows, then up rows) and experts.down_proj [E, H, I]
        if rest in ("experts.gate_up_proj", "experts.down_proj") and t.dim() == 3:
            if self.family == "llama4":
                t = t.transpose(1, 2)  # Llama 4 keeps [E, in, out] for its batched matmul
            per = max(cfg.num_experts // self.ep_size, 1)
            perm = self._perm_of(layer)
            for le in range(t.shape[0]):
                e = perm[le] if perm else le  # physical slot of logical expert le
                if self.ep_size > 1 and not (self.ep_rank * per <= e < (self.ep_rank + 1) * per):
                    continue
                if rest == "experts.gate_up_proj":
                    half = t.shape[1] // 2
                    self._experts[key][(e, "gate_proj.weight")] = t[le, :half]
                    self._experts[key][(e, "up_proj.weight")] = t[le, half:]
                else:
                    self._experts[key][(e, "down_proj.weight")] = t[le]
            self._maybe_flush_experts(key)
            return
        if cfg.quant.method in ("w4a8_awq", "modelopt"):
            wm = re.match(r"(.+)\.(weight|weight_scale|weight_scale_2|input_scale|pre_quant_scale)$", rest)
            if wm and not isinstance(t, QuantW) and (wm.group(2) != "weight" or t.dtype in (torch.int8, torch.uint8)):
                self._consume_w4a8(layer, block, wm.group(1), wm.group(2), t)
                return
        # expert weights: experts.E.{gate,up,down}_proj.(weight|weight_scale_inv)
        em = re.match(r"experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.(weight|weight_scale_inv)$", rest)
        if em:
            e = int(em.group(1))
            perm = self._perm_of(layer)
            if perm:
                e = perm[e]
            per = max(cfg.num_experts // self.ep_size, 1)
            if self.ep_size > 1 and not (self.ep_rank * per <= e < (self.ep_rank + 1) * per):
                return
            self._experts[key][(e, em.group(2) + "." + em.group(3))] = t
            self._maybe_flush_experts(key)
            return
        qm = re.match(r"(.+)\.(qweight|qzeros|scales|g_idx)$", rest)
        if qm and cfg.quant.method in ("gptq", "awq"):
            stem, part = qm.groups()
            parts = self._qparts[f"{key}.{stem}"]
            parts[part] = t
            need = {"qweight", "qzeros", "scales"} | ({"g_idx"} if cfg.quant.method == "gptq" else set())
            if need <= set(parts):
                del self._qparts[f"{key}.{stem}"]
                self._consume_quantised(layer, block, stem, parts)
            return
        self._pending[key][rest] = t
        self._maybe_flush(key)

    def _consume_quantised(self, layer: str, block: str, stem: str, parts: Dict[str, torch.Tensor]) -> None:
        """All tensors of one GPTQ / AWQ linear have arrived: unpack them and continue as if the checkpoint had
        carried a ``.weight`` - a QuantW for the dense attention / FFN projections (grid preserved), a dequantised
        tensor for everything else (experts, MLA projections, act-order GPTQ)."""
        cfg = self.cfg
        g = cfg.quant.group_size if cfg.quant.group_size > 0 else parts["qweight"].shape[0] * 8
        dense = None
        if cfg.quant.method == "gptq":
            v1 = str(cfg.raw.get("quantization_config", {}).get("checkpoint_format", "gptq")) != "gptq_v2"
            qw, dense = unpack_gptq(parts["qweight"], parts["qzeros"], parts["scales"], parts.get("g_idx"), g, v1)
        else:
            qw = unpack_awq(parts["qweight"], parts["qzeros"], parts["scales"], g)
        self._emit_quantised(layer, block, stem, qw, dense, g)

    def _consume_w4a8(self, layer: str, block: str, stem: str, part: str, t: torch.Tensor) -> None:
        """One tensor of a W4A8_AWQ linear. The weights keep their 4-bit grid and run through the 4-bit GEMM with
        16-bit activations, so the two activation-side scalars (``input_scale``, ``weight_scale_2``: the fp8 range
        of activations and of the rescaled weights) are not needed; ``pre_quant_scale`` (AWQ's per-input-channel
        smoothing factor) multiplies the layer's input and is stored beside the weight."""
        if part in ("weight_scale_2", "input_scale"):
            return
        if part == "pre_quant_scale":
            self._put_pre_quant(layer, block, stem, t.float().flatten())
            return
        parts = self._qparts[f"{layer}.{block}.{stem}"]
        parts[part] = t
        if {"weight", "weight_scale"} <= set(parts):
            del self._qparts[f"{layer}.{block}.{stem}"]
            qw = unpack_w4a8(parts["weight"], parts["weight_scale"])
            self._emit_quantised(layer, block, stem, qw, None, qw.group)

    def _put_pre_quant(self, layer: str, block: str, stem: str, t: torch.Tensor) -> None:
        r, n = self.rank, self.size
        em = re.fullmatch(r"experts\.(\d+)\.(gate_proj|up_proj|down_proj)", stem)
        if em:
            e = int(em.group(1))
            perm = self._perm_of(layer)
            if perm:
                e = perm[e]
            per = max(self.cfg.num_experts // self.ep_size, 1)
            if self.ep_size > 1 and not (self.ep_rank * per <= e < (self.ep_rank + 1) * per):
                return
            if em.group(2) != "up_proj":  # (gate and up read the same input)
                self._expert_pqs[f"{layer}.{block}"][(e, "down_proj" if em.group(2) == "down_proj" else "up_gate_proj")] = t
            return
        if self.cfg.use_mla and block == "self_attn":
            raise NotImplementedError("pre_quant_scale on multi-head latent attention projections is not supported")
        pre, _, leaf = stem.rpartition(".")
        pre = pre + "." if pre else ""
        if leaf in ("k_proj", "v_proj", "up_proj"):
            return  # fused with q_proj / gate_proj, which read the same input
        if leaf in ("o_proj", "down_proj"):  # row-parallel: this rank's slice of the input channels
            k = t.numel() // n
            t = t[r * k:(r + 1) * k]
        leaf = {"q_proj": "query_key_value", "gate_proj": "gate_up_proj"}.get(leaf, leaf)
        self._put(f"{layer}.{block}.{pre}{leaf}.pre_quant_scale", t)

    def _emit_quantised(self, layer: str, block: str, stem: str, qw, dense, g: int) -> None:
        cfg = self.cfg
        keep_grid = (not cfg.use_mla and block in ("self_attn", "mlp") and
                     re.fullmatch(r"(shared_expert\.)?(q_proj|k_proj|v_proj|o_proj|gate_proj|up_proj|down_proj)", stem)
                     and (qw is not None) and qw.shape[1] % 128 == 0 and g % 64 == 0)
        # routed experts keep their 4-bit grid too (also under MLA): they are most of a MoE checkpoint's bytes
        # (not act-order ones: the stacked expert kernels have no per-expert input gather)
        keep_grid = keep_grid or (block == "mlp" and (qw is not None) and g % 64 == 0 and qw.shape[1] % g == 0 and
                                  qw.perm is None and
                                  bool(re.fullmatch(r"experts\.\d+\.(gate_proj|up_proj|down_proj)", stem)))
        value = qw if keep_grid else (dense if dense is not None else qw.dequant())
        if not isinstance(value, QuantW):
            value = value.to(self.dtype)
        self._consume(f"{layer}.{block}.{stem}.weight", value)

    # ---- streaming: a block is assembled as soon as all of its parts have arrived ----------------------
    @staticmethod
    def _fp8(t: torch.Tensor) -> bool:
        return t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2)

    def _have(self, p: Dict[str, torch.Tensor], stem: str, bias: bool = False) -> bool:
        w = p.get(stem + ".weight")
        if w is None:
            return False
        if self._fp8(w) and (stem + ".weight_scale_inv") not in p:
            return False
        if bias and (stem + ".bias") not in p:
            return False
        return True

    def _maybe_flush(self, key: str) -> None:
        cfg = self.cfg
        p = self._pending[key]
        if key.endswith(".self_attn"):
            if cfg.use_mla:
                # (the *_layernorm weights never enter the pending set: norm tensors are placed directly)
                ok = self._have(p, "kv_a_proj_with_mqa") and self._have(p, "kv_b_proj") and self._have(p, "o_proj")
                if cfg.q_lora_rank:
                    ok = ok and self._have(p, "q_a_proj") and self._have(p, "q_b_proj")
                else:
                    ok = ok and self._have(p, "q_proj")
                if ok:
                    self._finish_mla(key, self._pending.pop(key))
                return
            b = cfg.qkv_bias
            qkv = (self._have(p, "q_proj", b) and self._have(p, "k_proj", b) and self._have(p, "v_proj", b)) or \
                self._have(p, "wpack", b) or self._have(p, "wpack_t", b) or self._have(p, "wqkv", b)
            o = self._have(p, "o_proj", cfg.o_bias) or self._have(p, "o_proj_t", cfg.o_bias)
            if qkv and o:
                self._finish_attn(key, self._pending.pop(key))
            return
        if key.endswith(".mlp"):
            li = self._layer_of(key + ".")
            moe = cfg.is_moe_layer(li) or (cfg.is_moe and li >= cfg.num_layers)
            b = cfg.mlp_bias

            def ffn_ok(pre):
                return (self._have(p, pre + "gate_proj") and self._have(p, pre + "up_proj") and
                        self._have(p, pre + "down_proj")) or \
                    (self._have(p, pre + "gate_up_proj") and self._have(p, pre + "down_proj")) or \
                    (not cfg.gated_mlp and ((self._have(p, pre + "up_proj", b) and self._have(p, pre + "down_proj", b)) or
                                            (self._have(p, pre + "up_proj_t", b) and self._have(p, pre + "down_proj_t", b))))
            if moe:
                ok = "gate.weight" in p
                if cfg.topk_method == "noaux_tc":
                    ok = ok and "gate.e_score_correction_bias" in p
                if cfg.num_shared_experts:
                    ok = ok and ffn_ok("shared_expert.")
                    if cfg.shared_expert_gate:
                        ok = ok and "shared_expert_gate.weight" in p
            else:
                ok = ffn_ok("")
            if ok:
                self._finish_mlp(key, self._pending.pop(key))

    def _maybe_flush_experts(self, key: str) -> None:
        ex = self._experts[key]
        per = max(self.cfg.num_experts // max(self.ep_size, 1), 1) if self.ep_size > 1 else self.cfg.num_experts
        first = next(iter(ex.values()))
        want = per * 3 * (2 if any(self._fp8(t) for t in ex.values()) else 1)
        if len(ex) >= want:
            self._finish_experts(key, self._experts.pop(key))

    # ---- assembling fused tensors --------------------------------------------------------------------
    def _finish(self) -> None:
        cfg, r, n = self.cfg, self.rank, self.size
        d = cfg.head_dim
        for key, parts in list(self._pending.items()):
            if key.endswith(".eh_proj"):
                self._put_linear(key, parts["weight"], parts.get("weight_scale_inv"))
            elif key.endswith(".self_attn"):
                if cfg.use_mla:
                    self._finish_mla(key, parts)
                else:
                    self._finish_attn(key, parts)
            else:
                self._finish_mlp(key, parts)
        for key, ex in list(self._experts.items()):
            self._finish_experts(key, ex)
        for key, pq in self._expert_pqs.items():  # [E_local, K] per projection, in local expert order
            for name in ("up_gate_proj", "down_proj"):
                ids = sorted(e for e, nm in pq if nm == name)
                if ids:
                    self._put(f"{key}.experts.{name}.pre_quant_scale", torch.stack([pq[(e, name)] for e in ids]))
        self._expert_pqs.clear()
        self._pending.clear()
        self._experts.clear()

    def _finish_attn(self, key: str, p: Dict[str, torch.Tensor]) -> None:
        cfg, r, n = self.cfg, self.rank, self.size
        d, hq, hk = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
        for suffix in ("weight", "bias", "weight_scale_inv"):
            q = k = v = None
            if f"q_proj.{suffix}" in p and f"k_proj.{suffix}" not in p and cfg.cla_share_factor:
                # cross-layer attention: this layer projects queries only and reuses the K/V projections of the
                # preceding layer that owns them (reference: modules/attention/cross_layer_attention.cpp:16-24)
                fused = _rows(p[f"q_proj.{suffix}"], r, n)
                if suffix == "bias":
                    self._put(f"{key}.query_key_value.bias", fused)
                elif suffix == "weight":
                    self._put_linear(f"{key}.query_key_value", fused)
                continue
            if f"q_proj.{suffix}" in p:
                q, k, v = p[f"q_proj.{suffix}"], p[f"k_proj.{suffix}"], p[f"v_proj.{suffix}"]
            elif f"wpack.{suffix}" in p:  # [q | k | v] stacked rows (Baichuan W_pack, ChatGLM)
                w = p[f"wpack.{suffix}"]
                q, k, v = w[:hq * d], w[hq * d:(hq + hk) * d], w[(hq + hk) * d:]
            elif f"wpack_t.{suffix}" in p:  # GPT-2 Conv1D: [in, out]
                w = p[f"wpack_t.{suffix}"]
                w = w.t() if w.dim() == 2 else w
                q, k, v = w[:hq * d], w[hq * d:(hq + hk) * d], w[(hq + hk) * d:]
            elif f"wqkv.{suffix}" in p:  # InternLM2: per KV group [q*g | k | v]
                w = p[f"wqkv.{suffix}"]
                g = hq // hk
                w = w.view(hk, g + 2, d, *w.shape[1:])
                q = w[:, :g].reshape(hq * d, *w.shape[3:])
                k = w[:, g].reshape(hk * d, *w.shape[3:])
                v = w[:, g + 1].reshape(hk * d, *w.shape[3:])
            if q is None:
                continue
            if suffix == "weight_scale_inv":
                # block-scaled fp8 qkv: slice in units of 128 rows
                qs, ks, vs = _rows(q, r, n), _kv_rows(k, r, n, hk, max(d // 128, 1)), _kv_rows(v, r, n, hk, max(d // 128, 1))
                self.out[f"{key}.query_key_value.weight_scale_inv"] = torch.cat((qs, ks, vs), 0).float().to(self.device)
                continue
            fused = _cat0((_rows(q, r, n), _kv_rows(k, r, n, hk, d), _kv_rows(v, r, n, hk, d)))
            if suffix == "bias":
                self._put(f"{key}.query_key_value.bias", fused)
            elif fused.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
                self.out[f"{key}.query_key_value.weight"] = fused.to(self.device).contiguous()
            else:
                self._put_linear(f"{key}.query_key_value", fused)
        o_w = p.get("o_proj.weight")
        if o_w is None and "o_proj_t.weight" in p:
            o_w = p["o_proj_t.weight"].t()
        if o_w is not None:
            s = p.get("o_proj.weight_scale_inv")
            self._put_linear(f"{key}.o_proj", _cols(o_w, r, n), None if s is None else _cols(s, r, n))
        ob = p.get("o_proj.bias", p.get("o_proj_t.bias"))
        if ob is not None:
            self._put(f"{key}.o_proj.bias", ob)

    def _finish_mla(self, key: str, p: Dict[str, torch.Tensor]) -> None:
        cfg, r, n = self.cfg, self.rank, self.size
        h = cfg.num_heads
        dn, dr, dv, rk = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank

        def deq(nm):
            w = p[nm + ".weight"]
            s = p.get(nm + ".weight_scale_inv")
            if s is not None:
                w = ref.dequant_fp8_block_weight(w.to(self.device), s.to(self.device))
            return w

        kv_a = p["kv_a_proj_with_mqa.weight"]
        kv_a_s = p.get("kv_a_proj_with_mqa.weight_scale_inv")
        if cfg.q_lora_rank:
            q_a, q_a_s = p["q_a_proj.weight"], p.get("q_a_proj.weight_scale_inv")
            fused = torch.cat((q_a, kv_a), 0)
            fs = None
            if q_a_s is not None and kv_a_s is not None and q_a.shape[0] % 128 == 0:
                fs = torch.cat((q_a_s, kv_a_s), 0)
            elif q_a_s is not None:
                fused = torch.cat((deq("q_a_proj"), deq("kv_a_proj_with_mqa")), 0)
            self._put_linear(f"{key}.fused_lora_a_proj", fused, fs)
            qb, qbs = p["q_b_proj.weight"], p.get("q_b_proj.weight_scale_inv")
            self._put_linear(f"{key}.q_b_nope_rope_proj", _rows(qb, r, n), None if qbs is None else _rows(qbs, r, n))
        else:
            self._put_linear(f"{key}.fused_lora_a_proj", kv_a, kv_a_s)
            qp, qps = p["q_proj.weight"], p.get("q_proj.weight_scale_inv")
            self._put_linear(f"{key}.q_proj", _rows(qp, r, n), None if qps is None else _rows(qps, r, n))
        # kv_b: [h * (dn + dv), rk] -> absorbed w_uk_t [h, dn, rk] and w_uv [h, rk, dv] (always dequantised)
        kvb = deq("kv_b_proj").to(self.device).float().view(h, dn + dv, rk)
        hl = h // n
        kvb = kvb[r * hl:(r + 1) * hl]
        self._put(f"{key}.w_uk_t", kvb[:, :dn, :].contiguous())
        self._put(f"{key}.w_uv", kvb[:, dn:, :].transpose(1, 2).contiguous())
        ow, ows = p["o_proj.weight"], p.get("o_proj.weight_scale_inv")
        self._put_linear(f"{key}.o_proj", _cols(ow, r, n), None if ows is None else _cols(ows, r, n))

    def _finish_mlp(self, key: str, p: Dict[str, torch.Tensor]) -> None:
        cfg, r, n = self.cfg, self.rank, self.size
        for pre in ("", "shared_expert."):
            gate, up, down = p.get(pre + "gate_proj.weight"), p.get(pre + "up_proj.weight"), p.get(pre + "down_proj.weight")
            if up is None and pre + "up_proj_t.weight" in p:
                up, down = p[pre + "up_proj_t.weight"].t(), p[pre + "down_proj_t.weight"].t()
            if pre + "gate_up_proj.weight" in p:  # already fused [gate | up] rows (ChatGLM, Phi-3 style)
                gu = p[pre + "gate_up_proj.weight"]
                half = gu.shape[0] // 2
                gate, up = gu[:half], gu[half:]
            if up is None:
                continue
            gs, us, ds = (p.get(pre + f"{x}_proj.weight_scale_inv") for x in ("gate", "up", "down"))
            if gate is not None:
                fused = _cat0((_rows(gate, r, n), _rows(up, r, n)))
                fs = None if gs is None else torch.cat((_rows(gs, r, n), _rows(us, r, n)), 0)
                self._put_linear(f"{key}.{pre}gate_up_proj", fused, fs)
            else:
                self._put_linear(f"{key}.{pre}up_proj", _rows(up, r, n), None if us is None else _rows(us, r, n))
            self._put_linear(f"{key}.{pre}down_proj", _cols(down, r, n), None if ds is None else _cols(ds, r, n))
            for b in ("up_proj", "up_proj_t"):
                if pre + b + ".bias" in p:
                    self._put(f"{key}.{pre}up_proj.bias", _rows(p[pre + b + ".bias"], r, n))
            for b in ("down_proj", "down_proj_t"):
                if pre + b + ".bias" in p:
                    self._put(f"{key}.{pre}down_proj.bias", p[pre + b + ".bias"])
        if "gate.weight" in p:
            self._put(f"{key}.gate.weight", p["gate.weight"], keep_dtype=p["gate.weight"].dtype == torch.float32)
        if "gate.e_score_correction_bias" in p:
            self._put(f"{key}.gate.e_score_correction_bias", p["gate.e_score_correction_bias"].float(), keep_dtype=True)
        if "shared_expert_gate.weight" in p:
            self._put(f"{key}.shared_expert_gate.weight", p["shared_expert_gate.weight"])

    def _finish_experts(self, key: str, ex: Dict[Tuple[int, str], torch.Tensor]) -> None:
        ids = sorted({e for e, _ in ex})
        if isinstance(ex[(ids[0], "gate_proj.weight")], QuantW):
            # GPTQ / AWQ experts: stacked packed words + group scales / zeros, [gate | up] rows fused per expert
            gus = [QuantW.cat0((ex[(e, "gate_proj.weight")], ex[(e, "up_proj.weight")])) for e in ids]
            dns = [ex[(e, "down_proj.weight")] for e in ids]
            for name, qs in (("up_gate_proj", gus), ("down_proj", dns)):
                self.out[f"{key}.experts.{name}.qweight"] = self._own(
                    torch.stack([ref.pack_int4(q.q.to(torch.int32)) for q in qs]))
                self.out[f"{key}.experts.{name}.scales"] = self._own(torch.stack([q.scales for q in qs]).to(self.dtype))
                self.out[f"{key}.experts.{name}.zeros"] = self._own(torch.stack([q.zeros for q in qs]).to(self.dtype))
            return
        has_scale = (ids[0], "gate_proj.weight_scale_inv") in ex
        gu = torch.stack([torch.cat((ex[(e, "gate_proj.weight")], ex[(e, "up_proj.weight")]), 0) for e in ids])
        dn = torch.stack([ex[(e, "down_proj.weight")] for e in ids])
        if has_scale:
            self.out[f"{key}.experts.up_gate_proj.weight"] = gu.to(self.device).contiguous()
            self.out[f"{key}.experts.down_proj.weight"] = dn.to(self.device).contiguous()
            self.out[f"{key}.experts.up_gate_proj.weight_scale_inv"] = torch.stack(
                [torch.cat((ex[(e, "gate_proj.weight_scale_inv")], ex[(e, "up_proj.weight_scale_inv")]), 0)
                 for e in ids]).float().to(self.device).contiguous()
            self.out[f"{key}.experts.down_proj.weight_scale_inv"] = torch.stack(
                [ex[(e, "down_proj.weight_scale_inv")] for e in ids]).float().to(self.device).contiguous()
        elif self.quantize == "fp8_block":
            E = gu.shape[0]
            q1, s1, q2, s2 = [], [], [], []
            for e in range(E):
                a, b = ref.quant_fp8_block_weight(gu[e].to(self.device).float())
                c, dd = ref.quant_fp8_block_weight(dn[e].to(self.device).float())
                q1.append(a); s1.append(b); q2.append(c); s2.append(dd)
            self.out[f"{key}.experts.up_gate_proj.weight"] = torch.stack(q1)
            self.out[f"{key}.experts.up_gate_proj.weight_scale_inv"] = torch.stack(s1)
            self.out[f"{key}.experts.down_proj.weight"] = torch.stack(q2)
            self.out[f"{key}.experts.down_proj.weight_scale_inv"] = torch.stack(s2)
        else:
            self._put(f"{key}.experts.up_gate_proj.weight", gu)
            self._put(f"{key}.experts.down_proj.weight", dn)


def load_model_weights(cfg: ModelConfig, model_dir: str = "", tp_rank: int = 0, tp_size: int = 1, device="cpu",
                       dtype: Optional[torch.dtype] = None, quantize: Optional[str] = None,
                       synthetic_seed: Optional[int] = None, synthetic_std: float = 0.02,
                       layer_range: Optional[range] = None, ep_rank: Optional[int] = None,
                       ep_size: Optional[int] = None) -> Dict[str, torch.Tensor]:
    """``ep_rank`` / ``ep_size`` shard the routed experts independently of the tensor-parallel slicing (attention
    data parallelism: tp_size 1, experts spread over the DP ranks)."""
    loader = WeightLoader(cfg, tp_rank, tp_size, device, dtype, quantize, ep_rank=ep_rank, ep_size=ep_size,
                          model_dir=model_dir, layer_range=layer_range)
    if synthetic_seed is not None or not model_dir:
        src = synthetic_checkpoint(cfg, synthetic_seed or 0, synthetic_std, device=device, dtype=dtype,
                                   expert_filter=loader.owns_expert if loader.ep_size > 1 else None)
        return loader.load(src)
    # ENABLE_MODEL_CACHE=1: the processed (sliced, fused, quantised) tensors of this rank are kept as one
    # safetensors file and reloaded at the next start instead of running the loader again
    from . import model_cache
    tag = "_".join(str(x) for x in (quantize or "plain", str(loader.dtype).split(".")[-1],
                                    f"ep{loader.ep_rank}of{loader.ep_size}",
                                    f"l{layer_range.start}-{layer_range.stop}" if layer_range is not None else "all"))
    cached = model_cache.cache_file(model_dir, tp_rank, tp_size, tag)
    if cached and os.path.isfile(cached):
        return model_cache.load_weights(cached, device)
    weights = loader.load(iter_checkpoint(model_dir))
    if cached:
        model_cache.save_weights(cached, weights)
    return weights
