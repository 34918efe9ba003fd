"""GPTQ and AWQ checkpoint layouts: a tiny Llama is quantised, written in each tool's tensor layout under the usual
Hugging Face names, loaded back (single rank and tensor-parallel) and must reproduce the model built from the
dequantised dense weights."""
import pytest
import torch

from ksanallm_b200.config.model_config import model_config_from_dict
from ksanallm_b200.engine.step_input import make_step_input
from ksanallm_b200.models.loader import WeightLoader, synthetic_checkpoint
from ksanallm_b200.models.transformer import TransformerModel
from ksanallm_b200.ops import reference as ref

BASE = dict(model_type="llama", hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
            intermediate_size=256, vocab_size=300, torch_dtype="float32", max_position_embeddings=64)
GROUP = 64
AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


def _pack_along(vals: torch.Tensor, dim: int, order=None) -> torch.Tensor:
    """uint4 values -> int32 words, eight consecutive positions of ``dim`` per word."""
    v = vals.to(torch.int64).movedim(dim, -1)
    v = v.reshape(*v.shape[:-1], v.shape[-1] // 8, 8)
    out = torch.zeros(v.shape[:-1], dtype=torch.int64)
    for i in range(8):
        out |= v[..., (order[i] if order else i)] << (4 * i)
    out = torch.where(out >= 2 ** 31, out - 2 ** 32, out).to(torch.int32)
    return out.movedim(-1, dim)


def _quantised_checkpoint(fmt: str, act_order: bool = False):
    cfg = model_config_from_dict(BASE)
    dense, quant = [], []
    for name, w in synthetic_checkpoint(cfg, seed=5, dtype=torch.float32):
        is_linear = name.endswith("_proj.weight")
        if not is_linear:
            dense.append((name, w))
            quant.append((name, w))
            continue
        packed, scales, zeros = ref.quant_int4_group(w, GROUP)
        q = ref.unpack_int4(packed)                      # [N, K] values 0..15
        dense.append((name, ref.dequant_int4_group(packed, scales, zeros, GROUP)))
        stem = name[:-len(".weight")]
        N, K = q.shape
        if fmt == "gptq":
            g_idx = torch.arange(K, dtype=torch.int32) // GROUP
            qk = q
            if act_order:  # shuffle input channels inside the checkpoint: groups are no longer contiguous
                perm = torch.randperm(K, generator=torch.Generator().manual_seed(1))
                qk, g_idx = q[:, perm], g_idx[perm]
                dense[-1] = (name, dense[-1][1][:, perm])
            quant += [(stem + ".qweight", _pack_along(qk.t().contiguous(), 0)),
                      (stem + ".qzeros", _pack_along((zeros - 1).to(torch.int64).t().contiguous(), 1)),
                      (stem + ".scales", scales.t().contiguous().half()), (stem + ".g_idx", g_idx)]
            dense[-1] = (name, (qk.float() - zeros[:, g_idx.long()]) * scales.half().float()[:, g_idx.long()])
        else:
            quant += [(stem + ".qweight", _pack_along(q.t().contiguous(), 1, AWQ_ORDER)),
                      (stem + ".qzeros", _pack_along(zeros.to(torch.int64).t().contiguous(), 1, AWQ_ORDER)),
                      (stem + ".scales", scales.t().contiguous().half())]
            dense[-1] = (name, (q.float().view(N, K // GROUP, GROUP) - zeros.unsqueeze(-1)).mul(
                scales.half().float().unsqueeze(-1)).view(N, K))
    qc = dict(BASE, quantization_config=dict(quant_method=fmt, bits=4, group_size=GROUP, desc_act=act_order,
                                             zero_point=True))
    return model_config_from_dict(BASE), dense, model_config_from_dict(qc), quant


def _hidden(cfg, sd, **kw):
    w = WeightLoader(cfg, dtype=torch.float32, **kw).load(sd)
    model = TransformerModel(cfg, w, max_positions=64)
    T = 9
    meta = make_step_input(list(range(5, 5 + T)), list(range(T)), list(range(T)), [0, T], [T], [[0, 1]], device="cpu")
    return model.forward(meta, model.allocate_kv_cache(2, 16)), w


@pytest.mark.parametrize("fmt", ["gptq", "awq"])
def test_quantised_checkpoint_keeps_its_grid(fmt):
    cfg, dense, qcfg, quant = _quantised_checkpoint(fmt)
    want, _ = _hidden(cfg, dense)
    got, w = _hidden(qcfg, quant)
    assert "model.layers.0.self_attn.query_key_value.qweight" in w and "model.layers.0.mlp.down_proj.qweight" in w
    assert "model.layers.0.self_attn.query_key_value.weight" not in w
    assert (got - want).abs().max().item() < 1e-5


def test_gptq_act_order_keeps_its_four_bit_grid():
    """Act-order: input channels quantised in a shuffled order (``g_idx`` not ascending). The columns are stored group
    by group, the layer gathers its input the same way (``.perm``), the 4-bit grid survives bit for bit."""
    cfg, dense, qcfg, quant = _quantised_checkpoint("gptq", act_order=True)
    want, _ = _hidden(cfg, dense)
    got, w = _hidden(qcfg, quant)
    for stem in ("self_attn.query_key_value", "self_attn.o_proj", "mlp.gate_up_proj", "mlp.down_proj"):
        p = f"model.layers.0.{stem}"
        assert p + ".qweight" in w and p + ".perm" in w and p + ".weight" not in w
        perm = w[p + ".perm"].long()
        assert torch.equal(torch.sort(perm).values, torch.arange(perm.numel()))
    assert (got - want).abs().max().item() < 1e-5


def test_gptq_act_order_tensor_parallel():
    """Column-parallel projections keep the grid (their K is whole); a row-parallel shard holds scattered members
    of every group and is stored dense."""
    cfg, dense, qcfg, quant = _quantised_checkpoint("gptq", act_order=True)
    for rank in range(2):
        wd = WeightLoader(cfg, tp_rank=rank, tp_size=2, dtype=torch.float32).load(dense)
        wq = WeightLoader(qcfg, tp_rank=rank, tp_size=2, dtype=torch.float32).load(quant)
        for stem in ("self_attn.query_key_value", "mlp.gate_up_proj"):
            p = f"model.layers.1.{stem}"
            deq = ref.dequant_int4_group(wq[p + ".qweight"], wq[p + ".scales"].float(), wq[p + ".zeros"].float(), GROUP)
            full = torch.empty_like(deq)
            full[:, wq[p + ".perm"].long()] = deq
            assert (full - wd[p + ".weight"]).abs().max().item() < 1e-6, (rank, stem)
        for stem in ("self_attn.o_proj", "mlp.down_proj"):
            p = f"model.layers.1.{stem}"
            assert p + ".qweight" not in wq
            assert (wq[p + ".weight"] - wd[p + ".weight"]).abs().max().item() < 1e-6, (rank, stem)


@pytest.mark.parametrize("fmt", ["gptq", "awq"])
def test_quantised_checkpoint_tensor_parallel_slices(fmt):
    cfg, dense, qcfg, quant = _quantised_checkpoint(fmt)
    for rank in range(2):
        wd = WeightLoader(cfg, tp_rank=rank, tp_size=2, dtype=torch.float32).load(dense)
        wq = WeightLoader(qcfg, tp_rank=rank, tp_size=2, dtype=torch.float32).load(quant)
        for stem in ("self_attn.query_key_value", "self_attn.o_proj", "mlp.gate_up_proj", "mlp.down_proj"):
            p = f"model.layers.1.{stem}"
            deq = ref.dequant_int4_group(wq[p + ".qweight"], wq[p + ".scales"].float(), wq[p + ".zeros"].float(), GROUP)
            assert deq.shape == wd[p + ".weight"].shape
            assert (deq - wd[p + ".weight"]).abs().max().item() < 1e-6, (rank, stem)


def test_fp8_block_scaled_experts_stay_fp8_and_match_dequantised_weights():
    """A DeepSeek-V3 style checkpoint whose expert (and dense) projections are e4m3 with 128 x 128 block scales: the
    experts stay in fp8, and the outputs agree with the same checkpoint dequantised to fp32 up to the activation
    quantisation (one scale per token per 128 channels) the fp8 GEMM applies."""
    import torch
    from ksanallm_b200.config.model_config import model_config_from_dict
    from ksanallm_b200.engine.step_input import make_step_input
    from ksanallm_b200.models.loader import WeightLoader, synthetic_checkpoint
    from ksanallm_b200.models.transformer import TransformerModel
    from ksanallm_b200.ops import reference as ref
    cfg = model_config_from_dict(dict(model_type="mixtral", hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                                      num_key_value_heads=2, intermediate_size=256, num_local_experts=4,
                                      num_experts_per_tok=2, vocab_size=300, torch_dtype="float32",
                                      max_position_embeddings=64))
    fp8, deq = [], []
    for k, v in synthetic_checkpoint(cfg, seed=3, std=0.05, dtype=torch.float32):
        if ".experts." in k and k.endswith("_proj.weight"):
            q, s = ref.quant_fp8_block_weight(v)
            fp8 += [(k, q), (k + "_scale_inv", s)]
            deq.append((k, ref.dequant_fp8_block_weight(q, s)))
        else:
            fp8.append((k, v))
            deq.append((k, v))
    w8 = WeightLoader(cfg, dtype=torch.float32).load(fp8)
    assert w8["model.layers.0.mlp.experts.up_gate_proj.weight"].dtype == torch.float8_e4m3fn
    assert w8["model.layers.0.mlp.experts.up_gate_proj.weight_scale_inv"].shape == (4, 4, 1)
    T = 12
    meta = make_step_input(list(range(5, 5 + T)), list(range(T)), list(range(T)), [0, T], [T], [[0, 1]], device="cpu")
    outs = []
    for w in (w8, WeightLoader(cfg, dtype=torch.float32).load(deq)):
        model = TransformerModel(cfg, w, max_positions=64)
        outs.append(model.forward(meta, model.allocate_kv_cache(2, 16)))
    err = (outs[0] - outs[1]).abs().max().item()
    assert 0 < err < 0.05 * outs[1].abs().max().item()


@pytest.mark.parametrize("fmt", ["gptq", "awq"])
def test_quantised_experts_keep_their_grid(fmt):
    """A MoE checkpoint whose expert projections are GPTQ / AWQ tensors: the experts stay packed (stacked words +
    scales + zeros per expert) and the model equals the one built from the dequantised experts."""
    base = dict(model_type="mixtral", hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, intermediate_size=128, num_local_experts=4, num_experts_per_tok=2,
                vocab_size=300, torch_dtype="float32", max_position_embeddings=64)
    cfg = model_config_from_dict(base)
    dense, quant = [], []
    for name, w in synthetic_checkpoint(cfg, seed=5, dtype=torch.float32):
        if ".experts." not in name:
            dense.append((name, w))
            quant.append((name, w))
            continue
        packed, scales, zeros = ref.quant_int4_group(w, GROUP)
        q = ref.unpack_int4(packed)
        stem = name[:-len(".weight")]
        N, K = q.shape
        deq = (q.float().view(N, K // GROUP, GROUP) - zeros.unsqueeze(-1)).mul(scales.half().float().unsqueeze(-1)).view(N, K)
        dense.append((name, deq))
        if fmt == "gptq":
            quant += [(stem + ".qweight", _pack_along(q.t().contiguous(), 0)),
                      (stem + ".qzeros", _pack_along((zeros - 1).to(torch.int64).t().contiguous(), 1)),
                      (stem + ".scales", scales.t().contiguous().half()),
                      (stem + ".g_idx", torch.arange(K, dtype=torch.int32) // GROUP)]
        else:
            quant += [(stem + ".qweight", _pack_along(q.t().contiguous(), 1, AWQ_ORDER)),
                      (stem + ".qzeros", _pack_along(zeros.to(torch.int64).t().contiguous(), 1, AWQ_ORDER)),
                      (stem + ".scales", scales.t().contiguous().half())]
    qcfg = model_config_from_dict(dict(base, quantization_config=dict(quant_method=fmt, bits=4, group_size=GROUP,
                                                                      desc_act=False, zero_point=True)))
    want, _ = _hidden(cfg, dense)
    got, w = _hidden(qcfg, quant)
    assert w["model.layers.0.mlp.experts.up_gate_proj.qweight"].shape == (4, 256, 16)
    assert "model.layers.0.mlp.experts.up_gate_proj.weight" not in w
    assert torch.allclose(got, want, atol=2e-4)


def _w4a8_tensors(name, w, with_pre=True, seed=0):
    """One linear in the ModelOpt W4A8_AWQ layout and the dense weight it stands for (smoothing factor folded in)."""
    g = torch.Generator().manual_seed(seed)
    N, K = w.shape
    pre = (torch.rand(K, generator=g) + 0.5) if with_pre else torch.ones(K)
    target = w / pre                                            # AWQ: W' = W / s, x' = x * s
    scale = target.view(N, K // GROUP, GROUP).abs().amax(-1).clamp_min(1e-8) / 7.0
    q = (target.view(N, K // GROUP, GROUP) / scale.unsqueeze(-1)).round().clamp(-8, 7)
    deq = (q * scale.unsqueeze(-1)).view(N, K) * pre            # what the layer computes on an un-smoothed input
    qi = q.view(N, K).to(torch.int8)
    packed = ((qi[0::2] & 0xF) | ((qi[1::2] & 0xF) << 4)).to(torch.uint8)   # two output rows per byte
    stem = name[:-len(".weight")]
    out = [(stem + ".input_scale", torch.tensor(0.02)), (stem + ".weight", packed),
           (stem + ".weight_scale", scale), (stem + ".weight_scale_2", torch.tensor(0.01))]
    if with_pre:
        out.insert(1, (stem + ".pre_quant_scale", pre))
    return out, deq


@pytest.mark.parametrize("moe", [False, True])
def test_w4a8_awq_checkpoint_runs_on_its_four_bit_grid(moe, tmp_path):
    """ModelOpt W4A8_AWQ: [N / 2, K] bytes of signed nibbles + group scales + per-channel smoothing factors. The
    weights stay 4-bit (16-bit activations), q/k/v and gate/up share one smoothing vector, row-parallel inputs are
    sliced with their weights, and the model equals the one built from the dequantised weights - also split over two
    tensor-parallel ranks. hf_quant_config.json selects the method."""
    import json
    from ksanallm_b200.config.model_config import load_model_config
    base = dict(BASE, intermediate_size=128)
    if moe:
        base = dict(base, model_type="mixtral", num_local_experts=4, num_experts_per_tok=2)
    (tmp_path / "config.json").write_text(json.dumps(base))
    (tmp_path / "hf_quant_config.json").write_text(json.dumps(
        {"producer": {"name": "modelopt"}, "quantization": {"quant_algo": "W4A8_AWQ", "group_size": GROUP,
                                                           "exclude_modules": ["lm_head"]}}))
    qcfg = load_model_config(str(tmp_path))
    assert qcfg.quant.method == "w4a8_awq"
    cfg = model_config_from_dict(base)
    dense, quant = [], []
    shared_pre = {}
    for i, (name, w) in enumerate(synthetic_checkpoint(cfg, seed=5, dtype=torch.float32)):
        if not name.endswith("_proj.weight"):
            dense.append((name, w))
            quant.append((name, w))
            continue
        # projections reading the same input carry the same smoothing vector
        group_key = name.replace("k_proj", "q_proj").replace("v_proj", "q_proj").replace("up_proj", "gate_proj")
        seed = shared_pre.setdefault(group_key, i)
        ts, deq = _w4a8_tensors(name, w, seed=seed)
        quant += ts
        dense.append((name, deq))
    want, _ = _hidden(cfg, dense)
    got, w = _hidden(qcfg, quant)
    assert "model.layers.0.self_attn.query_key_value.qweight" in w
    assert "model.layers.0.self_attn.o_proj.pre_quant_scale" in w
    if moe:
        assert w["model.layers.0.mlp.experts.up_gate_proj.qweight"].shape == (4, 256, 16)
        assert w["model.layers.0.mlp.experts.down_proj.pre_quant_scale"].shape == (4, 128)
    assert torch.allclose(got, want, atol=3e-4), (got - want).abs().max()
    for rank in range(2):  # row-parallel inputs: the smoothing vector is sliced with the weight's input channels
        wq = WeightLoader(qcfg, tp_rank=rank, tp_size=2, dtype=torch.float32).load(quant)
        wd = WeightLoader(cfg, tp_rank=rank, tp_size=2, dtype=torch.float32).load(dense)
        p = "model.layers.1.self_attn.o_proj"
        deq = ref.dequant_int4_group(wq[p + ".qweight"], wq[p + ".scales"].float(), wq[p + ".zeros"].float(), GROUP)
        assert torch.allclose(deq * wq[p + ".pre_quant_scale"].float(), wd[p + ".weight"], atol=1e-5)


@pytest.mark.parametrize("per_channel", [False, True])
def test_fp8_checkpoint_with_one_scale_per_weight(per_channel):
    """``quant_method: fp8`` without block sizes: e4m3 weights with a scalar ``weight_scale`` (kept e4m3, the scale
    spread over the 128 x 128 block grid) or one scale per output row (folded into a dense weight); static
    ``input_scale`` entries are ignored."""
    cfg = model_config_from_dict(BASE)
    qcfg = model_config_from_dict(dict(BASE, quantization_config=dict(quant_method="fp8", activation_scheme="static")))
    dense, quant = [], []
    for name, w in synthetic_checkpoint(cfg, seed=7, dtype=torch.float32):
        if not name.endswith("_proj.weight"):
            dense.append((name, w))
            quant.append((name, w))
            continue
        amax = w.abs().amax(dim=1, keepdim=True) if per_channel else w.abs().amax()
        scale = (amax / 448.0).clamp_min(1e-8)
        q = (w / scale).clamp(-448, 448).to(torch.float8_e4m3fn)
        dense.append((name, q.float() * scale))
        stem = name[:-len(".weight")]
        quant += [(stem + ".input_scale", torch.tensor(0.02)), (name, q),
                  (stem + ".weight_scale", scale.reshape(-1) if per_channel else scale.reshape(()))]
    want, _ = _hidden(cfg, dense)
    got, w = _hidden(qcfg, quant)
    k = "model.layers.0.mlp.down_proj"
    if per_channel:
        assert w[k + ".weight"].dtype == torch.float32 and (k + ".weight_scale_inv") not in w
        assert (got - want).abs().max().item() < 1e-5
    else:
        assert w[k + ".weight"].dtype == torch.float8_e4m3fn and w[k + ".weight_scale_inv"].shape == (1, 2)
        # the weights are the checkpoint's (re-rounded once onto power-of-two block scales); activations are
        # quantised per token and 128 channels at run time, which the dense reference is not
        assert (got - want).abs().max().item() < 0.15 * want.abs().max().item()
        assert (got - want).abs().mean().item() < 0.02 * want.abs().max().item()
    # tensor-parallel slices load too (this tiny model's shards are narrower than a 128-wide scale block, so only
    # the row-wise form, which ends up dense, can be cut here)
    if per_channel:
        for rank in range(2):
            WeightLoader(qcfg, tp_rank=rank, tp_size=2, dtype=torch.float32).load(quant)
