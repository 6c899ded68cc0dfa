"""A GPTQ- or AWQ-quantised teacher folder loads as the bf16 model it encodes (the packing below is the test's own inverse of
the documented layout, so a mistake in either direction shows)."""
import json
import os

import numpy as np
import pytest
import torch

from llm_distillery_b200.ckpt import gptq
from llm_distillery_b200.ckpt.hf import load_hf_model, load_hf_state_dict, load_tp_weights
from llm_distillery_b200.models.llama import preset
from llm_distillery_b200.utils import synthetic


def _pack_rows(vals: torch.Tensor, bits: int) -> torch.Tensor:      # [r * pack, c] -> int32 [r, c]
    pack = 32 // bits
    v = vals.to(torch.int64).reshape(-1, pack, vals.shape[1])
    word = torch.zeros(v.shape[0], v.shape[2], dtype=torch.int64)
    for j in range(pack):
        word |= v[:, j, :] << (bits * j)
    return torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)


def _quantize_linear(w: torch.Tensor, bits: int, group: int, act_order: bool, offset: int):
    """w [out, in] -> GPTQ tensors and the weight they encode."""
    out_f, in_f = w.shape
    groups = in_f // group
    g_idx = torch.arange(in_f) // group
    if act_order:
        g_idx = g_idx[torch.randperm(in_f, generator=torch.Generator().manual_seed(0))]
    wt = w.t().float()                                              # [in, out]
    qmax = (1 << bits) - 1
    scales = torch.empty(groups, out_f)
    zeros = torch.empty(groups, out_f, dtype=torch.int64)
    q = torch.empty(in_f, out_f, dtype=torch.int64)
    for g in range(groups):
        rows = (g_idx == g).nonzero().flatten()
        blk = wt[rows]
        lo, hi = blk.min(0).values, blk.max(0).values
        sc = ((hi - lo) / qmax).clamp_min(1e-8).half().float()
        zp = torch.round(-lo / sc).clamp(1, qmax).long()            # >= 1 so that "stored minus one" stays >= 0
        scales[g], zeros[g] = sc, zp
        q[rows] = torch.round(blk / sc + zp).clamp(0, qmax).long()
    deq = (scales[g_idx] * (q - zeros[g_idx]).float()).t().contiguous()
    qzeros = _pack_rows((zeros - offset).t().contiguous(), bits).t().contiguous()
    return {"qweight": _pack_rows(q, bits), "qzeros": qzeros, "scales": scales.half(), "g_idx": g_idx.to(torch.int32)}, deq


@pytest.mark.parametrize("bits,act_order,fmt", [(4, False, "gptq"), (4, True, "gptq"), (8, False, "gptq_v2"), (2, False, "gptq")])
def test_linear_round_trip(bits, act_order, fmt):
    torch.manual_seed(bits)
    w = torch.randn(48, 256) * 0.1
    t, deq = _quantize_linear(w, bits, 64, act_order, 0 if fmt == "gptq_v2" else 1)
    got = gptq.dequantize_linear(t["qweight"], t["qzeros"], t["scales"], t["g_idx"], bits, 64, 0 if fmt == "gptq_v2" else 1)
    assert torch.allclose(got, deq, atol=1e-6)
    if bits >= 4:
        assert (got - w).abs().max() < (0.2 if bits == 4 else 0.02)


def test_gptq_folder_loads_as_the_dequantised_model_and_exl2_is_refused(tmp_path):
    from safetensors.torch import save_file
    root = str(tmp_path)
    tok = os.path.join(root, "tok")
    synthetic.make_tokenizer(tok, 300)
    cfg = preset("plumbing-teacher", vocab_size=320, hidden_size=128, intermediate_size=256, max_position_embeddings=128)
    plain = synthetic.make_model_dir(os.path.join(root, "plain"), cfg, tok, seed=3)
    sd = load_hf_state_dict(plain)
    qsd, expect = {}, {}
    for k, v in sd.items():
        if k.endswith("proj.weight"):
            t, deq = _quantize_linear(v.float(), 4, 64, False, 1)
            base = k[: -len(".weight")]
            for name, tensor in t.items():
                qsd[f"{base}.{name}"] = tensor.contiguous()
            expect[k] = deq.to(torch.bfloat16)
        else:
            qsd[k] = v.contiguous()
            expect[k] = v
    qdir = os.path.join(root, "gptq")
    os.makedirs(qdir)
    save_file(qsd, os.path.join(qdir, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(plain, "config.json")) as f:
        conf = json.load(f)
    conf["quantization_config"] = {"quant_method": "gptq", "bits": 4, "group_size": 64, "desc_act": False}
    with open(os.path.join(qdir, "config.json"), "w") as f:
        json.dump(conf, f)
    got = load_hf_state_dict(qdir)
    assert set(got) == set(expect)
    for k in expect:
        assert torch.equal(got[k].to(torch.bfloat16), expect[k].to(torch.bfloat16)), k
    model = load_hf_model(qdir, dtype=torch.float32, device="cpu")
    ids = torch.randint(0, 300, (1, 16))
    with torch.no_grad():
        assert torch.isfinite(model.hidden_states(ids)).all()
    with pytest.raises(ValueError, match="quantised checkpoint"):
        load_tp_weights(qdir, 0, 2)
    with pytest.raises(ValueError, match="EXL2"):
        gptq.dequantize_state_dict({"model.layers.0.mlp.up_proj.q_weight": torch.zeros(1, dtype=torch.int32)}, {})


def _awq_quantize_linear(w: torch.Tensor, group: int):
    """w [out, in] -> AutoAWQ gemm tensors (packed with the packer's own loop over its order map, not with the
    loader's table) and the weight they encode."""
    out_f, in_f = w.shape
    wt = w.t().float()                                              # [in, out]
    groups = in_f // group
    blk = wt.reshape(groups, group, out_f)
    lo, hi = blk.min(1).values, blk.max(1).values                   # [groups, out]
    scales = ((hi - lo) / 15).clamp_min(1e-8).half().float()
    zeros = torch.round(-lo / scales).clamp(0, 15).long()
    g = torch.arange(in_f) // group
    q = torch.round(wt / scales[g] + zeros[g]).clamp(0, 15).long()
    deq = (scales[g] * (q - zeros[g]).float()).t().contiguous()

    def pack(vals):                                                 # [r, c] -> int32 [r, c / 8]
        word = torch.zeros(vals.shape[0], vals.shape[1] // 8, dtype=torch.int64)
        order_map = [0, 2, 4, 6, 1, 3, 5, 7]
        for col in range(vals.shape[1] // 8):
            for i in range(8):
                word[:, col] |= vals[:, col * 8 + order_map[i]] << (i * 4)
        return torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)
    return {"qweight": pack(q), "qzeros": pack(zeros), "scales": scales.half()}, deq


def test_awq_folder_loads_as_the_dequantised_model(tmp_path):
    from safetensors.torch import save_file
    torch.manual_seed(2)
    w = torch.randn(48, 256) * 0.1
    t, deq = _awq_quantize_linear(w, 64)
    got = gptq.dequantize_awq_linear(t["qweight"], t["qzeros"], t["scales"], 64)
    assert torch.allclose(got, deq, atol=1e-6) and (got - w).abs().max() < 0.2
    root = str(tmp_path)
    tok = os.path.join(root, "tok")
    synthetic.make_tokenizer(tok, 300)
    cfg = preset("plumbing-teacher", vocab_size=320, hidden_size=128, intermediate_size=256, max_position_embeddings=128)
    plain = synthetic.make_model_dir(os.path.join(root, "plain"), cfg, tok, seed=3)
    sd = load_hf_state_dict(plain)
    qsd, expect = {}, {}
    for k, v in sd.items():
        if k.endswith("proj.weight"):
            t, deq = _awq_quantize_linear(v.float(), 64)
            for name, tensor in t.items():
                qsd[f"{k[:-len('.weight')]}.{name}"] = tensor.contiguous()
            expect[k] = deq.to(torch.bfloat16)
        else:
            qsd[k] = v.contiguous()
            expect[k] = v
    qdir = os.path.join(root, "awq")
    os.makedirs(qdir)
    save_file(qsd, os.path.join(qdir, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(plain, "config.json")) as f:
        conf = json.load(f)
    conf["quantization_config"] = {"quant_method": "awq", "bits": 4, "group_size": 64, "version": "gemm", "zero_point": True}
    with open(os.path.join(qdir, "config.json"), "w") as f:
        json.dump(conf, f)
    got = load_hf_state_dict(qdir)
    assert set(got) == set(expect)
    for k in expect:
        assert torch.equal(got[k].to(torch.bfloat16), expect[k].to(torch.bfloat16)), k
    model = load_hf_model(qdir, dtype=torch.float32, device="cpu")
    with torch.no_grad():
        assert torch.isfinite(model.hidden_states(torch.randint(0, 300, (1, 16)))).all()
    with pytest.raises(ValueError, match="quantised checkpoint"):
        load_tp_weights(qdir, 0, 2)
    with pytest.raises(ValueError, match="gemm layout only"):
        gptq.dequantize_state_dict(qsd, {"quant_method": "awq", "bits": 4, "version": "gemv"})
