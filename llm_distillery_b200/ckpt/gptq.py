"""GPTQ- and AWQ-quantised checkpoints (AutoGPTQ / Optimum and AutoAWQ layouts) as teachers.

The reference loads its teachers through ExLlamaV2, which takes fp16, GPTQ and EXL2 folders alike
(classes/teacher/inference_worker.py:38-51). Here a GPTQ folder is dequantised once, while it is being loaded, into
the bf16 weights that the tcgen05 kernels run on: a 70 B teacher is 131 GiB in bf16, which one B200 holds, so nothing
is gained by keeping 4-bit weights resident, and the collected distributions are those of the quantised model exactly.

Layout per linear layer ``X`` (bits in {2, 4, 8}; ``pack = 32 // bits`` values per int32, lowest bits first):
    X.qweight int32 [in / pack, out]      value of input channel i: (qweight[i // pack, o] >> bits * (i % pack)) & mask
    X.qzeros  int32 [groups, out / pack]  zero point of output channel o, stored minus one (AutoGPTQ v1)
    X.scales  fp16  [groups, out]
    X.g_idx   int32 [in]                  group of each input channel (absent: i // group_size)
    weight[o, i] = scales[g, o] * (q[i, o] - (zeros[g, o] + 1)),  g = g_idx[i]
``quantization_config.checkpoint_format == "gptq_v2"`` stores the zero points without the offset.
AWQ (``quant_method == "awq"``, version ``gemm``, 4 bits) uses the same three tensor names, packed along the OUTPUT
dimension with the eight values of a word in the order 0, 2, 4, 6, 1, 3, 5, 7, and zero points without an offset:
    X.qweight int32 [in, out / 8]   X.qzeros int32 [groups, out / 8]   X.scales fp16 [groups, out]
    weight[o, i] = scales[i // group_size, o] * (q[i, o] - zeros[i // group_size, o])
EXL2 folders (variable bit rate, ``q_weight`` / ``q_scale`` / ``q_groups`` tensors) are refused with a message.
"""
from __future__ import annotations

import json
import os

import torch


def quantization_config(path: str) -> dict | None:
    cfg_path = os.path.join(path, "config.json")
    if not os.path.exists(cfg_path):
        return None
    with open(cfg_path, encoding="utf-8") as f:
        cfg = json.load(f)
    q = cfg.get("quantization_config")
    if q is None and os.path.exists(os.path.join(path, "quantize_config.json")):
        with open(os.path.join(path, "quantize_config.json"), encoding="utf-8") as f:
            q = dict(json.load(f), quant_method="gptq")
    if q is None and os.path.exists(os.path.join(path, "quant_config.json")):      # AutoAWQ's own file: w_bit, q_group_size
        with open(os.path.join(path, "quant_config.json"), encoding="utf-8") as f:
            q = dict(json.load(f), quant_method="awq")
    return q


def unpack_rows(packed: torch.Tensor, bits: int) -> torch.Tensor:
    """int32 [r, c] holding 32 // bits values per word along dim 0 -> int32 [r * pack, c]."""
    pack = 32 // bits
    shifts = torch.arange(pack, device=packed.device, dtype=torch.int32) * bits
    vals = (packed.to(torch.int32)[:, None, :] >> shifts[None, :, None]) & ((1 << bits) - 1)
    return vals.reshape(packed.shape[0] * pack, packed.shape[1])


def unpack_cols(packed: torch.Tensor, bits: int) -> torch.Tensor:
    """int32 [r, c] packed along dim 1 -> int32 [r, c * pack]."""
    pack = 32 // bits
    shifts = torch.arange(pack, device=packed.device, dtype=torch.int32) * bits
    vals = (packed.to(torch.int32)[:, :, None] >> shifts[None, None, :]) & ((1 << bits) - 1)
    return vals.reshape(packed.shape[0], packed.shape[1] * pack)


def dequantize_linear(qweight, qzeros, scales, g_idx, bits: int, group_size: int, zero_offset: int = 1) -> torch.Tensor:
    """Returns the HF-layout weight [out, in] in fp32."""
    if bits not in (2, 4, 8):
        raise ValueError(f"GPTQ with {bits}-bit weights is not supported (2, 4 and 8 are)")
    q = unpack_rows(qweight, bits)                              # [in, out]
    n_in = q.shape[0]
    zeros = unpack_cols(qzeros, bits)[:, : scales.shape[1]] + zero_offset   # [groups, out]
    if g_idx is None:
        gs = group_size if group_size and group_size > 0 else n_in
        g_idx = torch.arange(n_in, device=q.device) // gs
    g = g_idx.long()
    w = scales.float()[g] * (q - zeros[g]).float()              # [in, out]
    return w.t().contiguous()


_AWQ_NIBBLE_OF_COLUMN = (0, 4, 1, 5, 2, 6, 3, 7)     # output channel c of a word's eight sits in nibble _AWQ_...[c]


def unpack_awq(packed: torch.Tensor) -> torch.Tensor:
    """int32 [r, c] holding eight 4-bit values per word in AWQ's order -> int32 [r, 8 c] in channel order."""
    nib = unpack_cols(packed, 4).reshape(packed.shape[0], packed.shape[1], 8)
    return nib[:, :, list(_AWQ_NIBBLE_OF_COLUMN)].reshape(packed.shape[0], packed.shape[1] * 8)


def dequantize_awq_linear(qweight, qzeros, scales, group_size: int) -> torch.Tensor:
    """AWQ ``gemm`` layout -> the HF-layout weight [out, in] in fp32."""
    q = unpack_awq(qweight)                                     # [in, out]
    n_in, n_out = q.shape
    if scales.shape[1] != n_out or qzeros.shape[1] * 8 != n_out:
        raise ValueError(f"AWQ tensors do not fit together: qweight {tuple(qweight.shape)}, qzeros "
                         f"{tuple(qzeros.shape)}, scales {tuple(scales.shape)} (only the gemm layout is read)")
    gs = group_size if group_size and group_size > 0 else n_in
    g = torch.arange(n_in, device=q.device) // gs
    w = scales.float()[g] * (q - unpack_awq(qzeros)[g]).float()
    return w.t().contiguous()


def dequantize_state_dict(sd: dict[str, torch.Tensor], qcfg: dict) -> dict[str, torch.Tensor]:
    """Replaces every ``X.qweight`` group of ``sd`` by ``X.weight`` (bf16); other tensors pass through."""
    if any(k.endswith(".q_weight") or k.endswith(".q_groups") for k in sd):
        raise ValueError("this is an EXL2 checkpoint (variable bit-rate q_weight / q_groups tensors): that format is not "
                         "read here - use the model's fp16 / bf16 safetensors or a GPTQ export")
    bits = int(qcfg.get("bits", qcfg.get("w_bit", 4)))
    group_size = int(qcfg.get("group_size", qcfg.get("q_group_size", 128)))
    awq = str(qcfg.get("quant_method", "gptq")).lower() == "awq"
    if awq and (bits != 4 or str(qcfg.get("version", "gemm")).lower() != "gemm"):
        raise ValueError(f"AWQ checkpoints are read in the 4-bit gemm layout only (this one: {bits} bits, version "
                         f"{qcfg.get('version')!r})")
    zero_offset = 0 if str(qcfg.get("checkpoint_format", "gptq")).lower() == "gptq_v2" else 1
    out = {}
    for k, v in sd.items():
        if k.endswith(".qweight"):
            base = k[: -len(".qweight")]
            if awq:
                out[base + ".weight"] = dequantize_awq_linear(v, sd[base + ".qzeros"], sd[base + ".scales"],
                                                              group_size).to(torch.bfloat16)
                continue
            w = dequantize_linear(v, sd[base + ".qzeros"], sd[base + ".scales"], sd.get(base + ".g_idx"), bits, group_size,
                                  zero_offset)
            out[base + ".weight"] = w.to(torch.bfloat16)
        elif k.endswith((".qzeros", ".scales", ".g_idx")) and (k.rsplit(".", 1)[0] + ".qweight") in sd:
            continue
        else:
            out[k] = v
    return out
