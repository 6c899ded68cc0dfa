"""Frozen low-bit linear weights: what the reference's ``training_precision`` "4bit" / "8bit" mean.

With those names the reference loads the student through bitsandbytes (classes/student/model.py:138-148, 194-201):
every ``nn.Linear`` of the decoder layers becomes an NF4 (block size 64, double quantisation) or int8 weight that is
not trainable, the LM head is left alone, and the optimizer only moves embeddings, norms and the head. This module
does the same with this package's own storage and kernels:

* ``quantize_nf4`` / ``quantize_int8``: packed weights (PyTorch, any device). NF4 follows the published code book;
  the second-level quantisation of the block maxima uses a linear int8 code per group of 256 blocks plus a global
  offset (bitsandbytes uses its dynamic 8-bit code there: same storage cost, slightly different rounding).
* ``FrozenQuantLinears``: owns the packed weights of a model's decoder layers and two rotating layer-sized buffers
  in the compute dtype. The layer's parameters are views of a buffer; ``materialize(layer)`` expands the packed
  weights into it just before the layer's forward and again before its backward (csrc/ops/quant.cu on CUDA, the
  PyTorch restatement on CPU). The parameters are frozen, so they have no gradient, no master copy and no
  optimizer state.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import _VP, _LL, _I, _F

_lib.register("b200_dequant_nf4", [_VP, _VP, _VP, _F, _VP, _LL, _VP])
_lib.register("b200_dequant_int8", [_VP, _VP, _VP, _LL, _I, _VP])

NF4 = torch.tensor([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
                    -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
                    0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
                    0.7229568362236023, 1.0])
BLOCK = 64          # values per absmax block
GROUP = 256         # blocks per second-level scale


def quantize_nf4(w: torch.Tensor) -> dict:
    """w: any shape, numel % 64 == 0. Returns the packed representation (tensors on w's device)."""
    n = w.numel()
    if n % BLOCK:
        raise ValueError(f"NF4 needs a multiple of {BLOCK} values, got {n}")
    x = w.detach().float().reshape(-1, BLOCK)
    absmax = x.abs().amax(dim=1).clamp_min(1e-12)
    code_book = NF4.to(x.device)
    # nearest code-book entry: thresholds halfway between neighbours
    mid = (code_book[1:] + code_book[:-1]) / 2
    q = torch.bucketize((x / absmax[:, None]).contiguous(), mid).to(torch.uint8)          # [blocks, 64] in 0..15
    packed = ((q[:, 0::2] << 4) | q[:, 1::2]).reshape(-1).contiguous()
    offset = float(absmax.mean())
    nb = absmax.numel()
    pad = (-nb) % GROUP
    a = torch.cat([absmax - offset, absmax.new_zeros(pad)]).reshape(-1, GROUP)
    scale = (a.abs().amax(dim=1) / 127.0).clamp_min(1e-20)
    acode = torch.round(a / scale[:, None]).clamp_(-127, 127).to(torch.int8).reshape(-1)[:nb].contiguous()
    return {"kind": "nf4", "shape": tuple(w.shape), "packed": packed, "absmax_code": acode,
            "absmax_scale": scale.float().contiguous(), "offset": offset}


def quantize_int8(w: torch.Tensor) -> dict:
    """w [rows, cols], cols % 16 == 0: row-wise absmax int8."""
    if w.dim() != 2 or w.shape[1] % 16:
        raise ValueError("int8 weights need a [rows, cols] matrix with cols % 16 == 0")
    x = w.detach().float()
    scale = (x.abs().amax(dim=1) / 127.0).clamp_min(1e-20)
    code = torch.round(x / scale[:, None]).clamp_(-127, 127).to(torch.int8).contiguous()
    return {"kind": "int8", "shape": tuple(w.shape), "code": code, "row_scale": scale.float().contiguous()}


def dequantize_reference(q: dict, dtype=torch.float32) -> torch.Tensor:
    """PyTorch restatement (the CPU path and the oracle of the kernels)."""
    if q["kind"] == "int8":
        return (q["code"].float() * q["row_scale"][:, None]).to(dtype).reshape(q["shape"])
    packed = q["packed"]
    nb = q["absmax_code"].numel()
    absmax = q["absmax_code"].float() * q["absmax_scale"].repeat_interleave(GROUP)[:nb] + q["offset"]
    codes = torch.stack([(packed >> 4), (packed & 15)], dim=1).reshape(-1, BLOCK).long()
    vals = NF4.to(packed.device)[codes] * absmax[:, None]
    return vals.to(dtype).reshape(q["shape"])


def dequantize_into(q: dict, out: torch.Tensor) -> None:
    """out (compute dtype, q's shape, contiguous) = dequantised weights; a kernel on CUDA for bf16 outputs."""
    if out.is_cuda and out.dtype == torch.bfloat16:
        lib = _lib.kernels()
        if q["kind"] == "nf4":
            _lib.check(lib.b200_dequant_nf4(_lib.ptr(q["packed"]), _lib.ptr(q["absmax_code"]), _lib.ptr(q["absmax_scale"]),
                                            float(q["offset"]), _lib.ptr(out), out.numel(), _lib.stream()), "b200_dequant_nf4")
        else:
            _lib.check(lib.b200_dequant_int8(_lib.ptr(q["code"]), _lib.ptr(q["row_scale"]), _lib.ptr(out), out.shape[0],
                                             out.shape[1], _lib.stream()), "b200_dequant_int8")
        return
    out.copy_(dequantize_reference(q, out.dtype))


def packed_bytes(q: dict) -> int:
    return sum(t.numel() * t.element_size() for t in q.values() if isinstance(t, torch.Tensor))


LINEARS = ("qkv_proj", "o_proj", "gate_up_proj", "down_proj")


class FrozenQuantLinears:
    """Quantises and freezes the decoder layers' linear weights of a ``LlamaModel`` in place (see module docstring)."""

    def __init__(self, model, kind: str):
        if kind not in ("nf4", "int8"):
            raise ValueError(kind)
        self.kind = kind
        self.model = model
        quantize = quantize_nf4 if kind == "nf4" else quantize_int8
        first = model.layers[0]
        dtype, dev = first.qkv_proj.dtype, first.qkv_proj.device
        sizes = [getattr(first, n).numel() for n in LINEARS]
        self._offsets = [sum(sizes[:i]) for i in range(len(sizes))]
        self._buffers = [torch.empty(sum(sizes), dtype=dtype, device=dev) for _ in range(2)]
        self.layers: list[dict] = []
        self._layer_of: dict[int, int] = {}
        with torch.no_grad():
            for i, layer in enumerate(model.layers):
                packed = {}
                for n, off in zip(LINEARS, self._offsets):
                    p = getattr(layer, n)
                    packed[n] = quantize(p.data)
                    p.requires_grad = False
                    p.data = self._buffers[i & 1][off:off + p.numel()].view(p.shape)
                self.layers.append(packed)
                self._layer_of[id(layer.first_param)] = i

    def materialize(self, layer_index: int) -> None:
        layer = self.model.layers[layer_index]
        with torch.no_grad():
            for n in LINEARS:
                dequantize_into(self.layers[layer_index][n], getattr(layer, n).data)

    def before_layer(self, first_param) -> None:
        """Hook form of ``materialize``: called with the layer's first parameter before its forward / backward."""
        i = self._layer_of.get(id(first_param))
        if i is not None:
            self.materialize(i)

    def dequantized(self, layer_index: int) -> dict[str, torch.Tensor]:
        """Fresh copies of one layer's matrices (checkpoint export)."""
        layer = self.model.layers[layer_index]
        out = {}
        for n in LINEARS:
            p = getattr(layer, n)
            t = torch.empty(p.shape, dtype=p.dtype, device=p.device)
            dequantize_into(self.layers[layer_index][n], t)
            out[n] = t
        return out

    def packed_bytes(self) -> int:
        return sum(packed_bytes(q) for layer in self.layers for q in layer.values())
