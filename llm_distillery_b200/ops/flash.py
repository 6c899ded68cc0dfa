"""Bindings of the sm_100a flash-attention kernels (csrc/ops/flash_attn_fwd.cu, flash_attn_bwd.cu)."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import _VP, _I, _LL

_lib.register("b200_flash_attn_fwd", [_VP, _VP, _VP, _I, _I, _I, _I, _I, _VP])
_lib.register("b200_flash_attn_fwd_cached", [_VP, _VP, _VP, _LL, _VP, _VP, _I, _I, _I, _I, _I, _I, _VP])
_lib.register("b200_flash_attn_bwd", [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _VP])
_lib.register("b200_dq_convert_rope", [_VP, _VP, _VP, _VP, _VP, _LL, _I, _I, _LL, _VP])
_lib.register("b200_flash_attn_bwd_rope", [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _VP])


def flash_attn_fwd(qkv: torch.Tensor, B: int, L: int, H: int, Hkv: int, d: int):
    if qkv.dtype != torch.bfloat16 or not qkv.is_contiguous():
        raise TypeError("flash_attn_fwd: qkv must be contiguous bf16")
    T = B * L
    out = torch.empty((T, H * d), dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty((H, T), dtype=torch.float32, device=qkv.device)
    rc = _lib.kernels().b200_flash_attn_fwd(_lib.ptr(qkv), _lib.ptr(out), _lib.ptr(lse), B, L, H, Hkv, d, _lib.stream())
    _lib.check(rc, "b200_flash_attn_fwd")
    return out, lse


def flash_attn_bwd(dout, qkv, out, lse, B, L, H, Hkv, d, rope=None):
    """``rope = (pos, cos, sin)``: the inverse rotary embedding of the query heads' gradient is applied where the fp32
    dQ accumulator is converted (the key heads' gradient is left to the caller)."""
    if not dout.is_contiguous():
        dout = dout.contiguous()
    dqkv = torch.empty_like(qkv)
    # scratch: delta[h, t] = sum_d dout * out (pre-pass) and the fp32 dQ accumulator the key-block CTAs reduce into
    delta = torch.empty_like(lse)
    dq_acc = torch.empty((B * L, H * d), dtype=torch.float32, device=qkv.device)
    if rope is not None:
        pos, cos, sin = rope
        rc = _lib.kernels().b200_flash_attn_bwd_rope(_lib.ptr(dout), _lib.ptr(qkv), _lib.ptr(out), _lib.ptr(lse),
                                                     _lib.ptr(delta), _lib.ptr(dqkv), _lib.ptr(dq_acc), _lib.ptr(pos),
                                                     _lib.ptr(cos), _lib.ptr(sin), B, L, H, Hkv, d, _lib.stream())
        _lib.check(rc, "b200_flash_attn_bwd_rope")
        return dqkv
    rc = _lib.kernels().b200_flash_attn_bwd(_lib.ptr(dout), _lib.ptr(qkv), _lib.ptr(out), _lib.ptr(lse), _lib.ptr(delta),
                                            _lib.ptr(dqkv), _lib.ptr(dq_acc), B, L, H, Hkv, d, _lib.stream())
    _lib.check(rc, "b200_flash_attn_bwd")
    return dqkv


def flash_attn_fwd_cached(qkv, k_cache, v_cache, B, L, q_off, H, Hkv, d):
    if qkv.dtype != torch.bfloat16 or not (qkv.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise TypeError("flash_attn_fwd_cached: contiguous bf16 tensors expected")
    if k_cache.shape != v_cache.shape or k_cache.shape[0] != B or k_cache.shape[2] != Hkv * d:
        raise ValueError("key / value caches must be [B, rows, Hkv*d]")
    out = torch.empty((B * L, H * d), dtype=qkv.dtype, device=qkv.device)
    rc = _lib.kernels().b200_flash_attn_fwd_cached(_lib.ptr(qkv), _lib.ptr(k_cache), _lib.ptr(v_cache), k_cache.shape[1],
                                                   _lib.ptr(out), None, B, L, q_off, H, Hkv, d, _lib.stream())
    _lib.check(rc, "b200_flash_attn_fwd_cached")
    return out
