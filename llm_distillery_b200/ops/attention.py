"""Causal grouped-query attention over the fused QKV activation.

Layout: ``qkv`` is [T, (H + 2*Hkv) * d] with T = B * L tokens (sequence-major inside each batch row); columns
[0, H*d) hold Q, then K, then V. Output is [T, H*d]; ``lse`` is fp32 [H, T] (log-sum-exp of the scaled scores,
natural log), the only statistic the backward pass needs.

CUDA tensors run the sm_100a flash-attention kernels (csrc/ops/flash_attn.cu); CPU tensors run the plain
restatement below, which is also the oracle of the GPU tests.

Sliding-window layers (Mistral v0.1, Phi-3, the windowed layers of hybrid models): a query at position i sees the
keys j with i - window < j <= i. Up to ``window`` positions that IS causal attention and the paths above run. Longer
sequences take ``windowed_fwd`` / ``windowed_bwd`` below: PyTorch's scaled-dot-product attention under a band mask, on
either device - the flash kernels have no window, so this case is exact but runs at the library's speed. The same
path, without a window, serves heads of other sizes than 64 and 128 on a GPU (Gemma's 256).
"""
from __future__ import annotations

import math

import torch

from . import _lib


def _split(qkv: torch.Tensor, B: int, L: int, H: int, Hkv: int, d: int):
    q = qkv[:, : H * d].reshape(B, L, H, d)
    k = qkv[:, H * d: (H + Hkv) * d].reshape(B, L, Hkv, d)
    v = qkv[:, (H + Hkv) * d:].reshape(B, L, Hkv, d)
    return q, k, v


def attention_reference_fwd(qkv, B, L, H, Hkv, d):
    q, k, v = _split(qkv.float(), B, L, H, Hkv, d)
    g = H // Hkv
    k = k.repeat_interleave(g, dim=2)
    v = v.repeat_interleave(g, dim=2)
    s = torch.einsum("blhd,bmhd->bhlm", q, k) / math.sqrt(d)
    mask = torch.ones(L, L, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)  # [B,H,L]
    p = torch.exp(s - lse[..., None])
    o = torch.einsum("bhlm,bmhd->blhd", p, v).reshape(B * L, H * d)
    return o.to(qkv.dtype), lse.permute(1, 0, 2).reshape(H, B * L).contiguous()


def attention_reference_bwd(dout, qkv, out, lse, B, L, H, Hkv, d):
    q, k, v = _split(qkv.float(), B, L, H, Hkv, d)
    g = H // Hkv
    kk = k.repeat_interleave(g, dim=2)
    vv = v.repeat_interleave(g, dim=2)
    do = dout.float().reshape(B, L, H, d)
    o = out.float().reshape(B, L, H, d)
    scale = 1.0 / math.sqrt(d)
    s = torch.einsum("blhd,bmhd->bhlm", q, kk) * scale
    mask = torch.ones(L, L, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.exp(s - lse.reshape(H, B, L).permute(1, 0, 2)[..., None])
    dv = torch.einsum("bhlm,blhd->bmhd", p, do)
    dp = torch.einsum("blhd,bmhd->bhlm", do, vv)
    delta = (do * o).sum(-1).permute(0, 2, 1)  # [B,H,L]
    ds = p * (dp - delta[..., None]) * scale
    dq = torch.einsum("bhlm,bmhd->blhd", ds, kk)
    dk = torch.einsum("bhlm,blhd->bmhd", ds, q)
    dk = dk.reshape(B, L, Hkv, g, d).sum(3)
    dv = dv.reshape(B, L, Hkv, g, d).sum(3)
    dqkv = torch.cat([dq.reshape(B * L, H * d), dk.reshape(B * L, Hkv * d), dv.reshape(B * L, Hkv * d)], dim=1)
    return dqkv.to(qkv.dtype)


def _library_path(qkv: torch.Tensor, d: int) -> bool:
    """Heads the flash kernels do not take (they take 64 and 128) go to the library path on a GPU, e.g. Gemma's 256."""
    return qkv.is_cuda and d not in (64, 128)


def _band_mask(n_q: int, n_k: int, q_off: int, window: int, device) -> torch.Tensor:
    """[n_q, n_k] bool: key j visible to the query at position q_off + i."""
    qi = torch.arange(q_off, q_off + n_q, device=device)[:, None]
    kj = torch.arange(n_k, device=device)[None, :]
    return (kj <= qi) & (kj > qi - window)


def _sdpa_banded(q, k, v, q_off: int, window: int | None):
    """q [B, n_q, H, d], k / v [B, n_k, Hkv, d] -> [B, n_q, H, d]; ``window`` None: causal without a window."""
    causal = window is None and q_off == 0 and q.shape[1] == k.shape[1]       # plain causal: no mask tensor needed
    mask = None if causal else _band_mask(q.shape[1], k.shape[1], q_off, window or (q_off + q.shape[1]), q.device)
    g = q.shape[2] // k.shape[2]
    if g > 1:          # grouped queries: the key / value heads are repeated (differentiated through, in the backward)
        k, v = k.repeat_interleave(g, dim=2), v.repeat_interleave(g, dim=2)
    o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                         attn_mask=mask, is_causal=causal)
    return o.transpose(1, 2)


def windowed_fwd(qkv, B, L, H, Hkv, d, window: int | None):
    """Sliding-window attention of sequences longer than the window. Returns (out, lse placeholder): the backward
    below recomputes instead of using the log-sum-exp."""
    q, k, v = _split(qkv, B, L, H, Hkv, d)
    o = _sdpa_banded(q, k, v, 0, window).reshape(B * L, H * d).contiguous()
    return o, torch.zeros((H, B * L), dtype=torch.float32, device=qkv.device)


def windowed_bwd(dout, qkv, B, L, H, Hkv, d, window: int | None):
    """dqkv of ``windowed_fwd`` by differentiating its recomputation."""
    with torch.enable_grad():
        q, k, v = (t.detach().requires_grad_(True) for t in _split(qkv, B, L, H, Hkv, d))
        o = _sdpa_banded(q, k, v, 0, window)
        dq, dk, dv = torch.autograd.grad(o, (q, k, v), dout.reshape(B, L, H, d).to(o.dtype))
    return torch.cat([dq.reshape(B * L, H * d), dk.reshape(B * L, Hkv * d), dv.reshape(B * L, Hkv * d)], dim=1)


def attention_fwd(qkv: torch.Tensor, B: int, L: int, H: int, Hkv: int, d: int, window: int | None = None):
    """Returns (out [T, H*d], lse [H, T] fp32). ``window``: the layer's sliding window, or None."""
    if window is not None and L <= window:
        window = None
    if window is not None or _library_path(qkv, d):
        return windowed_fwd(qkv, B, L, H, Hkv, d, window)
    if not qkv.is_cuda:
        return attention_reference_fwd(qkv, B, L, H, Hkv, d)
    from . import flash
    return flash.flash_attn_fwd(qkv, B, L, H, Hkv, d)


def attention_bwd(dout, qkv, out, lse, B, L, H, Hkv, d, window: int | None = None):
    """Returns dqkv with the layout of qkv."""
    if window is not None and L <= window:
        window = None
    if window is not None or _library_path(qkv, d):
        return windowed_bwd(dout, qkv, B, L, H, Hkv, d, window)
    if not qkv.is_cuda:
        return attention_reference_bwd(dout, qkv, out, lse, B, L, H, Hkv, d)
    from . import flash
    return flash.flash_attn_bwd(dout, qkv, out, lse, B, L, H, Hkv, d)


def attention_bwd_unrotated(dout, qkv, out, lse, B, L, H, Hkv, d, pos, cos, sin, window: int | None = None):
    """dqkv with respect to the projection's output BEFORE the rotary embedding: attention backward followed by the
    inverse rotation of the query and key heads. On the GPU the query heads are rotated where their fp32 accumulator is
    converted to bf16 (one pass less over 8/9 of the rotated columns); same values as ``attention_bwd`` + ``rope_``."""
    from . import basic
    if window is not None and L <= window:
        window = None
    if window is not None or _library_path(qkv, d):
        return basic.rope_(windowed_bwd(dout, qkv, B, L, H, Hkv, d, window), pos, cos, sin, H + Hkv, d, inverse=True)
    if (qkv.is_cuda and qkv.dtype == torch.bfloat16 and pos.dtype == torch.int32 and cos.is_contiguous()
            and sin.is_contiguous() and 2 * cos.shape[1] == d):      # partial rotary: the separate kernel below
        from . import flash
        dqkv = flash.flash_attn_bwd(dout, qkv, out, lse, B, L, H, Hkv, d, rope=(pos, cos, sin))
        basic.rope_(dqkv[:, H * d:], pos, cos, sin, Hkv, d, inverse=True)      # the key heads
        return dqkv
    dqkv = attention_bwd(dout, qkv, out, lse, B, L, H, Hkv, d)
    return basic.rope_(dqkv, pos, cos, sin, H + Hkv, d, inverse=True)


def attention_cached_reference_fwd(qkv, k_cache, v_cache, B, L, q_off, H, Hkv, d):
    """Chunked prefill restated: the chunk's L queries (positions q_off .. q_off+L-1) against the cached keys /
    values of positions < q_off + L. k_cache, v_cache [B, rows, Hkv*d]. Returns out [B*L, H*d]."""
    q = qkv[:, : H * d].float().reshape(B, L, H, d)
    n = q_off + L
    g = H // Hkv
    k = k_cache[:, :n].float().reshape(B, n, Hkv, d).repeat_interleave(g, dim=2)
    v = v_cache[:, :n].float().reshape(B, n, Hkv, d).repeat_interleave(g, dim=2)
    s = torch.einsum("blhd,bmhd->bhlm", q, k) / math.sqrt(d)
    qpos = torch.arange(q_off, n, device=qkv.device)[:, None]
    s = s.masked_fill(torch.arange(n, device=qkv.device)[None, :] > qpos, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhlm,bmhd->blhd", p, v).reshape(B * L, H * d).to(qkv.dtype)


def attention_fwd_cached(qkv: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, B: int, L: int, q_off: int,
                         H: int, Hkv: int, d: int, window: int | None = None) -> torch.Tensor:
    """Attention of one prefill chunk against the key / value caches (which already contain the chunk's own keys and
    values at rows q_off .. q_off+L-1). Inference only: no log-sum-exp is kept."""
    if window is not None and q_off + L <= window:
        window = None
    if window is not None or _library_path(qkv, d):
        n = q_off + L
        q = qkv[:, : H * d].reshape(B, L, H, d)
        k = k_cache[:, :n].reshape(B, n, Hkv, d)
        v = v_cache[:, :n].reshape(B, n, Hkv, d)
        return _sdpa_banded(q, k, v, q_off, window).reshape(B * L, H * d).contiguous()
    if not qkv.is_cuda:
        return attention_cached_reference_fwd(qkv, k_cache, v_cache, B, L, q_off, H, Hkv, d)
    from . import flash
    return flash.flash_attn_fwd_cached(qkv, k_cache, v_cache, B, L, q_off, H, Hkv, d)
