"""Low-level ops: each function runs the sm_100a kernel when its tensors are on a CUDA device and the
plain-PyTorch restatement (the test oracle, also the CPU plumbing path) otherwise. There is no silent
fallback on a GPU: if the native library cannot be loaded the call raises.

Shapes use T = tokens (batch*seq flattened), h = hidden, f = FFN width.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p

import torch
import torch.nn.functional as F

from . import _lib

_BF16 = torch.bfloat16


def _native(*ts: torch.Tensor) -> bool:
    return any(t is not None and t.is_cuda for t in ts)


def _fmt(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return 1
    if dtype == torch.float16:
        return 0
    raise TypeError(f"tensor-core GEMM operands must be bf16 or fp16, got {dtype}")


# ------------------------------------------------------------------------------------------------ GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: torch.Tensor | None = None,
         out_dtype: torch.dtype | None = None, accumulate: bool = False, alpha: float = 1.0,
         residual: torch.Tensor | None = None, desc_cfg: list[int] | None = None) -> torch.Tensor:
    """C[M,N] = alpha * A @ B^T (+ C) (+ residual).

    ``a`` is [M,K] (``a_mn=False``) or stored transposed as [K,M] (``a_mn=True``); ``b`` is [N,K] or stored as [K,N].
    Rows must be contiguous (stride(1) == 1); row strides must be multiples of 8 elements.
    """
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"gemm: reduction dims differ ({K} vs {Kb})")
    out_dtype = out_dtype or (out.dtype if out is not None else a.dtype)
    if out is None:
        if accumulate:
            raise ValueError("gemm: accumulate=True needs out")
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if not _native(a, b):
        A = (a.t() if a_mn else a).float()
        B = (b if b_mn else b.t()).float()
        r = alpha * (A @ B)
        if residual is not None:
            r = r + residual.float()
        if accumulate:
            r = r + out.float()
        out.copy_(r.to(out.dtype))
        return out
    if a.stride(-1) != 1 or b.stride(-1) != 1 or out.stride(-1) != 1:
        raise ValueError("gemm: innermost stride must be 1")
    if a.dtype != b.dtype:
        raise TypeError("gemm: operand dtypes differ")
    fmt = _fmt(a.dtype)
    out_f32 = 1 if out.dtype == torch.float32 else 0
    if not out_f32 and out.dtype != a.dtype:
        raise TypeError("gemm: 16-bit output must match the operand dtype")
    if residual is not None and (residual.dtype != _BF16 or residual.stride(-1) != 1):
        raise TypeError("gemm: residual must be bf16 with contiguous rows")
    cfg = None
    if desc_cfg is not None:
        cfg = (ctypes.c_uint * 6)(*desc_cfg)
    rc = _lib.kernels().b200_gemm(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), M, N, K, a.stride(0), b.stride(0), out.stride(0), int(a_mn), int(b_mn),
        fmt, out_f32, int(accumulate), float(alpha), _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
        ctypes.cast(cfg, c_void_p) if cfg is not None else c_void_p(0), _lib.stream())
    _lib.check(rc, "b200_gemm")
    return out


def linear_fwd(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
    """y[T,N] = x[T,K] @ w[N,K]^T (+ residual)."""
    return gemm(x, w, residual=residual)


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """dx[T,K] = dy[T,N] @ w[N,K]  (w is read as an MN-major B operand: no transpose copy)."""
    return gemm(dy, w, b_mn=True)


def linear_wgrad(dy: torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False,
                 out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """dW[N,K] (+)= dy[T,N]^T @ x[T,K]  (both operands MN-major)."""
    return gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=accumulate, out_dtype=out_dtype)


# ------------------------------------------------------------------------------------------------ RMSNorm
def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, residual: torch.Tensor | None = None,
                out: torch.Tensor | None = None):
    """Returns (y, h, rstd): h = x + residual (or x itself), y = h * rsqrt(mean(h^2) + eps) * w.
    ``out`` (contiguous, same shape and dtype as x) receives y when given."""
    rows, hdim = x.shape
    if not _native(x):
        h = x if residual is None else (x.float() + residual.float()).to(x.dtype)
        hf = h.float()
        rstd = torch.rsqrt(hf.pow(2).mean(-1) + eps)
        y = (hf * rstd[:, None] * w.float()).to(x.dtype)
        if out is not None:
            out.copy_(y)
            y = out
        return y, h, rstd
    if out is not None and (out.shape != x.shape or out.dtype != x.dtype or not out.is_contiguous()):
        raise ValueError("rmsnorm_fwd: out must be contiguous with x's shape and dtype")
    y = out if out is not None else torch.empty_like(x)
    h = torch.empty_like(x) if residual is not None else x
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    rc = _lib.kernels().b200_rmsnorm_fwd(_lib.ptr(x), _lib.ptr(residual), _lib.ptr(w), _lib.ptr(y),
                                         _lib.ptr(h if residual is not None else None), _lib.ptr(rstd), rows, hdim,
                                         float(eps), _lib.stream())
    _lib.check(rc, "b200_rmsnorm_fwd")
    return y, h, rstd


def rmsnorm_bwd(dy: torch.Tensor, h: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor,
                dres: torch.Tensor | None = None, dw_out: torch.Tensor | None = None, dw_accumulate: bool = False):
    """Returns (dh, dw). dh includes ``dres`` (gradient arriving through the residual branch) when given.
    ``dw_out`` (fp32 [h]) is written or accumulated in place when supplied."""
    rows, hdim = h.shape
    if not _native(h):
        xh = h.float() * rstd[:, None]
        g = dy.float() * w.float()
        c = (g * xh).mean(-1, keepdim=True)
        dh = rstd[:, None] * (g - xh * c)
        if dres is not None:
            dh = dh + dres.float()
        dw = (dy.float() * xh).sum(0)
        if dw_out is not None:
            dw_out.copy_(dw_out + dw if dw_accumulate else dw)
            dw = dw_out
        return dh.to(h.dtype), dw
    dh = torch.empty_like(h)
    nblk = _lib.kernels().b200_rmsnorm_bwd_blocks(rows)
    partial = torch.empty((nblk, hdim), dtype=torch.float32, device=h.device)
    if dw_out is None:
        dw_out = torch.empty(hdim, dtype=torch.float32, device=h.device)
        dw_accumulate = False
    rc = _lib.kernels().b200_rmsnorm_bwd(_lib.ptr(dy), _lib.ptr(h), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dres),
                                         _lib.ptr(dh), _lib.ptr(partial), _lib.ptr(dw_out), int(dw_accumulate), rows,
                                         hdim, _lib.stream())
    _lib.check(rc, "b200_rmsnorm_bwd")
    return dh, dw_out


def linear_rope_fwd(x: torch.Tensor, w: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                    n_heads: int, head_dim: int) -> torch.Tensor:
    """qkv[T, N] = x w^T with the rotary embedding applied to the first ``n_heads`` heads of every row. On the GPU one
    launch when the shape allows (bf16, head_dim 64 or 128, N a multiple of 128, a few hundred rows): the rotation sits
    in the GEMM's epilogue. Same values as ``linear_fwd`` followed by ``rope_``."""
    T, N = x.shape[0], w.shape[0]
    if (_native(x, w) and x.dtype == _BF16 and w.dtype == _BF16 and head_dim in (64, 128) and N % 128 == 0 and T >= 512
            and x.stride(-1) == 1 and w.stride(-1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and pos.dtype == torch.int32 and cos.dtype == torch.float32 and cos.shape[1] == head_dim // 2
            and cos.is_contiguous() and sin.is_contiguous()):
        out = torch.empty((T, N), dtype=x.dtype, device=x.device)
        _lib.check(_lib.kernels().b200_gemm_rope(_lib.ptr(x), _lib.ptr(w), _lib.ptr(out), _lib.ptr(pos), _lib.ptr(cos),
                                                 _lib.ptr(sin), T, N, x.shape[1], n_heads, head_dim, x.stride(0),
                                                 w.stride(0), out.stride(0), _lib.stream()), "b200_gemm_rope")
        return out
    return rope_(linear_fwd(x, w), pos, cos, sin, n_heads, head_dim)


# ------------------------------------------------------------------------------------------------ per-head q/k norm
def headnorm_fwd(qkv: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor, n_q: int, n_kv: int, head_dim: int, eps: float):
    """Per-head RMSNorm of the query and key heads of fused qkv rows [T, (n_q + 2 n_kv) d] (Qwen3's q_norm / k_norm,
    applied before the rotary embedding); value heads are copied. Returns (normalised copy, rstd [T, n_q + n_kv])."""
    T = qkv.shape[0]
    nn = n_q + n_kv
    if not _native(qkv) or head_dim not in (64, 128):        # the kernels take heads of 64 and 128; others: PyTorch ops
        x = qkv.float().view(T, n_q + 2 * n_kv, head_dim)
        rstd = torch.rsqrt(x[:, :nn].pow(2).mean(-1) + eps)
        w = torch.cat([wq.float().expand(n_q, -1), wk.float().expand(n_kv, -1)])          # [nn, d]
        y = x.clone()
        y[:, :nn] = x[:, :nn] * rstd[..., None] * w
        return y.view(T, -1).to(qkv.dtype), rstd
    out = torch.empty_like(qkv)
    rstd = torch.empty((T, nn), dtype=torch.float32, device=qkv.device)
    _lib.check(_lib.kernels().b200_headnorm_fwd(_lib.ptr(qkv), _lib.ptr(out), _lib.ptr(wq), _lib.ptr(wk), _lib.ptr(rstd),
                                                T, n_q, n_kv, head_dim, qkv.stride(0), float(eps), _lib.stream()),
               "b200_headnorm_fwd")
    return out, rstd


def headnorm_bwd_(g: torch.Tensor, qkv_raw: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor, rstd: torch.Tensor,
                  n_q: int, n_kv: int, head_dim: int):
    """Backward of ``headnorm_fwd`` in place on ``g`` (gradient of the normalised rows; value heads untouched).
    Returns (dwq, dwk) fp32 [d] each."""
    T = g.shape[0]
    nn = n_q + n_kv
    if not _native(g) or head_dim not in (64, 128):
        gv = g.float().view(T, n_q + 2 * n_kv, head_dim)
        x = qkv_raw.float().view(T, n_q + 2 * n_kv, head_dim)[:, :nn]
        w = torch.cat([wq.float().expand(n_q, -1), wk.float().expand(n_kv, -1)])
        xh = x * rstd[..., None]
        gy = gv[:, :nn]
        gw = gy * w
        c = (gw * xh).mean(-1, keepdim=True)
        dx = rstd[..., None] * (gw - xh * c)
        dw = (gy * xh).sum(0)                                                             # [nn, d]
        out = gv.clone()
        out[:, :nn] = dx
        g.copy_(out.view(T, -1).to(g.dtype))
        return dw[:n_q].sum(0), dw[n_q:].sum(0)
    nblk = _lib.kernels().b200_headnorm_bwd_blocks(T, n_q, n_kv)
    partial = torch.empty((nblk, 2 * head_dim), dtype=torch.float32, device=g.device)
    dw = torch.empty(2 * head_dim, dtype=torch.float32, device=g.device)
    _lib.check(_lib.kernels().b200_headnorm_bwd(_lib.ptr(g), _lib.ptr(qkv_raw), _lib.ptr(wq), _lib.ptr(wk), _lib.ptr(rstd),
                                                _lib.ptr(partial), _lib.ptr(dw), 0, T, n_q, n_kv, head_dim, g.stride(0),
                                                _lib.stream()), "b200_headnorm_bwd")
    return dw[:head_dim], dw[head_dim:]


# ------------------------------------------------------------------------------------------------ RoPE
def rope_tables(max_pos: int, head_dim: int, theta: float, device, scaling: dict | None = None,
                model_max_pos: int | None = None, seq_len: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin tables [max_pos, head_dim/2] (HF Llama convention: pairs (i, i + d/2)).

    ``scaling`` is a HuggingFace ``rope_scaling`` dict: ``llama3`` (Llama 3.1 / 3.2: low frequencies divided by
    ``factor``, a smooth blend between ``original_max_position_embeddings / low_freq_factor`` and ``/ high_freq_factor``
    wavelengths), ``linear`` (every frequency divided by ``factor``) and ``yarn`` (frequencies that turn fewer than
    ``beta_slow`` times over the original context are interpolated by ``factor``, those that turn more than
    ``beta_fast`` times are kept, a linear ramp between; cos and sin carry the attention factor 0.1 ln(factor) + 1, or
    the ``mscale`` / ``mscale_all_dim`` ratio, or an explicit ``attention_factor``) are built; other types are refused.
    ``longrope`` (Phi-3 long-context checkpoints) divides every frequency by its entry of ``short_factor``, or of
    ``long_factor`` when the sequence (``seq_len``) is longer than the original context, and scales cos / sin by
    sqrt(1 + ln(factor) / ln(original context)).
    ``dynamic`` (NTK-aware): beyond the model's context the base grows with the sequence length,
    theta * (factor * seq_len / context - (factor - 1)) ^ (d / (d - 2)), inside it nothing changes; with an ``alpha`` key
    (HunYuan) the base is theta * alpha ^ (d / (d - 2)) at every length.
    ``model_max_pos`` is the model's ``max_position_embeddings`` (yarn's original context when the dict names none)."""
    import math
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    kind = (scaling or {}).get("rope_type", (scaling or {}).get("type")) if scaling else None
    amp = 1.0
    if kind in (None, "default"):
        pass
    elif kind == "yarn":
        orig = scaling.get("original_max_position_embeddings") or model_max_pos
        if not orig:
            raise ValueError("yarn rope scaling needs original_max_position_embeddings")
        factor = scaling.get("factor")
        factor = float(factor) if factor is not None else float(model_max_pos) / float(orig)

        def mscale_of(scale, m=1.0):
            return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0
        amp = scaling.get("attention_factor")
        if amp is None:
            ms, ms_all = scaling.get("mscale"), scaling.get("mscale_all_dim")
            amp = mscale_of(factor, ms) / mscale_of(factor, ms_all) if (ms and ms_all) else mscale_of(factor)
        amp = float(amp)
        fast, slow = float(scaling.get("beta_fast") or 32), float(scaling.get("beta_slow") or 1)

        def dim_of(rotations):      # the pair index whose frequency turns `rotations` times over the original context
            return head_dim * math.log(orig / (rotations * 2 * math.pi)) / (2 * math.log(theta))
        lo_d, hi_d = dim_of(fast), dim_of(slow)
        if scaling.get("truncate", True):
            lo_d, hi_d = math.floor(lo_d), math.ceil(hi_d)
        lo_d, hi_d = max(lo_d, 0), min(hi_d, head_dim - 1)
        if lo_d == hi_d:
            hi_d += 0.001
        ramp = ((torch.arange(head_dim // 2, dtype=torch.float32, device=device) - lo_d) / (hi_d - lo_d)).clamp(0, 1)
        inv = (inv / factor) * ramp + inv * (1.0 - ramp)
    elif kind == "longrope":
        orig = scaling.get("original_max_position_embeddings") or model_max_pos
        if not orig or "short_factor" not in scaling or "long_factor" not in scaling:
            raise ValueError("longrope scaling needs short_factor, long_factor and original_max_position_embeddings")
        factor = scaling.get("factor")
        factor = float(factor) if factor is not None else float(model_max_pos or orig) / float(orig)
        amp = scaling.get("attention_factor")
        if amp is None:
            amp = 1.0 if factor <= 1.0 else math.sqrt(1.0 + math.log(factor) / math.log(orig))
        amp = float(amp)
        use_long = (seq_len if seq_len is not None else max_pos) > orig
        ext = torch.tensor(scaling["long_factor" if use_long else "short_factor"], dtype=torch.float32, device=device)
        if ext.numel() != inv.numel():
            raise ValueError(f"longrope factors have {ext.numel()} entries, the head has {inv.numel()} frequency pairs")
        inv = inv / ext
    elif kind == "linear":
        inv = inv / float(scaling["factor"])
    elif kind == "dynamic":
        if scaling.get("alpha"):
            base = theta * float(scaling["alpha"]) ** (head_dim / (head_dim - 2))
        else:
            orig = model_max_pos or scaling.get("original_max_position_embeddings")
            if not orig:
                raise ValueError("dynamic rope scaling needs the model's max_position_embeddings")
            factor = float(scaling["factor"])
            length = max(int(seq_len if seq_len is not None else max_pos), int(orig))
            base = theta * (factor * length / float(orig) - (factor - 1.0)) ** (head_dim / (head_dim - 2))
        inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    elif kind == "llama3":
        factor = float(scaling["factor"])
        lo_f, hi_f = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2.0 * math.pi / inv
        smooth = ((old / wavelen - lo_f) / (hi_f - lo_f)).clamp(0.0, 1.0)
        blended = (1.0 - smooth) * inv / factor + smooth * inv
        inv = torch.where(wavelen > old / lo_f, inv / factor, torch.where(wavelen < old / hi_f, inv, blended))
    else:
        raise NotImplementedError(f"rope_scaling type {kind!r} is not built (default, linear, dynamic, llama3, yarn and "
                                  "longrope are)")
    ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    return (ang.cos() * amp).contiguous(), (ang.sin() * amp).contiguous()


def rope_(x: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_heads: int, head_dim: int,
          inverse: bool = False) -> torch.Tensor:
    """Rotate x[T, >= n_heads*head_dim] in place (only the first n_heads*head_dim columns of each row).
    ``pos`` is int32 [T]. ``inverse=True`` applies the transposed rotation (the backward pass). The tables' width sets
    how much of a head rotates: [max_pos, rot/2] with rot <= head_dim (partial rotary embeddings, e.g. Phi-4-mini's
    0.75); the other head_dim - rot elements of each head stay as they are."""
    T = x.shape[0]
    rot = 2 * cos.shape[1]
    if rot > head_dim:
        raise ValueError(f"rope_: tables of width {cos.shape[1]} for heads of {head_dim}")
    if not _native(x):
        half = rot // 2
        v = x[:, : n_heads * head_dim].reshape(T, n_heads, head_dim).float()
        c = cos[pos.long()][:, None, :]
        s = sin[pos.long()][:, None, :] * (-1.0 if inverse else 1.0)
        a, b = v[..., :half], v[..., half:rot]
        out = torch.cat([a * c - b * s, b * c + a * s, v[..., rot:]], dim=-1)
        x[:, : n_heads * head_dim] = out.reshape(T, n_heads * head_dim).to(x.dtype)
        return x
    if x.stride(-1) != 1 or pos.dtype != torch.int32:
        raise ValueError("rope_: x rows must be contiguous and pos int32")
    if rot % 16:
        raise ValueError(f"rope_: the kernel rotates 16-byte vectors - rotary width {rot} is not a multiple of 16")
    rc = _lib.kernels().b200_rope_partial(_lib.ptr(x), _lib.ptr(pos), _lib.ptr(cos), _lib.ptr(sin), T, n_heads,
                                          head_dim, rot, x.stride(0), int(inverse), _lib.stream())
    _lib.check(rc, "b200_rope_partial")
    return x


# ------------------------------------------------------------------------------------------------ bias
_lib.register("b200_bias_add", [_lib._VP, _lib._VP, _lib._LL, _lib._I, _lib._LL, _lib._VP])
_lib.register("b200_bias_grad", [_lib._VP, _lib._VP, _lib._LL, _lib._I, _lib._LL, _lib._I, _lib._VP])


def bias_add_(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x[T, N] += bias[N] in place (the q/k/v projection bias of Qwen2-style attention)."""
    if not _native(x):
        x.add_(bias.to(x.dtype))
        return x
    T, N = x.shape
    _lib.check(_lib.kernels().b200_bias_add(_lib.ptr(x), _lib.ptr(bias), T, N, x.stride(0), _lib.stream()),
               "b200_bias_add")
    return x


def bias_grad(dy: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """fp32 column sums of dy[T, N]; with ``out`` they are written (or added) there."""
    T, N = dy.shape
    if out is None:
        out = torch.zeros(N, dtype=torch.float32, device=dy.device)
        accumulate = True
    if not _native(dy):
        g = dy.float().sum(0)
        out.copy_(out + g if accumulate else g)
        return out
    _lib.check(_lib.kernels().b200_bias_grad(_lib.ptr(dy), _lib.ptr(out), T, N, dy.stride(0), int(accumulate),
                                             _lib.stream()), "b200_bias_grad")
    return out


# ------------------------------------------------------------------------------------------------ SwiGLU
def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    """act[T,f] = silu(gu[:, :f]) * gu[:, f:]"""
    T, f2 = gu.shape
    f = f2 // 2
    if not _native(gu):
        g, u = gu[:, :f].float(), gu[:, f:].float()
        return (F.silu(g) * u).to(gu.dtype)
    act = torch.empty((T, f), dtype=gu.dtype, device=gu.device)
    _lib.check(_lib.kernels().b200_swiglu_fwd(_lib.ptr(gu), _lib.ptr(act), T, f, _lib.stream()), "b200_swiglu_fwd")
    return act


def swiglu_fusable(x: torch.Tensor, w_gu: torch.Tensor) -> bool:
    """Whether ``linear_swiglu_fwd`` runs as one launch for these operands."""
    f = w_gu.shape[0] // 2
    return bool(_native(x, w_gu) and x.dtype == _BF16 and w_gu.dtype == _BF16 and f % 128 == 0 and x.shape[0] >= 512
                and x.stride(-1) == 1 and w_gu.stride(-1) == 1 and x.stride(0) % 8 == 0 and w_gu.stride(0) % 8 == 0)


def linear_swiglu_fwd(x: torch.Tensor, w_gu: torch.Tensor, out_gu: torch.Tensor | None = None,
                      out_act: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """(gu, act) with gu[T, 2f] = x w_gu^T (gate rows first, then up rows) and act[T, f] = silu(gate) * up. On the GPU
    one launch does both when the shape allows (bf16, f a multiple of 128, at least a few hundred rows): the SwiGLU
    sits in the epilogue of the gate / up GEMM. Same values as ``linear_fwd`` followed by ``swiglu_fwd``.
    ``out_gu`` / ``out_act`` (row slices of larger buffers are fine) receive the results when given."""
    T = x.shape[0]
    f = w_gu.shape[0] // 2
    if swiglu_fusable(x, w_gu):
        gu = out_gu if out_gu is not None else torch.empty((T, 2 * f), dtype=x.dtype, device=x.device)
        act = out_act if out_act is not None else torch.empty((T, f), dtype=x.dtype, device=x.device)
        _lib.check(_lib.kernels().b200_gemm_swiglu(_lib.ptr(x), _lib.ptr(w_gu), _lib.ptr(gu), _lib.ptr(act), T, f,
                                                   x.shape[1], x.stride(0), w_gu.stride(0), gu.stride(0), act.stride(0),
                                                   _lib.stream()), "b200_gemm_swiglu")
        return gu, act
    gu = gemm(x, w_gu, out=out_gu) if out_gu is not None else linear_fwd(x, w_gu)
    act = swiglu_fwd(gu)
    if out_act is not None:
        out_act.copy_(act)
        act = out_act
    return gu, act


def swiglu_bwd_fusable(dy: torch.Tensor, w_d: torch.Tensor, gu: torch.Tensor) -> bool:
    """Whether ``linear_dgrad_swiglu_bwd`` runs as one launch for these operands."""
    f = w_d.shape[1]
    return bool(_native(dy, w_d, gu) and dy.dtype == _BF16 and w_d.dtype == _BF16 and gu.dtype == _BF16 and f % 128 == 0
                and dy.shape[0] >= 512 and dy.stride(-1) == 1 and w_d.stride(-1) == 1 and gu.stride(-1) == 1
                and dy.stride(0) % 8 == 0 and w_d.stride(0) % 8 == 0 and gu.stride(0) % 8 == 0)


def linear_dgrad_swiglu_bwd(dy: torch.Tensor, w_d: torch.Tensor, gu: torch.Tensor,
                            out: torch.Tensor | None = None) -> torch.Tensor:
    """dgu[T, 2f] = SwiGLU backward of (gu, dact) with dact = dy[T, h] w_d[h, f] - the gradient through the down
    projection and the activation. On the GPU one launch when the shape allows: the dgrad GEMM's epilogue reads gate /
    up, rounds its accumulator to bf16 and writes d(gate), d(up); dact is never stored. Same values as
    ``linear_dgrad`` followed by ``swiglu_bwd``. ``out`` (a row slice of a larger buffer is fine) receives the result."""
    T = dy.shape[0]
    f = w_d.shape[1]
    if swiglu_bwd_fusable(dy, w_d, gu):
        dgu = out if out is not None else torch.empty((T, 2 * f), dtype=gu.dtype, device=gu.device)
        _lib.check(_lib.kernels().b200_gemm_swiglu_bwd(_lib.ptr(dy), _lib.ptr(w_d), _lib.ptr(gu), _lib.ptr(dgu), T, f,
                                                       dy.shape[1], dy.stride(0), w_d.stride(0), gu.stride(0),
                                                       dgu.stride(0), _lib.stream()), "b200_gemm_swiglu_bwd")
        return dgu
    dgu = swiglu_bwd(gu, linear_dgrad(dy, w_d))
    if out is not None:
        out.copy_(dgu)
        return out
    return dgu


def swiglu_bwd(gu: torch.Tensor, dact: torch.Tensor) -> torch.Tensor:
    T, f2 = gu.shape
    f = f2 // 2
    if not _native(gu):
        g, u, d = gu[:, :f].float(), gu[:, f:].float(), dact.float()
        sg = torch.sigmoid(g)
        silu = g * sg
        return torch.cat([d * u * (sg + silu * (1 - sg)), d * silu], dim=1).to(gu.dtype)
    dgu = torch.empty_like(gu)
    _lib.check(_lib.kernels().b200_swiglu_bwd(_lib.ptr(gu), _lib.ptr(dact), _lib.ptr(dgu), T, f, _lib.stream()),
               "b200_swiglu_bwd")
    return dgu


# ------------------------------------------------------------------------------------------------ GeGLU (Gemma)
def glu_fwd(gu: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """act(gate) * up of fused rows [T, 2f]. ``silu``: the SwiGLU kernel; ``gelu_tanh`` (Gemma's GeGLU): PyTorch's
    elementwise ops on either device - no kernel of this library covers it."""
    if act == "silu":
        return swiglu_fwd(gu)
    if act != "gelu_tanh":
        raise NotImplementedError(f"gated activation {act!r} is not built (silu and gelu_tanh are)")
    f = gu.shape[1] // 2
    return (F.gelu(gu[:, :f].float(), approximate="tanh") * gu[:, f:].float()).to(gu.dtype)


def glu_bwd(gu: torch.Tensor, dact: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """Gradient of ``glu_fwd`` with respect to the fused rows."""
    if act == "silu":
        return swiglu_bwd(gu, dact)
    if act != "gelu_tanh":
        raise NotImplementedError(f"gated activation {act!r} is not built (silu and gelu_tanh are)")
    f = gu.shape[1] // 2
    up, d = gu[:, f:].float(), dact.float()
    with torch.enable_grad():
        g = gu[:, :f].detach().float().requires_grad_(True)
        y = F.gelu(g, approximate="tanh")
        (dg,) = torch.autograd.grad(y, g, d * up)
    return torch.cat([dg, d * y.detach()], dim=1).to(gu.dtype)


def linear_glu_fwd(x: torch.Tensor, w_gu: torch.Tensor, act: str = "silu"):
    """(gu, act(gate) * up) of x w_gu^T: ``linear_swiglu_fwd`` for silu, projection + ``glu_fwd`` otherwise."""
    if act == "silu":
        return linear_swiglu_fwd(x, w_gu)
    gu = linear_fwd(x, w_gu)
    return gu, glu_fwd(gu, act)


def linear_dgrad_glu_bwd(dy: torch.Tensor, w_d: torch.Tensor, gu: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """dgu through the down projection and the gated activation: ``linear_dgrad_swiglu_bwd`` for silu."""
    if act == "silu":
        return linear_dgrad_swiglu_bwd(dy, w_d, gu)
    return glu_bwd(gu, linear_dgrad(dy, w_d), act)


# ------------------------------------------------------------------------------------------------ embedding
def embed_fwd(ids: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """out[T,h] = w[ids]; ids int64 [T]."""
    if not _native(w):
        return w[ids.clamp(0, w.shape[0] - 1)]
    T = ids.numel()
    out = torch.empty((T, w.shape[1]), dtype=w.dtype, device=w.device)
    _lib.check(_lib.kernels().b200_embed_fwd(_lib.ptr(ids), _lib.ptr(w), _lib.ptr(out), T, w.shape[1], w.shape[0],
                                             _lib.stream()), "b200_embed_fwd")
    return out


def embed_bwd(ids: torch.Tensor, dout: torch.Tensor, dw: torch.Tensor) -> torch.Tensor:
    """dw[ids[t]] += dout[t]   (dw fp32 [V,h], accumulated in place)."""
    if not _native(dw):
        dw.index_add_(0, ids, dout.float())
        return dw
    T = ids.numel()
    _lib.check(_lib.kernels().b200_embed_bwd(_lib.ptr(ids), _lib.ptr(dout), _lib.ptr(dw), T, dw.shape[1], dw.shape[0],
                                             _lib.stream()), "b200_embed_bwd")
    return dw


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """out[i] = x[rows[i]] (rows int64)."""
    return embed_fwd(rows, x)


def scatter_rows(src: torch.Tensor, rows: torch.Tensor, n_rows: int) -> torch.Tensor:
    """out [n_rows, h] zero except out[rows[i]] = src[i] (rows unique): the backward of ``gather_rows``."""
    if not _native(src):
        out = torch.zeros((n_rows, src.shape[1]), dtype=src.dtype, device=src.device)
        out[rows] = src
        return out
    out = torch.empty((n_rows, src.shape[1]), dtype=src.dtype, device=src.device)
    _lib.check(_lib.kernels().b200_scatter_rows(_lib.ptr(rows), _lib.ptr(src), _lib.ptr(out), rows.numel(), src.shape[1],
                                                n_rows, _lib.stream()), "b200_scatter_rows")
    return out


class GatherRowsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, rows):
        ctx.save_for_backward(rows)
        ctx.n = x.shape[0]
        return gather_rows(x, rows)

    @staticmethod
    def backward(ctx, dout):
        (rows,) = ctx.saved_tensors
        return scatter_rows(dout.contiguous(), rows, ctx.n), None


# ------------------------------------------------------------------------------------------------ casts
def cast_to_bf16(src_f32: torch.Tensor, dst_bf16: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    if not _native(src_f32):
        dst_bf16.copy_((src_f32 * scale).to(dst_bf16.dtype))
        return dst_bf16
    _lib.check(_lib.kernels().b200_cast_f32_to_bf16(_lib.ptr(src_f32), _lib.ptr(dst_bf16), src_f32.numel(), float(scale),
                                                    _lib.stream()), "b200_cast_f32_to_bf16")
    return dst_bf16


def cast_to_f32(src_bf16: torch.Tensor, dst_f32: torch.Tensor, scale: float = 1.0, accumulate: bool = False):
    if not _native(src_bf16):
        v = src_bf16.float() * scale
        dst_f32.copy_(dst_f32 + v if accumulate else v)
        return dst_f32
    _lib.check(_lib.kernels().b200_cast_bf16_to_f32(_lib.ptr(src_bf16), _lib.ptr(dst_f32), src_bf16.numel(), float(scale),
                                                    int(accumulate), _lib.stream()), "b200_cast_bf16_to_f32")
    return dst_f32
