"""Decoder layers whose branches are normalised on the way OUT as well as (or instead of) on the way in:

    h1 = h  + [OutNorm_a]( Attn( [InNorm_1](h)  ) )
    h2 = h1 + [OutNorm_m]( MLP(  [InNorm_2](h1) ) )

OLMo 2 has only the output norms and normalises the whole query / key projections (one RMSNorm over all heads) before
the rotation; GLM-4 (0414) has all four norms; HunYuan is a plain pre-norm layer whose per-head q/k norms come AFTER
the rotation (the norm's weight does not commute with it), which the fused layer of ``llama.py`` does not do; Gemma's
gate activation is GELU. The
reference trains such students through ``AutoModelForCausalLM`` (classes/student/model.py:194-201). One autograd node with an explicit backward, built from the same kernels as
``llama.DecoderLayerFn`` (tcgen05 GEMMs with the SwiGLU epilogues, RMSNorm, RoPE, flash attention); the residual adds
that the plain layer folds into GEMM epilogues are separate here because a norm sits between the GEMM and the add.
"""
from __future__ import annotations

import torch

from ..ops import attention, basic
from . import llama as _ll


def _qk_full_fwd(qkv, w_qn, w_kn, q, kv, eps):
    """RMSNorm over the whole query block and the whole key block of fused rows [T, q + 2 kv]."""
    q_raw = qkv[:, :q].contiguous()
    k_raw = qkv[:, q:q + kv].contiguous()
    qn, _, rq = basic.rmsnorm_fwd(q_raw, w_qn, eps)
    kn, _, rk = basic.rmsnorm_fwd(k_raw, w_kn, eps)
    return torch.cat([qn, kn, qkv[:, q + kv:]], dim=1), (q_raw, k_raw, rq, rk)


def _forward(h, pos, cos, sin, meta, w_qkv, w_o, w_gu, w_d, w_ln1, w_ln2, w_pa, w_pm, b_qkv, w_qn, w_kn):
    B, L, H, Hkv, d, eps, _recompute, window, qk_mode, _first, act_fn = meta
    q, kv = H * d, Hkv * d
    r1 = r2 = ra = rm = None
    x1 = h
    if w_ln1 is not None:
        x1, _, r1 = basic.rmsnorm_fwd(h, w_ln1, eps)
    qkv = basic.linear_fwd(x1, w_qkv)
    if b_qkv is not None:
        basic.bias_add_(qkv, b_qkv)
    qk_saved = ()
    if qk_mode == 2:
        qkv, qk_saved = _qk_full_fwd(qkv, w_qn, w_kn, q, kv, eps)
    elif qk_mode == 1:
        qkv_raw = qkv
        qkv, rstd_qk = basic.headnorm_fwd(qkv_raw, w_qn, w_kn, H, Hkv, d, eps)
        qk_saved = (qkv_raw, rstd_qk)
    basic.rope_(qkv, pos, cos, sin, H + Hkv, d)
    if qk_mode == 3:                       # per-head norms of the ROTATED queries and keys
        qkv_rot = qkv
        qkv, rstd_qk = basic.headnorm_fwd(qkv_rot, w_qn, w_kn, H, Hkv, d, eps)
        qk_saved = (qkv_rot, rstd_qk)
    att, lse = attention.attention_fwd(qkv, B, L, H, Hkv, d, window)
    if w_pa is None:
        a = None
        h1 = basic.linear_fwd(att, w_o, residual=h)
    else:
        a = basic.linear_fwd(att, w_o)
        an, _, ra = basic.rmsnorm_fwd(a, w_pa, eps)
        h1 = h + an
    x2 = h1
    if w_ln2 is not None:
        x2, _, r2 = basic.rmsnorm_fwd(h1, w_ln2, eps)
    gu, act = basic.linear_glu_fwd(x2, w_gu, act_fn)
    if w_pm is None:
        m = None
        h2 = basic.linear_fwd(act, w_d, residual=h1)
    else:
        m = basic.linear_fwd(act, w_d)
        mn, _, rm = basic.rmsnorm_fwd(m, w_pm, eps)
        h2 = h1 + mn
    return h2, (x1, r1, qkv, att, lse, a, ra, h1, x2, r2, gu, act, m, rm), qk_saved


class SandwichLayerFn(torch.autograd.Function):
    """meta = (B, L, heads, kv heads, head dim, eps, recompute in backward, sliding window or None, q/k norm: 0 none / 1 per head / 2 over the
    whole projection / 3 per head after the rotation, the layer's first parameter, the gate's activation). Norm weights
    that the family does not have are None."""

    @staticmethod
    def forward(ctx, h, pos, cos, sin, meta, w_qkv, w_o, w_gu, w_d, w_ln1=None, w_ln2=None, w_pa=None, w_pm=None,
                b_qkv=None, w_qn=None, w_kn=None):
        weights = (w_qkv, w_o, w_gu, w_d, w_ln1, w_ln2, w_pa, w_pm, b_qkv, w_qn, w_kn)
        h2, inter, qk_saved = _forward(h, pos, cos, sin, meta, *weights)
        ctx.meta = meta
        ctx.weights = weights
        ctx.slots = tuple(_ll._slot(w) if w is not None else None for w in weights)
        if meta[6]:
            ctx.save_for_backward(h, pos, cos, sin)
            ctx.n_inter = 0
        else:
            keep = [t for t in inter if t is not None]
            ctx.present = tuple(t is not None for t in inter)
            ctx.n_inter = len(keep)
            ctx.save_for_backward(h, pos, cos, sin, *keep, *qk_saved)
        return h2

    @staticmethod
    def backward(ctx, dh2):
        B, L, H, Hkv, d, eps, recompute, window, qk_mode, first, act_fn = ctx.meta
        w_qkv, w_o, w_gu, w_d, w_ln1, w_ln2, w_pa, w_pm, b_qkv, w_qn, w_kn = ctx.weights
        s_qkv, s_o, s_gu, s_d, s_ln1, s_ln2, s_pa, s_pm, s_b, s_qn, s_kn = ctx.slots
        q, kv = H * d, Hkv * d
        if _ll.UNIT_PRE[0] is not None:                 # the layer's backward starts here
            _ll.UNIT_PRE[0](first, True)
        if _ll.LAYER_WEIGHTS_PRE[0] is not None:
            _ll.LAYER_WEIGHTS_PRE[0](first)
        if recompute:
            h, pos, cos, sin = ctx.saved_tensors
            _, inter, qk_saved = _forward(h, pos, cos, sin, ctx.meta, *ctx.weights)
        else:
            h, pos, cos, sin, *rest = ctx.saved_tensors
            it = iter(rest[:ctx.n_inter])
            inter = tuple(next(it) if p else None for p in ctx.present)
            qk_saved = tuple(rest[ctx.n_inter:])
        x1, r1, qkv, att, lse, a, ra, h1, x2, r2, gu, act, m, rm = inter
        dh2 = dh2.contiguous()
        # MLP branch
        g_pm = None
        dm = dh2
        if w_pm is not None:
            dm, dw = basic.rmsnorm_bwd(dh2, m, w_pm, rm)
            g_pm = _ll._vec_grad(dw, w_pm, s_pm)
        g_d = _ll._wgrad(dm, act, w_d, s_d)
        dgu = basic.linear_dgrad_glu_bwd(dm, w_d, gu, act_fn)
        g_gu = _ll._wgrad(dgu, x2, w_gu, s_gu)
        dx2 = basic.linear_dgrad(dgu, w_gu)
        del dgu
        g_ln2 = None
        if w_ln2 is not None:
            dh1, dw = basic.rmsnorm_bwd(dx2, h1, w_ln2, r2, dres=dh2)
            g_ln2 = _ll._vec_grad(dw, w_ln2, s_ln2)
        else:
            dh1 = dh2 + dx2
        # attention branch
        g_pa = None
        da = dh1
        if w_pa is not None:
            da, dw = basic.rmsnorm_bwd(dh1, a, w_pa, ra)
            g_pa = _ll._vec_grad(dw, w_pa, s_pa)
        g_o = _ll._wgrad(da, att, w_o, s_o)
        datt = basic.linear_dgrad(da, w_o)
        g_qn = g_kn = None
        if qk_mode == 3:
            qkv_rot, rstd_qk = qk_saved
            dqkv = attention.attention_bwd(datt, qkv, att, lse, B, L, H, Hkv, d, window)
            dwq, dwk = basic.headnorm_bwd_(dqkv, qkv_rot, w_qn, w_kn, rstd_qk, H, Hkv, d)
            basic.rope_(dqkv, pos, cos, sin, H + Hkv, d, inverse=True)
            g_qn = _ll._vec_grad(dwq, w_qn, s_qn)
            g_kn = _ll._vec_grad(dwk, w_kn, s_kn)
        else:
            dqkv = attention.attention_bwd_unrotated(datt, qkv, att, lse, B, L, H, Hkv, d, pos, cos, sin, window)
        del datt
        if qk_mode == 2:
            q_raw, k_raw, rq, rk = qk_saved
            dq, dwq = basic.rmsnorm_bwd(dqkv[:, :q].contiguous(), q_raw, w_qn, rq)
            dk, dwk = basic.rmsnorm_bwd(dqkv[:, q:q + kv].contiguous(), k_raw, w_kn, rk)
            dqkv = torch.cat([dq, dk, dqkv[:, q + kv:]], dim=1)
            g_qn = _ll._vec_grad(dwq, w_qn, s_qn)
            g_kn = _ll._vec_grad(dwk, w_kn, s_kn)
        elif qk_mode == 1:
            qkv_raw, rstd_qk = qk_saved
            dwq, dwk = basic.headnorm_bwd_(dqkv, qkv_raw, w_qn, w_kn, rstd_qk, H, Hkv, d)
            g_qn = _ll._vec_grad(dwq, w_qn, s_qn)
            g_kn = _ll._vec_grad(dwk, w_kn, s_kn)
        g_b = _ll._bias_grad(dqkv, b_qkv, s_b)
        g_qkv = _ll._wgrad(dqkv, x1, w_qkv, s_qkv)
        dx1 = basic.linear_dgrad(dqkv, w_qkv)
        del dqkv
        g_ln1 = None
        if w_ln1 is not None:
            dh, dw = basic.rmsnorm_bwd(dx1, h, w_ln1, r1, dres=dh1)
            g_ln1 = _ll._vec_grad(dw, w_ln1, s_ln1)
        else:
            dh = dh1 + dx1
        if _ll.LAYER_BACKWARD_DONE[0] is not None:      # all of the layer's gradients are final
            _ll.LAYER_BACKWARD_DONE[0](first)
        return dh, None, None, None, None, g_qkv, g_o, g_gu, g_d, g_ln1, g_ln2, g_pa, g_pm, g_b, g_qn, g_kn


@torch.no_grad()
def layer_inference(layer, cfg, h, qkv_hook, eps):
    """Forward of one such layer for the chunked-prefill path. ``qkv_hook(qkv, after_rotation) -> att`` receives the
    projected (bias added, normalised) rows before the rotation and returns the attention output: it rotates, applies
    ``after_rotation`` (None, or a function of the rotated rows), fills the key / value cache and runs attention
    against it."""
    H, Hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    x1 = h
    if cfg.pre_norm:
        x1, _, _ = basic.rmsnorm_fwd(h, layer.input_layernorm, eps)
    qkv = basic.linear_fwd(x1, layer.qkv_proj)
    if hasattr(layer, "qkv_bias"):
        basic.bias_add_(qkv, layer.qkv_bias)
    if cfg.qk_norm_full:
        qkv, _ = _qk_full_fwd(qkv, layer.q_norm, layer.k_norm, H * d, Hkv * d, eps)
    elif cfg.qk_norm and not cfg.qk_norm_after_rope:
        qkv, _ = basic.headnorm_fwd(qkv, layer.q_norm, layer.k_norm, H, Hkv, d, eps)
    after = None
    if cfg.qk_norm_after_rope:
        after = lambda rows: basic.headnorm_fwd(rows, layer.q_norm, layer.k_norm, H, Hkv, d, eps)[0]
    att = qkv_hook(qkv, after)
    if cfg.post_norm:
        a, _, _ = basic.rmsnorm_fwd(basic.linear_fwd(att, layer.o_proj), layer.attn_out_norm, eps)
        h1 = h + a
    else:
        h1 = basic.linear_fwd(att, layer.o_proj, residual=h)
    x2 = h1
    if cfg.pre_norm:
        x2, _, _ = basic.rmsnorm_fwd(h1, layer.post_attention_layernorm, eps)
    _, act = basic.linear_glu_fwd(x2, layer.gate_up_proj, cfg.mlp_act)
    if cfg.post_norm:
        m, _, _ = basic.rmsnorm_fwd(basic.linear_fwd(act, layer.down_proj), layer.mlp_out_norm, eps)
        return h1 + m
    return basic.linear_fwd(act, layer.down_proj, residual=h1)
