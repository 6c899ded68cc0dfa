"""Sparse mixture-of-experts decoder blocks (Mixtral layout: a linear router, top-k of the softmax renormalised over
the chosen experts, SwiGLU experts; Qwen2-MoE adds a dense "shared" expert behind a sigmoid gate to every token) for
both roles, student training and teacher inference.

The reference loads such students through ``AutoModelForCausalLM`` (classes/student/model.py:194-201) and its shipped
``freeze_layers`` default names Mixtral's router (config.json: ``block_sparse_moe.gate``). Here a decoder layer with
experts is two autograd nodes with explicit backward: ``AttnBlockFn`` (the attention half of the dense layer) and
``MoEBlockFn``. The expert half sorts the (token, choice) pairs by expert once per layer, gathers the rows, runs every
expert's two GEMMs on its contiguous slab of rows with the same tcgen05 GEMM kernels as the dense layers (the fused
gate/up projection of all experts fills one buffer, so SwiGLU is one launch), and combines by GATHERING each token's k
results - a fixed order of additions, no atomic scatter. Routing arithmetic ([T, E] tensors) is PyTorch in fp32.
The number of rows per expert comes back to the host once per layer (the GEMM shapes depend on it).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops import attention, basic
from . import llama as _ll


# ------------------------------------------------------------------------------------------------ routing
def route(n2: torch.Tensor, w_router: torch.Tensor, k: int, renorm: bool = True):
    """Router of one layer: (probs [T,E] fp32, chosen experts [T,k] int64, their weights [T,k] fp32 - renormalised
    over the chosen experts (Mixtral; Qwen3-MoE with ``norm_topk_prob``) or the plain softmax values).
    Logits are computed in the model's dtype and the softmax in fp32, as HuggingFace's blocks do."""
    logits = F.linear(n2, w_router)
    probs = torch.softmax(logits.float(), dim=-1)
    top_p, top_e = torch.topk(probs, k, dim=-1)
    return probs, top_e, (top_p / top_p.sum(-1, keepdim=True) if renorm else top_p)


def permutation(top_e: torch.Tensor, n_experts: int):
    """(order, inverse, counts): ``order`` lists the T*k (token, choice) pairs sorted by expert (stable, so tokens keep
    their order inside an expert's slab), ``inverse`` undoes it, ``counts`` are the slab lengths as Python ints."""
    flat = top_e.reshape(-1)
    order = torch.argsort(flat, stable=True)
    inverse = torch.empty_like(order)
    inverse[order] = torch.arange(order.numel(), device=order.device)
    counts = torch.bincount(flat, minlength=n_experts).tolist()
    return order, inverse, counts


def experts_forward(x_perm: torch.Tensor, counts: list[int], w_gu: torch.Tensor, w_d: torch.Tensor):
    """x_perm [T*k, h] (rows grouped by expert) -> (gu [T*k, 2f], act [T*k, f], y [T*k, h])."""
    n, h = x_perm.shape
    two_f = w_gu.shape[1]
    gu = torch.empty((n, two_f), dtype=x_perm.dtype, device=x_perm.device)
    offs, o = [], 0
    for c in counts:
        offs.append(o)
        o += c
    if all(c == 0 or basic.swiglu_fusable(x_perm[o:o + c], w_gu[e]) for e, (o, c) in enumerate(zip(offs, counts))):
        # every expert has enough rows for the GEMM that applies SwiGLU in its epilogue
        act = torch.empty((n, two_f // 2), dtype=x_perm.dtype, device=x_perm.device)
        for e, (o, c) in enumerate(zip(offs, counts)):
            if c:
                basic.linear_swiglu_fwd(x_perm[o:o + c], w_gu[e], gu[o:o + c], act[o:o + c])
    else:
        for e, (o, c) in enumerate(zip(offs, counts)):
            if c:
                basic.gemm(x_perm[o:o + c], w_gu[e], out=gu[o:o + c])
        act = basic.swiglu_fwd(gu)
    y = torch.empty((n, h), dtype=x_perm.dtype, device=x_perm.device)
    o = 0
    for e, c in enumerate(counts):
        if c:
            basic.gemm(act[o:o + c], w_d[e], out=y[o:o + c])
        o += c
    return gu, act, y


def shared_expert_forward(n2: torch.Tensor, w_sgu: torch.Tensor, w_sd: torch.Tensor, w_sg: torch.Tensor):
    """Qwen2-MoE's shared expert: a dense SwiGLU MLP every token passes through, scaled per token by
    sigmoid(n2 . w_sg) (Qwen2-MoE) or added as it is (``w_sg`` None: Granite's shared MLP).
    Returns (gu_s [T, 2fs], act_s [T, fs], y_s [T, h], gate [T, 1] fp32)."""
    gu_s, act_s = basic.linear_swiglu_fwd(n2, w_sgu)
    y_s = basic.linear_fwd(act_s, w_sd)
    if w_sg is None:         # Granite's shared MLP joins ungated
        gate = torch.ones((n2.shape[0], 1), dtype=torch.float32, device=n2.device)
    else:
        gate = torch.sigmoid(F.linear(n2, w_sg).float())
    return gu_s, act_s, y_s, gate


def moe_mlp(n2: torch.Tensor, w_router: torch.Tensor, w_gu: torch.Tensor, w_d: torch.Tensor, k: int,
            renorm: bool = True, shared=None) -> torch.Tensor:
    """Inference-only expert half: sum_k weight * expert(n2) as [T, h] in n2's dtype. ``shared`` = (gate/up matrix,
    down matrix, gate vector) of a shared expert, or None."""
    T, h = n2.shape
    _, top_e, top_w = route(n2, w_router, k, renorm)
    order, inverse, counts = permutation(top_e, w_gu.shape[0])
    x_perm = n2.index_select(0, torch.div(order, k, rounding_mode="floor"))
    _, _, y = experts_forward(x_perm, counts, w_gu, w_d)
    y_tok = y.index_select(0, inverse).view(T, k, h)
    out = (y_tok.float() * top_w.unsqueeze(-1)).sum(1)
    if shared is not None:
        _, _, y_s, gate = shared_expert_forward(n2, *shared)
        out = out + gate * y_s.float()
    return out.to(n2.dtype)


# ------------------------------------------------------------------------------------------------ autograd nodes
class AttnBlockFn(torch.autograd.Function):
    """h1 = h + Attn(RMSNorm(h)): the attention half of ``llama.DecoderLayerFn`` as a node of its own."""

    @staticmethod
    def forward(ctx, h, pos, cos, sin, w_ln1, w_qkv, w_o, meta, b_qkv=None, w_qn=None, w_kn=None, rmul=1.0):
        B, L, H, Hkv, d, eps, recompute, window = meta
        ctx.rmul = rmul          # Granite's residual multiplier: the branch is scaled before it joins the stream
        n1, _, rstd1 = basic.rmsnorm_fwd(h, w_ln1, eps)
        qkv = basic.linear_fwd(n1, w_qkv)
        if b_qkv is not None:
            basic.bias_add_(qkv, b_qkv)
        qk_saved = ()
        if w_qn is not None and w_qn.numel() != d:       # one norm over the whole projection (OLMoE)
            from .sandwich import _qk_full_fwd
            qkv, qk_saved = _qk_full_fwd(qkv, w_qn, w_kn, H * d, Hkv * d, eps)
        elif w_qn is not None:
            qkv_raw = qkv
            qkv, rstd_qk = basic.headnorm_fwd(qkv_raw, w_qn, w_kn, H, Hkv, d, eps)
            qk_saved = (qkv_raw, rstd_qk)
        basic.rope_(qkv, pos, cos, sin, H + Hkv, d)
        att, lse = attention.attention_fwd(qkv, B, L, H, Hkv, d, window)
        h1 = basic.gemm(att, w_o, residual=h, alpha=rmul)
        ctx.meta = meta
        ctx.weights = (w_ln1, w_qkv, w_o)
        ctx.slots = tuple(_ll._slot(w) for w in ctx.weights)
        ctx.b_qkv = b_qkv
        ctx.b_slot = _ll._slot(b_qkv) if b_qkv is not None else None
        ctx.qk_w = (w_qn, w_kn)
        ctx.qk_slots = (_ll._slot(w_qn), _ll._slot(w_kn)) if w_qn is not None else (None, None)
        if recompute:
            ctx.save_for_backward(h, pos, cos, sin)
        else:
            ctx.save_for_backward(h, pos, cos, sin, rstd1, n1, qkv, att, lse, *qk_saved)
        return h1

    @staticmethod
    def backward(ctx, dh1):
        B, L, H, Hkv, d, eps, recompute, window = ctx.meta
        w_ln1, w_qkv, w_o = ctx.weights
        s_ln1, s_qkv, s_o = ctx.slots
        w_qn, w_kn = ctx.qk_w
        qkv_raw = rstd_qk = None
        full = w_qn is not None and w_qn.numel() != d
        qk_full = ()
        if recompute:
            h, pos, cos, sin = ctx.saved_tensors
            n1, _, rstd1 = basic.rmsnorm_fwd(h, w_ln1, eps)
            qkv = basic.linear_fwd(n1, w_qkv)
            if ctx.b_qkv is not None:
                basic.bias_add_(qkv, ctx.b_qkv)
            if full:
                from .sandwich import _qk_full_fwd
                qkv, qk_full = _qk_full_fwd(qkv, w_qn, w_kn, H * d, Hkv * d, eps)
            elif w_qn is not None:
                qkv_raw = qkv
                qkv, rstd_qk = basic.headnorm_fwd(qkv_raw, w_qn, w_kn, H, Hkv, d, eps)
            basic.rope_(qkv, pos, cos, sin, H + Hkv, d)
            att, lse = attention.attention_fwd(qkv, B, L, H, Hkv, d, window)
        elif full:
            h, pos, cos, sin, rstd1, n1, qkv, att, lse, *qk_full = ctx.saved_tensors
        elif w_qn is not None:
            h, pos, cos, sin, rstd1, n1, qkv, att, lse, qkv_raw, rstd_qk = ctx.saved_tensors
        else:
            h, pos, cos, sin, rstd1, n1, qkv, att, lse = ctx.saved_tensors
        dh1 = dh1.contiguous()
        da = dh1 if ctx.rmul == 1.0 else dh1 * ctx.rmul
        g_o = _ll._wgrad(da, att, w_o, s_o)
        datt = basic.linear_dgrad(da, w_o)
        del da
        dqkv = attention.attention_bwd_unrotated(datt, qkv, att, lse, B, L, H, Hkv, d, pos, cos, sin, window)
        del datt
        g_qn = g_kn = None
        if full:
            q_raw, k_raw, rq, rk = qk_full
            qw, kvw = H * d, Hkv * d
            dq, dwq = basic.rmsnorm_bwd(dqkv[:, :qw].contiguous(), q_raw, w_qn, rq)
            dk, dwk = basic.rmsnorm_bwd(dqkv[:, qw:qw + kvw].contiguous(), k_raw, w_kn, rk)
            dqkv = torch.cat([dq, dk, dqkv[:, qw + kvw:]], dim=1)
        elif w_qn is not None:
            dwq, dwk = basic.headnorm_bwd_(dqkv, qkv_raw, w_qn, w_kn, rstd_qk, H, Hkv, d)
        if w_qn is not None:
            g_qn = _ll._vec_grad(dwq, w_qn, ctx.qk_slots[0])
            g_kn = _ll._vec_grad(dwk, w_kn, ctx.qk_slots[1])
        g_b = None
        if ctx.b_qkv is not None and ctx.b_qkv.requires_grad:
            if ctx.b_slot is not None:
                basic.bias_grad(dqkv, out=ctx.b_slot.buf, accumulate=not ctx.b_slot.fresh)
                ctx.b_slot.fresh = False
            else:
                g_b = basic.bias_grad(dqkv).to(ctx.b_qkv.dtype)
        g_qkv = _ll._wgrad(dqkv, n1, w_qkv, s_qkv)
        dn1 = basic.linear_dgrad(dqkv, w_qkv)
        del dqkv
        dh, dw1 = basic.rmsnorm_bwd(dn1, h, w_ln1, rstd1, dres=dh1)
        g_ln1 = _ll._vec_grad(dw1, w_ln1, s_ln1)
        if _ll.LAYER_BACKWARD_DONE[0] is not None:      # the layer's first parameter: all of its gradients are final
            _ll.LAYER_BACKWARD_DONE[0](w_ln1)
        return dh, None, None, None, g_ln1, g_qkv, g_o, None, g_b, g_qn, g_kn, None


def _expert_wgrad(dy, x, w, slot, e, first):
    """Weight gradient of expert e's matrix (a slice of the stacked parameter). With a slot: accumulated into the
    slice of the flat fp32 gradient; else added into ``first`` (a zero-initialised fp32 tensor of w's shape)."""
    if not w.requires_grad:
        return
    if slot is not None:
        basic.linear_wgrad(dy, x, out=slot.buf[e], accumulate=True)
    else:
        basic.linear_wgrad(dy, x, out=first[e], accumulate=True)


class MoEBlockFn(torch.autograd.Function):
    """h2 = h1 + sum_k weight_k * Expert_k(n2) [+ sigmoid(n2 . w_sg) * SharedExpert(n2)], n2 = RMSNorm(h1), with the
    router's top-k experts per token. The shared expert's three tensors are optional (Qwen2-MoE has them)."""

    @staticmethod
    def forward(ctx, h1, w_ln2, w_router, w_gu, w_d, meta, w_sgu=None, w_sd=None, w_sg=None):
        eps, k, recompute, _first, renorm = meta[:5]
        rmul = meta[5] if len(meta) > 5 else 1.0         # Granite's residual multiplier on the whole expert branch
        T, hdim = h1.shape
        n2, _, rstd2 = basic.rmsnorm_fwd(h1, w_ln2, eps)
        probs, top_e, top_w = route(n2, w_router, k, renorm)
        order, inverse, counts = permutation(top_e, w_gu.shape[0])
        tok = torch.div(order, k, rounding_mode="floor")
        x_perm = n2.index_select(0, tok)
        gu, act, y = experts_forward(x_perm, counts, w_gu, w_d)
        y_tok = y.index_select(0, inverse).view(T, k, hdim)
        branch = (y_tok.float() * top_w.unsqueeze(-1)).sum(1)
        shared_saved = ()
        if w_sgu is not None:
            gu_s, act_s, y_s, gate = shared_expert_forward(n2, w_sgu, w_sd, w_sg)
            branch = branch + gate * y_s.float()
            shared_saved = (gu_s, act_s, y_s, gate)
        h2 = (h1.float() + (branch if rmul == 1.0 else branch * rmul)).to(h1.dtype)
        ctx.meta = meta
        ctx.counts = counts
        ctx.weights = (w_ln2, w_router, w_gu, w_d)
        ctx.slots = tuple(_ll._slot(w) for w in ctx.weights)
        ctx.shared = (w_sgu, w_sd, w_sg)
        ctx.shared_slots = (tuple(_ll._slot(w) if w is not None else None for w in ctx.shared) if w_sgu is not None
                            else (None, None, None))
        if recompute:
            ctx.save_for_backward(h1, top_e, order, inverse)
        else:
            ctx.save_for_backward(h1, top_e, order, inverse, rstd2, n2, probs, top_w, gu, act, y, *shared_saved)
        return h2

    @staticmethod
    def backward(ctx, dh2):
        eps, k, recompute, first_param, renorm = ctx.meta[:5]
        rmul = ctx.meta[5] if len(ctx.meta) > 5 else 1.0
        counts = ctx.counts
        w_ln2, w_router, w_gu, w_d = ctx.weights
        s_ln2, s_router, s_gu, s_d = ctx.slots
        w_sgu, w_sd, w_sg = ctx.shared
        s_sgu, s_sd, s_sg = ctx.shared_slots
        if _ll.UNIT_PRE[0] is not None:                 # the layer's backward starts here
            _ll.UNIT_PRE[0](first_param, True)
        if recompute:
            h1, top_e, order, inverse = ctx.saved_tensors
            n2, _, rstd2 = basic.rmsnorm_fwd(h1, w_ln2, eps)
            probs = torch.softmax(F.linear(n2, w_router).float(), dim=-1)
            top_p = probs.gather(1, top_e)
            top_w = top_p / top_p.sum(-1, keepdim=True) if renorm else top_p
            tok = torch.div(order, k, rounding_mode="floor")
            gu, act, y = experts_forward(n2.index_select(0, tok), counts, w_gu, w_d)
            if w_sgu is not None:
                gu_s, act_s, y_s, gate = shared_expert_forward(n2, w_sgu, w_sd, w_sg)
        else:
            h1, top_e, order, inverse, rstd2, n2, probs, top_w, gu, act, y, *rest = ctx.saved_tensors
            if w_sgu is not None:
                gu_s, act_s, y_s, gate = rest
            tok = torch.div(order, k, rounding_mode="floor")
        T, hdim = h1.shape
        E = w_gu.shape[0]
        dh2 = dh2.contiguous()
        dh2f = dh2.float()              # from here on the gradient of the BRANCH (the residual path keeps dh2)
        if rmul != 1.0:
            dh2f = dh2f * rmul
        # combine: h2 = h1 + rmul * sum_k w_k y_k
        y_tok = y.index_select(0, inverse).view(T, k, hdim)
        d_top_w = (y_tok.float() * dh2f.unsqueeze(1)).sum(-1)                        # [T, k]
        dy_perm = (dh2f.unsqueeze(1) * top_w.unsqueeze(-1)).to(y.dtype).view(T * k, hdim).index_select(0, order)
        del y_tok
        # experts
        x_perm = n2.index_select(0, tok)
        g_gu = g_d = None
        for w, s in ((w_gu, s_gu), (w_d, s_d)):
            if w.requires_grad and s is not None and s.fresh:
                s.buf.zero_()                     # experts without rows this step must not keep stale gradients
                s.fresh = False
        if w_gu.requires_grad and s_gu is None:
            g_gu = torch.zeros(w_gu.shape, dtype=torch.float32, device=w_gu.device)
        if w_d.requires_grad and s_d is None:
            g_d = torch.zeros(w_d.shape, dtype=torch.float32, device=w_d.device)
        offs, o = [], 0
        for c in counts:
            offs.append(o)
            o += c
        fuse = all(c == 0 or basic.swiglu_bwd_fusable(dy_perm[o:o + c], w_d[e], gu[o:o + c])
                   for e, (o, c) in enumerate(zip(offs, counts)))
        dgu = torch.empty_like(gu) if fuse else None
        dact = None if fuse else torch.empty_like(act)
        for e, (o, c) in enumerate(zip(offs, counts)):
            if c:
                _expert_wgrad(dy_perm[o:o + c], act[o:o + c], w_d, s_d, e, g_d)
                if fuse:     # dgrad of the expert's down projection with the SwiGLU derivative in its epilogue
                    basic.linear_dgrad_swiglu_bwd(dy_perm[o:o + c], w_d[e], gu[o:o + c], out=dgu[o:o + c])
                else:
                    basic.gemm(dy_perm[o:o + c], w_d[e], b_mn=True, out=dact[o:o + c])
        if not fuse:
            dgu = basic.swiglu_bwd(gu, dact)
            del dact
        dx_perm = torch.empty_like(x_perm)
        o = 0
        for e, c in enumerate(counts):
            if c:
                _expert_wgrad(dgu[o:o + c], x_perm[o:o + c], w_gu, s_gu, e, g_gu)
                basic.gemm(dgu[o:o + c], w_gu[e], b_mn=True, out=dx_perm[o:o + c])
            o += c
        del dgu
        dn2 = dx_perm.index_select(0, inverse).view(T, k, hdim).float().sum(1)
        # router: w = p_sel / sum(p_sel) (or w = p_sel without renormalisation), p = softmax(logits)
        if renorm:
            ssum = probs.gather(1, top_e).sum(-1, keepdim=True)
            d_top_p = (d_top_w - (d_top_w * top_w).sum(-1, keepdim=True)) / ssum
        else:
            d_top_p = d_top_w
        d_probs = torch.zeros_like(probs).scatter_(1, top_e, d_top_p)
        d_logits = probs * (d_probs - (d_probs * probs).sum(-1, keepdim=True))         # [T, E] fp32
        dn2 = dn2 + d_logits @ w_router.float()
        g_router = None
        if w_router.requires_grad:
            dwr = d_logits.t() @ n2.float()                                              # [E, h]
            g_router = _ll._vec_grad(dwr, w_router, s_router)
        g_sgu = g_sd = g_sg = None
        if w_sgu is not None:
            # h2 += gate * y_s with gate = sigmoid(n2 . w_sg), y_s = act_s w_sd^T, act_s = SwiGLU(n2 w_sgu^T)
            d_gate = (y_s.float() * dh2f).sum(-1, keepdim=True)                          # [T, 1]
            d_glogit = d_gate * gate * (1.0 - gate)
            dy_s = (dh2f * gate).to(y_s.dtype)
            g_sd = _ll._wgrad(dy_s, act_s, w_sd, s_sd)
            dgu_s = basic.linear_dgrad_swiglu_bwd(dy_s, w_sd, gu_s)
            g_sgu = _ll._wgrad(dgu_s, n2, w_sgu, s_sgu)
            dn2 = dn2 + basic.linear_dgrad(dgu_s, w_sgu).float()
            if w_sg is not None:
                dn2 = dn2 + d_glogit * w_sg.float()
                if w_sg.requires_grad:
                    g_sg = _ll._vec_grad(d_glogit.t() @ n2.float(), w_sg, s_sg)          # [1, h]
        dh1, dw2 = basic.rmsnorm_bwd(dn2.to(h1.dtype), h1, w_ln2, rstd2, dres=dh2)
        g_ln2 = _ll._vec_grad(dw2, w_ln2, s_ln2)
        if g_gu is not None:
            g_gu = g_gu.to(w_gu.dtype)
        if g_d is not None:
            g_d = g_d.to(w_d.dtype)
        return dh1, g_ln2, g_router, g_gu, g_d, None, g_sgu, g_sd, g_sg
