"""LM head fused with the distillation loss.

``lmhead_stats(Hc, W, ids, T, vocab)`` -> ``(lse [M], zk [M,K])`` is the differentiable primitive: the full-vocabulary
log-sum-exp of ``Hc W^T / T`` and the scaled logits at the teacher's ids. On CUDA it is one tcgen05 GEMM whose
epilogue does the online softmax statistics and the sparse gather (csrc/loss/distill_head.cu); its backward
recomputes the GEMM, writes bf16 dlogits in row chunks bounded by a byte budget and feeds them to the dgrad /
wgrad GEMMs. fp32 logits never exist. Any loss written on ``(lse, zk)`` trains through it (the reference loss does).

``fused_distill_rows`` additionally evaluates forward KL / reverse KL / JSD and their gradient coefficients in a
row kernel, so the training step for those losses is: GEMM+stats, row kernel, GEMM+dlogits, dgrad, wgrad.

Teacher ids must be sorted ascending within each row (``sort_teacher_rows``); the loss is invariant to that order.
"""
from __future__ import annotations

import torch

from ..ops import _lib, basic
from ..ops._lib import _VP, _I, _LL, _F
from ..models.llama import _slot
from . import divergence as dv

_lib.register("b200_head_num_tiles", [_I])
_lib.register("b200_lmhead_lse_gather", [_VP, _VP, _I, _I, _I, _LL, _LL, _VP, _I, _F, _VP, _VP, _VP, _VP])
_lib.register("b200_distill_rows", [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _F, _VP])
_lib.register("b200_lmhead_dlogits", [_VP, _VP, _I, _I, _I, _LL, _LL, _VP, _VP, _VP, _VP, _VP, _I, _F, _VP, _LL, _VP])

KIND_CODES = {"kl": 0, "rkl": 1, "jsd": 2, "jsd_renorm": 3, "none": 4}
DZ_CHUNK_BYTES = 2 << 30  # bf16 dlogits materialised per backward chunk


def sort_teacher_rows(ids: torch.Tensor, u: torch.Tensor):
    """Sort each row by token id (what the fused kernels expect). Returns (ids int32, u fp32)."""
    sid, order = torch.sort(ids.long(), dim=-1)
    return sid.to(torch.int32).contiguous(), torch.gather(u.float(), 1, order).contiguous()


def _pass1(Hc, W, ids, inv_T, vocab):
    M, h = Hc.shape
    K = ids.shape[1]
    lib = _lib.kernels()
    nt = lib.b200_head_num_tiles(vocab)
    dev = Hc.device
    zk = torch.zeros((M, K), dtype=torch.float32, device=dev)
    pmax = torch.empty((nt, M), dtype=torch.float32, device=dev)
    psum = torch.empty((nt, M), dtype=torch.float32, device=dev)
    _lib.check(lib.b200_lmhead_lse_gather(_lib.ptr(Hc), _lib.ptr(W), M, vocab, h, Hc.stride(0), W.stride(0),
                                          _lib.ptr(ids), K, float(inv_T), _lib.ptr(zk), _lib.ptr(pmax), _lib.ptr(psum),
                                          _lib.stream()), "b200_lmhead_lse_gather")
    return zk, pmax, psum, nt


def _rows(pmax, psum, zk, u, ids, M, K, nt, vocab, kind, inv_T):
    dev = pmax.device
    lse = torch.empty(M, dtype=torch.float32, device=dev)
    if kind == 4:
        _lib.check(_lib.kernels().b200_distill_rows(_lib.ptr(pmax), _lib.ptr(psum), None, None, None, _lib.ptr(lse),
                                                    None, None, None, M, max(K, 1), nt, vocab, 4, float(inv_T),
                                                    _lib.stream()), "b200_distill_rows")
        return lse, None, None, None
    loss = torch.empty(M, dtype=torch.float32, device=dev)
    a = torch.empty((M, K), dtype=torch.float32, device=dev)
    A = torch.empty(M, dtype=torch.float32, device=dev)
    _lib.check(_lib.kernels().b200_distill_rows(_lib.ptr(pmax), _lib.ptr(psum), _lib.ptr(zk), _lib.ptr(u), _lib.ptr(ids),
                                                _lib.ptr(lse), _lib.ptr(loss), _lib.ptr(a), _lib.ptr(A), M, K, nt, vocab,
                                                kind, float(inv_T), _lib.stream()), "b200_distill_rows")
    return lse, loss, a, A


def _backward_chunks(Hc, W, ids, a, A, lse, g, inv_T, vocab, w_slot, need_dh: bool):
    """dH [M,h] (or None) and the LM-head weight gradient (into the slot, or returned) from the dlogits pass."""
    M, h = Hc.shape
    K = ids.shape[1]
    lib = _lib.kernels()
    ldz = (vocab + 7) // 8 * 8
    rows = max(128, min(M, (DZ_CHUNK_BYTES // (2 * ldz)) // 128 * 128))
    dz = torch.empty((min(rows, M), ldz), dtype=torch.bfloat16, device=Hc.device)
    dH = torch.empty_like(Hc) if need_dh else None
    dW = None
    Wc = W[:vocab]
    want_w = W.requires_grad
    if want_w and w_slot is None:
        dW = torch.zeros((W.shape[0], h), dtype=torch.float32, device=Hc.device)
    for r0 in range(0, M, rows):
        r1 = min(M, r0 + rows)
        n = r1 - r0
        _lib.check(lib.b200_lmhead_dlogits(_lib.ptr(Hc[r0:r1]), _lib.ptr(W), n, vocab, h, Hc.stride(0), W.stride(0),
                                           _lib.ptr(ids[r0:r1]), _lib.ptr(a[r0:r1]), _lib.ptr(A[r0:r1]),
                                           _lib.ptr(lse[r0:r1]), _lib.ptr(g[r0:r1]), K, float(inv_T), _lib.ptr(dz), ldz,
                                           _lib.stream()), "b200_lmhead_dlogits")
        dzv = dz[:n, :vocab]
        if need_dh:
            basic.gemm(dzv, Wc, b_mn=True, out=dH[r0:r1])
        if want_w:
            if w_slot is not None:
                basic.gemm(dzv, Hc[r0:r1], a_mn=True, b_mn=True, out=w_slot.buf[:vocab], accumulate=not w_slot.fresh)
                if w_slot.fresh and vocab < W.shape[0]:
                    w_slot.buf[vocab:].zero_()
                w_slot.fresh = False
            else:
                basic.gemm(dzv, Hc[r0:r1], a_mn=True, b_mn=True, out=dW[:vocab], accumulate=True)
    return dH, (dW.to(W.dtype) if dW is not None else None)


class _LmHeadStatsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Hc, W, ids, inv_T, vocab):
        M, K = ids.shape
        zk, pmax, psum, nt = _pass1(Hc, W, ids, inv_T, vocab)
        lse, _, _, _ = _rows(pmax, psum, None, None, None, M, K, nt, vocab, 4, inv_T)
        ctx.save_for_backward(Hc, ids, lse)
        ctx.W, ctx.slot, ctx.inv_T, ctx.vocab = W, _slot(W), inv_T, vocab
        return lse, zk

    @staticmethod
    def backward(ctx, dlse, dzk):
        Hc, ids, lse = ctx.saved_tensors
        M = Hc.shape[0]
        a = (dzk if dzk is not None else torch.zeros(ids.shape, device=Hc.device)).float().contiguous()
        A = (-(dlse.float()) if dlse is not None else torch.zeros(M, device=Hc.device)).contiguous()
        g = torch.ones(M, dtype=torch.float32, device=Hc.device)
        dH, dW = _backward_chunks(Hc, ctx.W, ids, a, A, lse, g, ctx.inv_T, ctx.vocab, ctx.slot, ctx.needs_input_grad[0])
        return dH, dW, None, None, None


class _FusedDistillFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Hc, W, ids, u, kind, inv_T, vocab):
        M, K = ids.shape
        zk, pmax, psum, nt = _pass1(Hc, W, ids, inv_T, vocab)
        lse, loss, a, A = _rows(pmax, psum, zk, u, ids, M, K, nt, vocab, kind, inv_T)
        ctx.save_for_backward(Hc, ids, lse, a, A)
        ctx.W, ctx.slot, ctx.inv_T, ctx.vocab = W, _slot(W), inv_T, vocab
        return loss

    @staticmethod
    def backward(ctx, dloss):
        Hc, ids, lse, a, A = ctx.saved_tensors
        g = dloss.float().contiguous()
        dH, dW = _backward_chunks(Hc, ctx.W, ids, a, A, lse, g, ctx.inv_T, ctx.vocab, ctx.slot, ctx.needs_input_grad[0])
        return dH, dW, None, None, None, None, None


def _torch_stats(Hc, W, ids, inv_T, vocab):
    z = (Hc.float() @ W[:vocab].float().t()) * inv_T
    lse = torch.logsumexp(z, dim=-1)
    safe = ids.long().clamp(max=vocab - 1)
    zk = torch.gather(z, 1, safe)
    return lse, torch.where(ids.long() < vocab, zk, torch.zeros_like(zk))


def lmhead_stats(Hc: torch.Tensor, W: torch.Tensor, ids: torch.Tensor, temperature: float = 1.0,
                 vocab: int | None = None):
    """(lse [M], zk [M,K]) of z = Hc W[:vocab]^T / T. ids: int32 [M,K], ascending per row on CUDA."""
    vocab = min(vocab or W.shape[0], W.shape[0])
    if not Hc.is_cuda:
        return _torch_stats(Hc, W, ids, 1.0 / temperature, vocab)
    return _LmHeadStatsFn.apply(Hc.contiguous(), W, ids.contiguous(), 1.0 / temperature, vocab)


def fused_distill_rows(Hc, W, ids, u, kind: str, temperature: float = 1.0, vocab: int | None = None,
                       jsd_renorm: bool = False) -> torch.Tensor:
    """Per-row loss [M] for kind in {kl, rkl, jsd}. u: stored teacher log-probs (T = 1) aligned with ids."""
    vocab = min(vocab or W.shape[0], W.shape[0])
    if kind == "jsd" and jsd_renorm:
        kind = "jsd_renorm"
    if not Hc.is_cuda:
        lse, zk = _torch_stats(Hc, W, ids, 1.0 / temperature, vocab)
        s, t = dv.student_teacher_logprobs(lse, zk, u.float(), ids.long() < vocab, temperature)
        if kind == "jsd_renorm":
            return dv.loss_rows("jsd", s, t, jsd_renorm=True)
        return dv.loss_rows(kind, s, t)
    return _FusedDistillFn.apply(Hc.contiguous(), W, ids.contiguous(), u.float().contiguous(), KIND_CODES[kind],
                                 1.0 / temperature, vocab)


def distill_head_loss(Hc, W, ids, u, *, kind: str, temperature: float, vocab: int | None, alpha: float = 2.0,
                      labels=None, avoid=None, seg=None, n_seg: int = 1, jsd_renorm: bool = False):
    """Loss of a micro-batch of content rows.

    Returns (train_loss scalar = sum over conversations of the per-conversation loss, logs dict of detached sums
    over conversations). For kl / rkl / jsd the per-conversation loss is the mean over that conversation's rows.
    """
    vocab = min(vocab or W.shape[0], W.shape[0])
    if kind == "reference":
        lse, zk = lmhead_stats(Hc, W, ids, temperature, vocab)
        s, t = dv.student_teacher_logprobs(lse, zk, u.float(), ids.long() < vocab, temperature)
        custom, logs = dv.reference_loss_segments(s, t, ids.long(), labels, avoid, seg, n_seg, alpha)
        return custom.sum(), {k: v.detach().sum() for k, v in logs.items()}
    rows = fused_distill_rows(Hc, W, ids, u, kind, temperature, vocab, jsd_renorm)
    per_convo = dv._seg_sum(rows, seg, n_seg) / dv.seg_count(seg, n_seg, rows.dtype)
    key = {"kl": "kl_div", "rkl": "reverse kl_div", "jsd": "jsd"}[kind]
    return per_convo.sum(), {key: per_convo.detach().sum(), "custom loss": per_convo.detach().sum()}
