"""Loss math on [rows, K] tensors (PyTorch; runs on any device, differentiable by autograd).

Every loss here sees the student only through ``s[r,k] = z[r, I[r,k]]/T - lse_r`` - its log-probability at the
teacher's top-K ids under the full (cropped) vocabulary softmax - and the teacher through
``t = log_softmax(U/T over K)``. The fused LM head (``loss.head``) produces ``lse`` and ``z_k`` without forming
logits, so these functions are the whole "loss head" above the GEMM.

``reference_loss_segments`` restates the reference's per-conversation loss (utils/finetuning_utils.py:47-124) for
a whole micro-batch at once with segment reductions instead of a Python loop over conversations:

    CE(x)  : x at the label's slot inside the top-K ids, rows without a hit (or excluded rows) take the mean of
             the rows that have one; negated                                                   (:68-84)
    D      = relu(CE(s) - CE(t))                                                              (:97-102)
    kl     = sum_k e^t (t - s) ; rkl = sum_k e^s' (s' - t), s' = log_softmax(s over K)       (:104-105)
    W(x)   = mean_r x_r * ((x_r / max_r x + 1)^alpha + D_r)      per conversation            (:58-66)
    loss   = (W(kl) + W(rkl)) / 2                                                             (:107-110)
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

LOSS_KEYS = ("custom loss", "CE loss", "kl_div", "reverse kl_div", "weighted kl_div", "weighted rev. kl_div",
             "teacher CE loss", "CE diff")


def student_teacher_logprobs(lse: torch.Tensor, zk: torch.Tensor, u: torch.Tensor, valid: torch.Tensor | None,
                             temperature: float):
    """s [M,K] (not renormalised), t [M,K] (renormalised over the support at temperature T).
    ``valid`` [M,K] bool marks usable entries (ids inside the cropped vocabulary)."""
    s = zk - lse[:, None]
    ut = u / temperature
    finite = torch.isfinite(ut)
    valid = finite if valid is None else (valid & finite)      # -inf entries (no teacher target) are outside the support
    if valid is not None:
        ut = ut.masked_fill(~valid, float("-inf"))
        s = s.masked_fill(~valid, float("-inf"))
    row_ok = valid.any(-1, keepdim=True)                       # rows without any target stay finite (and unused)
    t = F.log_softmax(torch.where(row_ok, ut, torch.zeros_like(ut)), dim=-1)
    t = torch.where(valid, t, torch.full_like(t, float("-inf")))
    return s, t


def loss_rows(kind: str, s: torch.Tensor, t: torch.Tensor, jsd_renorm: bool = False) -> torch.Tensor:
    """Per-row loss [M] for kind in {kl, rkl, jsd}. Entries whose teacher log-prob is -inf (ids outside the cropped
    vocabulary) are outside the support: they contribute nothing and receive no gradient."""
    valid = torch.isfinite(t)
    zero = torch.zeros_like(t)
    t0 = torch.where(valid, t, zero)
    if kind == "kl":
        s0 = torch.where(valid, s, zero)
        return torch.where(valid, t0.exp() * (t0 - s0), zero).sum(-1)
    row_ok = valid.any(-1, keepdim=True)
    s_in = torch.where(valid, s, torch.full_like(s, float("-inf")))
    s1 = torch.where(valid, F.log_softmax(torch.where(row_ok, s_in, zero), dim=-1), zero)
    if kind == "rkl":
        return torch.where(valid, s1.exp() * (s1 - t0), zero).sum(-1)
    if kind == "jsd":
        q = s1 if jsd_renorm else torch.where(valid, s, zero)
        m = torch.logaddexp(t0, q) - 0.6931471805599453
        return 0.5 * torch.where(valid, t0.exp() * (t0 - m) + q.exp() * (q - m), zero).sum(-1)
    raise ValueError(f"unknown loss kind {kind}")


class _SegSumFn(torch.autograd.Function):
    """Sum of ``x`` per conversation on CUDA with a fixed order of additions (csrc/loss/segment.cu): ``seg`` must be
    non-decreasing, which is how micro-batches are laid out (one conversation's rows after the other's)."""

    @staticmethod
    def forward(ctx, x, seg, n):
        from ..ops import _lib
        out = torch.empty(n, dtype=torch.float32, device=x.device)
        _lib.check(_lib.kernels().b200_segment_reduce(_lib.ptr(x), _lib.ptr(seg), _lib.ptr(out), x.numel(), n, 0,
                                                      _lib.stream()), "b200_segment_reduce")
        ctx.save_for_backward(seg)
        return out

    @staticmethod
    def backward(ctx, g):
        (seg,) = ctx.saved_tensors
        return g.index_select(0, seg), None, None


def _seg_sum(x, seg, n):
    """out[c] = sum of x over the rows of conversation c. Bit-repeatable on both devices: an ordered loop on CPU, the
    segment kernel on CUDA (``index_add_`` there is an atomic scatter whose order changes from run to run)."""
    if x.is_cuda:
        return _SegSumFn.apply(x.float().contiguous(), seg.contiguous(), n)
    return torch.zeros(n, dtype=x.dtype, device=x.device).index_add_(0, seg, x)


def seg_count(seg, n, dtype=torch.float32):
    """Number of rows of each conversation."""
    if seg.is_cuda:
        from ..ops import _lib
        out = torch.empty(n, dtype=torch.float32, device=seg.device)
        _lib.check(_lib.kernels().b200_segment_reduce(None, _lib.ptr(seg.contiguous()), _lib.ptr(out), seg.numel(), n, 2,
                                                      _lib.stream()), "b200_segment_reduce")
        return out.to(dtype)
    return torch.zeros(n, dtype=dtype, device=seg.device).index_add_(0, seg, torch.ones(seg.numel(), dtype=dtype))


def _seg_max(x, seg, n):
    out = torch.full((n,), float("-inf"), dtype=x.dtype, device=x.device)
    return out.scatter_reduce(0, seg, x, reduce="amax", include_self=True)


def reference_loss_segments(s: torch.Tensor, t: torch.Tensor, ids: torch.Tensor, labels: torch.Tensor,
                            avoid: torch.Tensor, seg: torch.Tensor, n_seg: int, alpha: float):
    """Reference loss for a batch of conversations.

    s, t      [M,K] student / teacher log-probs at the teacher ids (see ``student_teacher_logprobs``)
    ids       [M,K] teacher token ids
    labels    [M]   id of the true next token of each row, -1 where the row has none (last row of a conversation)
    avoid     [M]   bool, rows left out of the cross-entropy term (last row of every content range when a
                    conversation has several ranges)
    seg       [M]   conversation index of each row, in [0, n_seg)
    Returns (train_loss_per_conversation [n_seg], dict of logged per-conversation scalars [n_seg] each).
    """
    has_label = labels >= 0
    hit = (ids == labels[:, None]) & has_label[:, None] & (~avoid)[:, None]
    valid = hit.any(-1)

    def ce(x):
        picked = torch.where(hit, x, torch.zeros_like(x)).sum(-1)                       # value at the label slot
        n_valid = _seg_sum(valid.to(x.dtype), seg, n_seg)
        # a conversation none of whose labels is inside the teacher's top-K has no CE signal: use 0 there (the
        # reference divides by zero and turns the whole step into NaN)
        mean_valid = _seg_sum(torch.where(valid, picked, torch.zeros_like(picked)), seg, n_seg) / n_valid.clamp_min(1)
        filled = torch.where(valid, picked, mean_valid[seg])
        return -filled

    ce_s, ce_t = ce(s), ce(t)
    ce_diff = ce_s - ce_t
    d = torch.where(has_label, torch.relu(ce_diff), torch.zeros_like(ce_diff))          # last row: padded 0
    kl = loss_rows("kl", s, t)
    rkl = loss_rows("rkl", s, t)
    n_rows = seg_count(seg, n_seg, s.dtype)
    n_lab = _seg_sum(has_label.to(s.dtype), seg, n_seg)

    def weighted(x):
        w = (x / _seg_max(x, seg, n_seg)[seg] + 1).pow(alpha) + d
        return _seg_sum(x * w, seg, n_seg) / n_rows

    wkl, wrkl = weighted(kl), weighted(rkl)
    custom = (wkl + wrkl) / 2

    def lab_mean(x):
        return _seg_sum(torch.where(has_label, x, torch.zeros_like(x)), seg, n_seg) / n_lab

    logs = {
        "custom loss": custom, "CE loss": lab_mean(ce_s), "kl_div": _seg_sum(kl, seg, n_seg) / n_rows,
        "reverse kl_div": _seg_sum(rkl, seg, n_seg) / n_rows, "weighted kl_div": wkl, "weighted rev. kl_div": wrkl,
        "teacher CE loss": lab_mean(ce_t), "CE diff": lab_mean(ce_diff),
    }
    return custom, logs


def calculate_divergence(student_logits: torch.Tensor, teacher_logits: torch.Tensor, indices: torch.Tensor,
                         convo_CE_tokens: torch.Tensor, alpha: float, avoid_indices: torch.Tensor) -> dict:
    """One conversation, full student logits [Lc, Vc] (already divided by T) - same call shape and returned keys as
    the reference's ``calculate_divergence``; used by the CPU path and as a cross-check of the fused path."""
    n = min(student_logits.size(0), teacher_logits.size(0), indices.size(0))
    z = student_logits[:n].float()
    lse = torch.logsumexp(z, dim=-1)
    zk = torch.gather(z, 1, indices[:n].long())
    s = zk - lse[:, None]
    t = F.log_softmax(teacher_logits[:n].float(), dim=-1)
    labels = torch.full((n,), -1, dtype=torch.long, device=z.device)
    m = min(n, convo_CE_tokens.numel())
    labels[:m] = convo_CE_tokens[:m]
    avoid = torch.zeros(n, dtype=torch.bool, device=z.device)
    if avoid_indices is not None and avoid_indices.numel():
        avoid[avoid_indices[avoid_indices < n].long()] = True
    seg = torch.zeros(n, dtype=torch.long, device=z.device)
    custom, logs = reference_loss_segments(s, t, indices[:n].long(), labels, avoid, seg, 1, alpha)
    out = {k: v[0] for k, v in logs.items()}
    out["train_loss"] = custom[0]
    return out
