"""Vocabulary-parallel LM head + loss inside data-parallel training (config key ``vocab_parallel_loss``).

Every rank trains on its own micro-batch, but the LM head is split over the vocabulary: rank r owns rows
[r*Vl, (r+1)*Vl) of the head. Per micro-batch the ranks' content-row hidden states, teacher ids / log-probs and
per-row loss weights are all-gathered; ``parallel.vp_head.VocabParallelHead`` then runs its fused passes on ALL
ranks' rows against this rank's slice (no rank ever forms logits of the whole vocabulary, and the cross-rank softmax
statistics are combined by peer loads inside its kernels); each rank gets back the loss rows, the hidden-state
gradient of every row summed over the slices, and the weight gradient of its slice over every rank's rows.

Equivalence with plain data parallelism: a rank keeps the hidden-state gradient of its OWN rows (other ranks' losses
do not depend on them), and writes the slice's weight gradient into its slice of the flat gradient with zeros
elsewhere, so the data-parallel reduction (a sum over ranks) delivers exactly the head gradient that replicated heads
would have summed to. Losses: kl, rkl, jsd (the reference's weighted loss needs per-conversation statistics of the
whole row set and stays on the replicated head).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..loss import divergence as dv
from ..models.llama import _slot

ROW_UNIT = 128


class VocabParallelLoss:
    def __init__(self, model, vocab: int, kind: str, temperature: float, max_rows_per_rank: int, jsd_renorm: bool = False):
        if kind not in ("kl", "rkl", "jsd"):
            raise ValueError("vocab_parallel_loss supports the kl, rkl and jsd losses")
        self.kind = "jsd_renorm" if (kind == "jsd" and jsd_renorm) else kind
        self.T = float(temperature)
        self.vocab = int(vocab)
        self.model = model
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self.dev = model.embed_tokens.device
        self.h = model.cfg.hidden_size
        unit = ROW_UNIT
        self.max_rows = -(-int(max_rows_per_rank) // unit) * unit
        self._head = None           # built at the first call, when K is known
        self._mx = None

    def _build(self, K: int):
        from ..parallel.tp import TPGroup
        from ..parallel.vp_head import VocabParallelHead
        total = self.max_rows * self.world
        grp = TPGroup(self.dev, total, self.h, dtype=self.model.lm_head.dtype)
        self._head = VocabParallelHead(grp, total, self.h, K, self.vocab)

    def _gather(self, t: torch.Tensor) -> torch.Tensor:
        out = torch.empty((self.world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous()) if t.is_cuda else dist.all_gather(list(out.chunk(self.world)), t.contiguous())
        return out

    def __call__(self, Hc, W, ids, u, seg, n_seg):
        """Returns (sum over this rank's conversations of the mean row loss [differentiable], logs)."""
        M, K = ids.shape
        if self._head is None:
            self._build(K)
        head = self._head
        # every rank pads to the largest row count of the step (a multiple of 128 rows)
        m = torch.tensor([M], dtype=torch.int64, device=Hc.device)
        dist.all_reduce(m, op=dist.ReduceOp.MAX)
        Mp = -(-int(m.item()) // ROW_UNIT) * ROW_UNIT
        if Mp > self.max_rows:
            raise ValueError(f"{Mp} content rows in a micro-batch exceed the {self.max_rows} the vocabulary-parallel head was sized for")
        n_rows = dv.seg_count(seg, n_seg, torch.float32)
        g_rows = (1.0 / n_rows)[seg]                                   # d(total) / d(row loss): mean per conversation
        pad = Mp - M
        Hp = torch.cat([Hc.detach(), Hc.new_zeros((pad, Hc.shape[1]))]) if pad else Hc.detach()
        # padding rows: K distinct ascending ids with uniform targets and zero weight (they cost FLOPs, not correctness)
        ip = torch.cat([ids, torch.arange(K, dtype=ids.dtype, device=ids.device).repeat(pad, 1)]) if pad else ids
        up = torch.cat([u.float(), u.new_zeros((pad, K), dtype=torch.float32)]) if pad else u.float()
        gp = torch.cat([g_rows, g_rows.new_zeros(pad)]) if pad else g_rows
        H_all, i_all, u_all, g_all = self._gather(Hp), self._gather(ip), self._gather(up), self._gather(gp)
        vl, lo, valid = head.vl, head.lo, head.valid
        W_slice = W.detach()[lo:lo + vl]
        if W_slice.shape[0] < vl:                                      # last rank: zero-padded slice
            Wp = W.new_zeros((vl, W.shape[1]))
            Wp[:W_slice.shape[0]] = W_slice
            W_slice = Wp
        loss_rows, dH_all, dW = head.loss_and_grads(H_all, W_slice.contiguous(), i_all.contiguous(), u_all.contiguous(),
                                                    self.kind, self.T, grad_rows=g_all.contiguous(),
                                                    need_dh=Hc.requires_grad)
        mine = slice(self.rank * Mp, self.rank * Mp + M)
        total = (loss_rows[mine] * g_rows).sum()
        dH = dH_all[mine] if dH_all is not None else None
        out = _VPLossFn.apply(Hc, W, total.detach(), dH, dW, lo, valid)
        key = {"kl": "kl_div", "rkl": "reverse kl_div", "jsd": "jsd", "jsd_renorm": "jsd"}[self.kind]
        return out, {key: total.detach(), "custom loss": total.detach()}


class _VPLossFn(torch.autograd.Function):
    """Carries the gradients that the fused head already computed into autograd."""

    @staticmethod
    def forward(ctx, Hc, W, total, dH, dW, lo, valid):
        ctx.save_for_backward(dH if dH is not None else torch.empty(0), dW)
        ctx.has_dh = dH is not None
        ctx.W, ctx.slot, ctx.lo, ctx.valid = W, _slot(W), lo, valid
        return total.clone()

    @staticmethod
    def backward(ctx, g):
        dH, dW = ctx.saved_tensors
        gH = (dH.float() * g).to(dH.dtype) if ctx.has_dh else None
        W, slot, lo, valid = ctx.W, ctx.slot, ctx.lo, ctx.valid
        gW = None
        if W.requires_grad:
            piece = dW[:valid].float() * g
            if slot is not None:        # this rank's slice of the flat gradient; the other rows are zero on this rank
                if slot.fresh:
                    slot.buf.zero_()
                    slot.fresh = False
                slot.buf[lo:lo + valid] += piece
            else:
                gW = torch.zeros_like(W, dtype=torch.float32)
                gW[lo:lo + valid] = piece
                gW = gW.to(W.dtype)
        return gH, gW, None, None, None, None, None
