"""Vocabulary-parallel fused LM head + distillation loss (kernels: csrc/loss/distill_head.cu, csrc/comm/tp_gemm.cu).

The reference materialises the student's full fp32 logits on one GPU (classes/student/model.py:408) and evaluates
the loss with ATen ops (utils/finetuning_utils.py:47-124). Here the LM head is split over the vocabulary: rank r holds
rows [r*Vl, (r+1)*Vl) of W. For hidden states Hc [M, h] that every rank holds:

    pass 1   tcgen05 GEMM on the slice; the epilogue keeps (max, sum-exp) per row and gathers z at the teacher ids that
             fall into the slice                                                    (no logits are written)
    combine  ONE kernel reads all ranks' partial statistics out of their memory over NVLink (peer loads) and forms the
             whole-vocabulary log-sum-exp and the complete z_k
    rows     KL / reverse KL / JSD per row and the gradient coefficients (a_k, A)   (replicated, tiny)
    pass 2   the slice GEMM again; bf16 dlogits of the slice
    wgrad    dW_slice += dlogits^T Hc                                               (local)
    dgrad    dH = sum over ranks dlogits_slice W_slice: GEMM -> reduce-scatter in one kernel (peer stores from the
             epilogue), then an all-gather by peer stores

On CPU / gloo the same interface runs with PyTorch math and ``all_reduce`` (tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..loss import divergence as dv
from ..loss.head import KIND_CODES
from ..ops import _lib, basic
from ..ops._lib import _VP, _I, _LL, _F
from .tp import TPGroup

_lib.register("b200_lmhead_lse_gather_shard", [_VP, _VP, _I, _I, _I, _LL, _LL, _VP, _I, _F, _I, _VP, _VP, _VP, _VP])
_lib.register("b200_lmhead_dlogits_shard", [_VP, _VP, _I, _I, _I, _LL, _LL, _VP, _VP, _VP, _VP, _VP, _I, _F, _I, _VP, _LL, _VP])
_lib.register("b200_vp_combine", [_VP, _VP, _VP, _I, _I, _I, _I, _VP, _VP, _VP, _VP])


def vocab_slice(vocab: int, rank: int, world: int) -> tuple[int, int, int]:
    """(rows per rank rounded up to 8, first id, number of valid ids) of rank's slice of a ``vocab``-sized head."""
    vl = -(-(-(-vocab // world)) // 8) * 8
    lo = min(rank * vl, vocab)
    return vl, lo, min((rank + 1) * vl, vocab) - lo


class VocabParallelHead:
    def __init__(self, group: TPGroup, max_rows: int, hidden: int, topk: int, vocab: int):
        self.g = group
        self.vocab = vocab
        self.K = topk
        self.h = hidden
        self.vl, self.lo, self.valid = vocab_slice(vocab, group.rank, group.world)
        self.native = group.native
        if not self.native:
            return
        from .p2p import SymmetricBuffer
        dev = group.device
        self.nt = _lib.kernels().b200_head_num_tiles(self.vl)
        self.max_rows = max_rows
        self.pmax = SymmetricBuffer(self.nt * max_rows, torch.float32, dev, group.group)
        self.psum = SymmetricBuffer(self.nt * max_rows, torch.float32, dev, group.group)
        self.zk = SymmetricBuffer(max_rows * topk, torch.float32, dev, group.group)
        self.dh = SymmetricBuffer(max_rows * hidden, torch.bfloat16, dev, group.group)
        torch.cuda.synchronize(dev)
        dist.barrier(group.group)

    # ------------------------------------------------------------------ forward + backward in one call
    def loss_and_grads(self, Hc: torch.Tensor, W_slice: torch.Tensor, ids: torch.Tensor, u: torch.Tensor, kind: str,
                       temperature: float, grad_rows: torch.Tensor | None = None, dW: torch.Tensor | None = None,
                       need_dh: bool = True):
        """Hc [M, h]; W_slice [Vl, h] (this rank's rows, zero-padded); ids int32 [M, K] ascending per row, global ids;
        u fp32 [M, K] stored teacher log-probs. grad_rows [M] = d(total)/d(loss_row) (default: 1/M, the mean).
        Returns (loss_rows [M], dH [M, h] summed over ranks or None, dW fp32 [Vl, h] accumulated into ``dW``)."""
        M, h = Hc.shape
        K = ids.shape[1]
        g = self.g
        inv_T = 1.0 / temperature
        if grad_rows is None:
            grad_rows = torch.full((M,), 1.0 / M, dtype=torch.float32, device=Hc.device)
        if not self.native:
            return self._reference(Hc, W_slice, ids, u, kind, temperature, grad_rows, dW, need_dh)
        if M > self.max_rows or K != self.K:
            raise ValueError("VocabParallelHead was sized for other shapes")
        lib = _lib.kernels()
        dev = Hc.device
        n = max(self.valid, 8)
        pmax = self.pmax.tensor[: self.nt * M]
        psum = self.psum.tensor[: self.nt * M]
        zk = self.zk.tensor[: M * K]
        g.barrier()                    # every rank has consumed the partials of the previous call
        zk.zero_()
        _lib.check(lib.b200_lmhead_lse_gather_shard(_lib.ptr(Hc), _lib.ptr(W_slice), M, n, h, Hc.stride(0),
                                                    W_slice.stride(0), _lib.ptr(ids), K, float(inv_T), self.lo,
                                                    _lib.ptr(zk), _lib.ptr(pmax), _lib.ptr(psum), _lib.stream()),
                   "b200_lmhead_lse_gather_shard")
        g.barrier()                    # all partials are in place
        cm = torch.empty(M, dtype=torch.float32, device=dev)
        cs = torch.empty(M, dtype=torch.float32, device=dev)
        czk = torch.empty((M, K), dtype=torch.float32, device=dev)
        _lib.check(lib.b200_vp_combine(self.pmax.c_ptrs, self.psum.c_ptrs, self.zk.c_ptrs, g.world, self.nt, M, K,
                                       _lib.ptr(cm), _lib.ptr(cs), _lib.ptr(czk), _lib.stream()), "b200_vp_combine")
        lse = torch.empty(M, dtype=torch.float32, device=dev)
        loss = torch.empty(M, dtype=torch.float32, device=dev)
        a = torch.empty((M, K), dtype=torch.float32, device=dev)
        A = torch.empty(M, dtype=torch.float32, device=dev)
        _lib.check(lib.b200_distill_rows(_lib.ptr(cm), _lib.ptr(cs), _lib.ptr(czk), _lib.ptr(u), _lib.ptr(ids),
                                         _lib.ptr(lse), _lib.ptr(loss), _lib.ptr(a), _lib.ptr(A), M, K, 1, self.vocab,
                                         KIND_CODES[kind], float(inv_T), _lib.stream()), "b200_distill_rows")
        ldz = self.vl
        dz = torch.empty((M, ldz), dtype=torch.bfloat16, device=dev)
        if ldz > n:
            dz[:, n:].zero_()
        _lib.check(lib.b200_lmhead_dlogits_shard(_lib.ptr(Hc), _lib.ptr(W_slice), M, n, h, Hc.stride(0),
                                                 W_slice.stride(0), _lib.ptr(ids), _lib.ptr(a), _lib.ptr(A),
                                                 _lib.ptr(lse), _lib.ptr(grad_rows), K, float(inv_T), self.lo,
                                                 _lib.ptr(dz), ldz, _lib.stream()), "b200_lmhead_dlogits_shard")
        if dW is None:
            dW = torch.zeros((self.vl, h), dtype=torch.float32, device=dev)
        basic.gemm(dz, Hc, a_mn=True, b_mn=True, out=dW, accumulate=True)
        dH = None
        if need_dh:
            Wt = W_slice.t().contiguous()                      # [h, Vl]: the reduction dimension contiguous
            shard = g.gemm_rs(dz, Wt)                           # [M / world, h], summed over ranks
            Ms = M // g.world
            _lib.check(lib.b200_p2p_allgather(self.dh.c_ptrs, _lib.ptr(shard), g.rank * Ms * h * 2, Ms * h * 2, g.rank,
                                              g.world, 0, _lib.stream()), "b200_p2p_allgather")
            g.barrier()                # every rank's rows have landed
            dH = self.dh.tensor[: M * h].view(M, h)
        return loss, dH, dW

    # ------------------------------------------------------------------ PyTorch statement (CPU ranks, oracle)
    def _reference(self, Hc, W_slice, ids, u, kind, temperature, grad_rows, dW, need_dh):
        g = self.g
        Hc32 = Hc.float().detach().requires_grad_(True)
        W32 = W_slice.float().detach().requires_grad_(True)
        z = (Hc32 @ W32[: max(self.valid, 0)].t()) / temperature
        m = z.max(dim=-1).values.detach() if self.valid > 0 else torch.full((Hc.shape[0],), -1e30)
        gm = m.clone()
        dist.all_reduce(gm, op=dist.ReduceOp.MAX, group=g.group)
        se = torch.exp(z - gm[:, None]).sum(-1)
        se_all = _AllReduceSum.apply(se, g.group)
        lse = gm + torch.log(se_all)
        local = ids.long() - self.lo
        inside = (local >= 0) & (local < self.valid)
        zk_part = torch.where(inside, torch.gather(z, 1, local.clamp(0, max(self.valid - 1, 0))), torch.zeros(()))
        zk = _AllReduceSum.apply(zk_part, g.group)
        s, t = dv.student_teacher_logprobs(lse, zk, u.float(), ids.long() < self.vocab, temperature)
        rows = dv.loss_rows("jsd", s, t, jsd_renorm=True) if kind == "jsd_renorm" else dv.loss_rows(kind, s, t)
        (rows * grad_rows).sum().backward()
        dw = torch.zeros((self.vl, Hc.shape[1]))
        dw.copy_(W32.grad)
        if dW is not None:
            dW += dw
        else:
            dW = dw
        dH = None
        if need_dh:
            dH = Hc32.grad.clone()
            dist.all_reduce(dH, group=g.group)
            dH = dH.to(Hc.dtype)
        return rows.detach(), dH, dW


class _AllReduceSum(torch.autograd.Function):
    """y = sum over ranks of x; every rank's loss uses y, so dL/dx = dL/dy on every rank (the loss is replicated and
    each rank backpropagates its own copy once)."""

    @staticmethod
    def forward(ctx, x, group):
        y = x.detach().clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, gy):
        return gy, None
