"""Top-K log-prob extraction and multi-teacher top-K merge (csrc/loss/topk_logprob.cu) with PyTorch restatements."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import _VP, _I, _LL

_lib.register("b200_topk_logprob", [_VP, _LL, _I, _I, _I, _VP, _VP, _VP])
_lib.register("b200_topk_merge", [_VP, _VP, _VP, _VP, _I, _I, _VP, _VP, _VP])
_lib.register("b200_remap_topk", [_VP, _VP, _VP, _I, _I, _I, _I, _VP, _VP, _VP])
_lib.register("b200_logprob_full", [_VP, _LL, _I, _I, _VP, _LL, _VP])


def topk_logprob(logits: torch.Tensor, vocab: int, k: int):
    """(fp16 log-probs [rows, k] sorted descending, int32 ids [rows, k]) of log_softmax(logits[:, :vocab])."""
    rows = logits.shape[0]
    if not logits.is_cuda:
        z = logits[:, :vocab].float()
        _, i = torch.sort(z, dim=-1, descending=True, stable=True)   # rank on the logits: subtraction can merge values
        i = i[:, :k]
        lp = torch.gather(z, 1, i) - torch.logsumexp(z, dim=-1, keepdim=True)
        return lp.to(torch.float16), i.to(torch.int32)
    if logits.dtype != torch.float32 or logits.stride(-1) != 1:
        raise TypeError("topk_logprob: logits must be fp32 with contiguous rows")
    out_lp = torch.empty((rows, k), dtype=torch.float16, device=logits.device)
    out_ix = torch.empty((rows, k), dtype=torch.int32, device=logits.device)
    _lib.check(_lib.kernels().b200_topk_logprob(_lib.ptr(logits), logits.stride(0), rows, vocab, k, _lib.ptr(out_lp),
                                                _lib.ptr(out_ix), _lib.stream()), "b200_topk_logprob")
    return out_lp, out_ix


def logprob_full(logits: torch.Tensor, vocab: int) -> torch.Tensor:
    """fp16 log_softmax(logits[:, :vocab]) (full-distribution storage)."""
    rows = logits.shape[0]
    if not logits.is_cuda:
        return torch.log_softmax(logits[:, :vocab].float(), dim=-1).to(torch.float16)
    out = torch.empty((rows, vocab), dtype=torch.float16, device=logits.device)
    _lib.check(_lib.kernels().b200_logprob_full(_lib.ptr(logits), logits.stride(0), rows, vocab, _lib.ptr(out),
                                                out.stride(0), _lib.stream()), "b200_logprob_full")
    return out


def topk_merge(a_lp: torch.Tensor, a_id: torch.Tensor, b_lp: torch.Tensor, b_id: torch.Tensor):
    """Union of two top-K lists per row with probabilities of equal ids summed; best K; (fp32 log, int32 id)."""
    rows, K = a_lp.shape
    if not a_lp.is_cuda:
        ids = torch.cat([a_id, b_id], 1).long()
        p = torch.cat([a_lp, b_lp], 1).float().exp()
        o_lp = torch.empty((rows, K)); o_id = torch.empty((rows, K), dtype=torch.int32)
        for r in range(rows):
            u, inv = torch.unique(ids[r], return_inverse=True)
            acc = torch.zeros(len(u)).index_add_(0, inv, p[r])
            v, j = torch.sort(acc, descending=True, stable=True)
            o_lp[r] = v[:K].log(); o_id[r] = u[j[:K]].to(torch.int32)
        return o_lp, o_id
    o_lp = torch.empty((rows, K), dtype=torch.float32, device=a_lp.device)
    o_id = torch.empty((rows, K), dtype=torch.int32, device=a_lp.device)
    _lib.check(_lib.kernels().b200_topk_merge(_lib.ptr(a_lp.float().contiguous()), _lib.ptr(a_id.int().contiguous()),
                                              _lib.ptr(b_lp.float().contiguous()), _lib.ptr(b_id.int().contiguous()), rows, K,
                                              _lib.ptr(o_lp), _lib.ptr(o_id), _lib.stream()), "b200_topk_merge")
    return o_lp, o_id


def remap_topk(lp: torch.Tensor, ids: torch.Tensor, table: torch.Tensor, k_out: int):
    """Send top-K rows through a teacher-id -> student-id table (-1 = no image), sum probabilities that meet on one
    student id, keep the best ``k_out``. Returns (fp32 log-prob [rows, k_out], int32 id); empty slots are -inf / 0."""
    rows, K = lp.shape
    if not lp.is_cuda:
        o_lp = torch.full((rows, k_out), float("-inf"))
        o_id = torch.zeros((rows, k_out), dtype=torch.int32)
        tab = table.long()
        for r in range(rows):
            sid = tab[ids[r].long().clamp(0, len(tab) - 1)]
            ok = (sid >= 0) & torch.isfinite(lp[r]) & (ids[r] >= 0) & (ids[r] < len(tab))
            if not ok.any():
                continue
            u, inv = torch.unique(sid[ok], return_inverse=True)
            acc = torch.zeros(len(u)).index_add_(0, inv, lp[r][ok].float().exp())
            v, j = torch.sort(acc, descending=True, stable=True)
            n = min(k_out, len(u))
            o_lp[r, :n] = v[:n].log()
            o_id[r, :n] = u[j[:n]].to(torch.int32)
        return o_lp, o_id
    o_lp = torch.empty((rows, k_out), dtype=torch.float32, device=lp.device)
    o_id = torch.empty((rows, k_out), dtype=torch.int32, device=lp.device)
    _lib.check(_lib.kernels().b200_remap_topk(_lib.ptr(lp.float().contiguous()), _lib.ptr(ids.int().contiguous()),
                                              _lib.ptr(table.int().contiguous()), table.numel(), rows, K, k_out,
                                              _lib.ptr(o_lp), _lib.ptr(o_id), _lib.stream()), "b200_remap_topk")
    return o_lp, o_id
