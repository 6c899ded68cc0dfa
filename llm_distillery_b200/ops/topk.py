"""Top-K log-prob extraction and multi-teacher top-K merge (csrc/loss/topk_logprob.cu) with PyTorch restatements."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import _VP, _I, _LL

_lib.register("b200_topk_logprob", [_VP, _LL, _I, _I, _I, _VP, _VP, _VP])
_lib.register("b200_topk_merge", [_VP, _VP, _VP, _VP, _I, _I, _VP, _VP, _VP])
_lib.register("b200_remap_topk", [_VP, _VP, _VP, _I, _I, _I, _I, _VP, _VP, _VP])
_lib.register("b200_trie_walk", [_VP, _VP, _VP, _VP, _I, _VP, _VP, _I, _VP, _VP, _VP])
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
        o_lp = torch.full((rows, K), float("-inf")); o_id = torch.zeros((rows, K), dtype=torch.int32)
        for r in range(rows):
            ok = p[r] > 0                    # empty slots (id 0, log-prob -inf) take no part and come out as such
            u, inv = torch.unique(ids[r][ok], return_inverse=True)
            acc = torch.zeros(len(u)).index_add_(0, inv, p[r][ok])
            v, j = torch.sort(acc, descending=True, stable=True)
            n = min(K, len(u))
            o_lp[r, :n] = v[:n].log(); o_id[r, :n] = u[j[:n]].to(torch.int32)
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


def trie_walk(flat: dict, token_bytes: list[bytes], device):
    """Longest-prefix lookup of every byte string in ``token_bytes`` in a flattened byte trie
    (``align.aligner.ByteTrie.flatten``). Returns (int32 id per string, -1 = no prefix is stored; int32 number of bytes
    the found prefix covers). CUDA devices run one thread per string (kernel ``trie_walk``); the CPU path walks the
    same arrays in Python."""
    import numpy as np
    lens = np.fromiter((len(b) for b in token_bytes), dtype=np.int64, count=len(token_bytes))
    off = np.zeros(len(token_bytes) + 1, dtype=np.int64)
    np.cumsum(lens, out=off[1:])
    blob = np.frombuffer(b"".join(token_bytes) or b"\0", dtype=np.uint8)
    dev = torch.device(device)
    if dev.type != "cuda":
        es, eb, ec, nv = flat["edge_start"], flat["edge_byte"], flat["edge_child"], flat["node_value"]
        out = np.full(len(token_bytes), -1, dtype=np.int32)
        out_len = np.zeros(len(token_bytes), dtype=np.int32)
        for t in range(len(token_bytes)):
            node = 0
            for i in range(int(off[t]), int(off[t + 1])):
                a, e = int(es[node]), int(es[node + 1])
                j = a + int(np.searchsorted(eb[a:e], blob[i]))
                if j >= e or eb[j] != blob[i]:
                    break
                node = int(ec[j])
                if nv[node] >= 0:
                    out[t], out_len[t] = nv[node], i - int(off[t]) + 1
        return torch.from_numpy(out), torch.from_numpy(out_len)
    g = {k: torch.from_numpy(np.ascontiguousarray(v)).to(dev) for k, v in flat.items()}
    tb, to = torch.from_numpy(blob.copy()).to(dev), torch.from_numpy(off).to(dev)
    out = torch.empty(len(token_bytes), dtype=torch.int32, device=dev)
    out_len = torch.empty(len(token_bytes), dtype=torch.int32, device=dev)
    _lib.check(_lib.kernels().b200_trie_walk(_lib.ptr(g["edge_start"]), _lib.ptr(g["edge_byte"]), _lib.ptr(g["edge_child"]),
                                             _lib.ptr(g["node_value"]), g["node_value"].numel(), _lib.ptr(tb), _lib.ptr(to),
                                             len(token_bytes), _lib.ptr(out), _lib.ptr(out_len), _lib.stream()),
               "b200_trie_walk")
    return out, out_len
