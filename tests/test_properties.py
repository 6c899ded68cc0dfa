"""Property tests (hypothesis) of the loss definitions, the multi-teacher merge and the vocabulary remap, on the
PyTorch statements that are also the oracles of the GPU kernels."""
import math

import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from llm_distillery_b200.loss import divergence as dv
from llm_distillery_b200.loss.head import fused_distill_rows, sort_teacher_rows
from llm_distillery_b200.ops import topk as tk

SETTINGS = dict(max_examples=25, deadline=None)


def _case(seed, rows, V, K, h=16):
    g = torch.Generator().manual_seed(seed)
    Hc = torch.randn((rows, h), generator=g)
    W = torch.randn((V, h), generator=g) * 0.5
    ids = torch.stack([torch.randperm(V, generator=g)[:K] for _ in range(rows)]).to(torch.int32)
    u = torch.log_softmax(torch.randn((rows, K), generator=g) * 2, -1)
    return Hc, W, ids, u


@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), kind=st.sampled_from(["kl", "rkl", "jsd"]), T=st.sampled_from([1.0, 2.0]))
def test_losses_are_non_negative_bounded_and_order_invariant(seed, kind, T):
    Hc, W, ids, u = _case(seed, rows=6, V=50, K=8)
    sid, su = sort_teacher_rows(ids, u)
    loss = fused_distill_rows(Hc, W, sid, su, kind, T, vocab=50)
    if kind == "rkl":
        assert (loss > -1e-5).all()                       # both sides are renormalised over the support
    if kind == "jsd":
        assert (loss > -1e-5).all() and (loss < math.log(2) + 1e-5).all()
    # any permutation of a row's (id, log-prob) pairs gives the same loss
    perm = torch.stack([torch.randperm(8, generator=torch.Generator().manual_seed(seed + r)) for r in range(6)])
    pid, pu = torch.gather(ids, 1, perm), torch.gather(u, 1, perm)
    sid2, su2 = sort_teacher_rows(pid, pu)
    loss2 = fused_distill_rows(Hc, W, sid2, su2, kind, T, vocab=50)
    assert torch.allclose(loss, loss2, atol=1e-6)


@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000))
def test_forward_kl_is_zero_iff_student_matches_teacher_on_the_support(seed):
    g = torch.Generator().manual_seed(seed)
    K = 6
    t = torch.log_softmax(torch.randn((4, K), generator=g), -1)
    # student whose log-probs at the ids equal the teacher's (rest of the vocabulary carries no mass: lse = logsumexp(zk))
    zk = t + 3.0
    lse = torch.logsumexp(zk, -1)
    s, tt = dv.student_teacher_logprobs(lse, zk, t, None, 1.0)
    assert dv.loss_rows("kl", s, tt).abs().max() < 1e-5
    zk2 = zk + torch.randn((4, K), generator=g)
    s2, _ = dv.student_teacher_logprobs(torch.logsumexp(zk2, -1), zk2, t, None, 1.0)
    assert (dv.loss_rows("kl", s2, tt) > -1e-6).all()


@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000), K=st.sampled_from([4, 16]))
def test_merge_conserves_mass_of_the_kept_entries_and_is_symmetric(seed, K):
    g = torch.Generator().manual_seed(seed)
    V = 40
    def topk_rows():
        lp = torch.log_softmax(torch.randn((5, V), generator=g) * 2, -1)
        v, i = torch.topk(lp, K, dim=-1)
        return v, i.to(torch.int32)
    a_lp, a_id = topk_rows()
    b_lp, b_id = topk_rows()
    o_lp, o_id = tk.topk_merge(a_lp, a_id, b_lp, b_id)
    p_lp, p_id = tk.topk_merge(b_lp, b_id, a_lp, a_id)
    assert torch.allclose(o_lp.exp().sum(-1), p_lp.exp().sum(-1), atol=1e-5)
    for r in range(5):
        union = {}
        for lp, ids in ((a_lp[r], a_id[r]), (b_lp[r], b_id[r])):
            for x, i in zip(lp.tolist(), ids.tolist()):
                union[i] = union.get(i, 0.0) + math.exp(x)
        best = sorted(union.values(), reverse=True)[:K]
        assert abs(o_lp[r].exp().sum().item() - sum(best)) < 1e-4      # exactly the K heaviest ids of the union
        assert len(set(o_id[r].tolist())) == K


@settings(**SETTINGS)
@given(seed=st.integers(0, 10_000))
def test_remap_never_creates_mass_and_conserves_it_when_every_token_has_an_image(seed):
    g = torch.Generator().manual_seed(seed)
    Vt, Vs, K = 60, 30, 8
    lp = torch.log_softmax(torch.randn((5, Vt), generator=g) * 2, -1)
    v, i = torch.topk(lp, K, dim=-1)
    full = torch.randint(0, Vs, (Vt,), generator=g, dtype=torch.int32)           # every teacher token has an image
    o_lp, o_id = tk.remap_topk(v, i.to(torch.int32), full, K)
    assert torch.allclose(o_lp.exp().sum(-1), v.exp().sum(-1), atol=1e-5)
    holes = full.clone()
    holes[torch.rand(Vt, generator=g) < 0.3] = -1
    h_lp, _ = tk.remap_topk(v, i.to(torch.int32), holes, K)
    assert (h_lp.exp().sum(-1) <= v.exp().sum(-1) + 1e-5).all()
