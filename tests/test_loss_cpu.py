"""Loss math: parity with the reference's calculate_divergence, closed-form properties, gradients."""
import math

import pytest
import torch

from llm_distillery_b200.loss import divergence as dv
from llm_distillery_b200.loss import head
from tests.ref_import import import_reference


def _case(n=37, V=300, K=20, seed=0, n_ranges=2):
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(n, V, generator=g) * 2
    tl = torch.randn(n, V, generator=g) * 2
    u, idx = torch.log_softmax(tl, -1).topk(K, dim=-1)
    labels = torch.randint(0, V, (n - 1,), generator=g)
    labels[::2] = idx[: n - 1: 2, 3]          # half of the labels are inside the teacher's top-K
    avoid = torch.tensor([n // 2 - 1]) if n_ranges > 1 else torch.zeros(0, dtype=torch.long)
    return z, u, idx, labels, avoid


@pytest.mark.parametrize("T,alpha,n_ranges", [(1.0, 2.0, 2), (2.0, 1.0, 1), (1.5, 3.0, 2)])
def test_reference_loss_matches_reference_implementation(T, alpha, n_ranges):
    ref = import_reference("utils.finetuning_utils")
    z, u, idx, labels, avoid = _case(n_ranges=n_ranges)
    zr = z.clone().requires_grad_()
    exp = ref.calculate_divergence(zr / T, u / T, idx, labels, alpha, avoid)
    exp["train_loss"].backward()
    zm = z.clone().requires_grad_()
    got = dv.calculate_divergence(zm / T, u / T, idx, labels, alpha, avoid)
    got["train_loss"].backward()
    for k in dv.LOSS_KEYS + ("train_loss",):
        assert torch.allclose(got[k], exp[k], atol=1e-5, rtol=1e-4), k
    assert torch.allclose(zm.grad, zr.grad, atol=1e-6, rtol=1e-3)


def test_segmented_batch_equals_per_conversation():
    ref = import_reference("utils.finetuning_utils")
    convs = [_case(n=21, seed=1), _case(n=33, seed=2, n_ranges=1), _case(n=9, seed=3)]
    total = 0.0
    S, Tt, I, Lb, Av, Sg = [], [], [], [], [], []
    for ci, (z, u, idx, labels, avoid) in enumerate(convs):
        total = total + ref.calculate_divergence(z, u, idx, labels, 2.0, avoid)["train_loss"]
        lse = torch.logsumexp(z, -1)
        s, t = dv.student_teacher_logprobs(lse, torch.gather(z, 1, idx), u, None, 1.0)
        S.append(s); Tt.append(t); I.append(idx)
        Lb.append(torch.cat([labels, torch.tensor([-1])]))
        a = torch.zeros(z.shape[0], dtype=torch.bool); a[avoid] = True
        Av.append(a); Sg.append(torch.full((z.shape[0],), ci))
    custom, logs = dv.reference_loss_segments(torch.cat(S), torch.cat(Tt), torch.cat(I), torch.cat(Lb), torch.cat(Av),
                                              torch.cat(Sg), 3, 2.0)
    assert torch.allclose(custom.sum(), total, atol=1e-5, rtol=1e-5)


def test_simple_losses_properties():
    z, u, idx, _, _ = _case(n=50, V=400, K=400)      # K = V: the support is the whole vocabulary
    lse = torch.logsumexp(z, -1)
    s, t = dv.student_teacher_logprobs(lse, torch.gather(z, 1, idx), u, None, 1.0)
    kl = dv.loss_rows("kl", s, t)
    full_kl = torch.nn.functional.kl_div(torch.log_softmax(z, -1), torch.gather(u, 1, idx.argsort(-1)), log_target=True,
                                         reduction="none").sum(-1)
    assert torch.allclose(kl, full_kl, atol=1e-5)
    assert (kl >= -1e-6).all() and (dv.loss_rows("rkl", s, t) >= -1e-6).all()
    jsd = dv.loss_rows("jsd", s, t)
    assert (jsd >= -1e-6).all() and (jsd <= math.log(2) + 1e-6).all()
    assert torch.allclose(dv.loss_rows("kl", t, t), torch.zeros(50), atol=1e-6)


@pytest.mark.parametrize("kind", ["kl", "rkl", "jsd", "reference"])
def test_head_cpu_path_gradients_match_full_logits(kind):
    torch.manual_seed(3)
    M, h, V, K, Vc = 40, 32, 120, 10, 100
    Hc = torch.randn(M, h, requires_grad=True)
    W = (torch.randn(V, h) * 0.3).requires_grad_()
    tl = torch.randn(M, V)
    u, ids = torch.log_softmax(tl, -1).topk(K, -1)
    ids32, us = head.sort_teacher_rows(ids, u)
    seg = torch.cat([torch.zeros(25, dtype=torch.long), torch.ones(15, dtype=torch.long)])
    labels = torch.randint(0, Vc, (M,)); labels[24] = -1; labels[39] = -1
    labels[::3] = ids32[::3, 2].long()
    avoid = torch.zeros(M, dtype=torch.bool); avoid[10] = True
    loss, logs = head.distill_head_loss(Hc, W, ids32, us, kind=kind, temperature=2.0, vocab=Vc, alpha=2.0, labels=labels,
                                        avoid=avoid, seg=seg, n_seg=2)
    loss.backward()
    assert torch.isfinite(loss) and Hc.grad.abs().sum() > 0
    assert W.grad[Vc:].abs().sum() == 0   # cropped vocabulary rows get no gradient
