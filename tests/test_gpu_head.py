"""Fused LM head + distillation loss kernels against the full-logits PyTorch computation."""
import pytest
import torch

from llm_distillery_b200.loss import head, divergence as dv
from llm_distillery_b200.models.llama import GradSlot
from llm_distillery_b200.ops import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _setup(M, h, V, K, seed=0):
    torch.manual_seed(seed)
    Hc = torch.randn(M, h, device=DEV).bfloat16()
    W = (torch.randn(V, h, device=DEV) * 0.05).bfloat16()
    tl = torch.randn(M, V, device=DEV) * 3
    u, ids = torch.log_softmax(tl, -1).topk(K, -1)
    ids32, us = head.sort_teacher_rows(ids, u.half().float())
    return Hc, W, ids32, us


@pytest.mark.parametrize("M,h,V,K,Vc,T", [(128, 64, 256, 8, 256, 1.0), (300, 256, 1000, 50, 1000, 2.0),
                                           (517, 512, 5000, 200, 4800, 1.0), (2048, 2048, 32000, 200, 32000, 2.0)])
def test_stats_forward(M, h, V, K, Vc, T):
    Hc, W, ids, u = _setup(M, h, V, K)
    lse, zk = head.lmhead_stats(Hc, W, ids, T, Vc)
    assert _lib.take_device_error() == 0
    rl, rz = head._torch_stats(Hc, W, ids, 1.0 / T, Vc)
    assert torch.allclose(lse, rl, atol=2e-3, rtol=1e-4), (lse - rl).abs().max()
    assert torch.allclose(zk, rz, atol=2e-3, rtol=1e-3), (zk - rz).abs().max()


@pytest.mark.parametrize("kind", ["kl", "rkl", "jsd", "jsd_renorm"])
@pytest.mark.parametrize("M,h,V,K,Vc,T", [(300, 256, 1000, 50, 1000, 2.0), (517, 512, 5000, 200, 4800, 1.0)])
def test_fused_loss_and_gradients(kind, M, h, V, K, Vc, T):
    Hc, W, ids, u = _setup(M, h, V, K, seed=1)
    Hr = Hc.float().requires_grad_()
    Wr = W.float().requires_grad_()
    lse, zk = head._torch_stats(Hr, Wr, ids, 1.0 / T, Vc)
    s, t = dv.student_teacher_logprobs(lse, zk, u, ids.long() < Vc, T)
    ref_rows = dv.loss_rows("jsd", s, t, jsd_renorm=True) if kind == "jsd_renorm" else dv.loss_rows(kind, s, t)
    w = torch.rand(M, device=DEV) / M
    (ref_rows * w).sum().backward()

    Hg = Hc.clone().requires_grad_()
    Wg = W.clone().requires_grad_()
    Wg.grad_slot = GradSlot(torch.zeros(V, h, device=DEV))
    rows = head.fused_distill_rows(Hg, Wg, ids, u, "jsd" if kind == "jsd_renorm" else kind, T, Vc,
                                   jsd_renorm=(kind == "jsd_renorm"))
    (rows * w).sum().backward()
    assert _lib.take_device_error() == 0
    assert torch.allclose(rows, ref_rows.detach(), atol=3e-3, rtol=3e-3), (rows - ref_rows).abs().max()
    gH, gW = Hg.grad.float(), Wg.grad_slot.buf
    assert (gH - Hr.grad).abs().max() <= 2e-2 * Hr.grad.abs().max() + 1e-6
    assert (gW - Wr.grad).abs().max() <= 2e-2 * Wr.grad.abs().max() + 1e-6
    assert gW[Vc:].abs().max() == 0 if Vc < V else True


def test_reference_loss_through_fused_stats():
    M, h, V, K, Vc, T = 400, 256, 2000, 64, 2000, 1.0
    Hc, W, ids, u = _setup(M, h, V, K, seed=2)
    seg = torch.cat([torch.zeros(250, dtype=torch.long), torch.ones(150, dtype=torch.long)]).to(DEV)
    labels = torch.randint(0, V, (M,), device=DEV)
    labels[::2] = ids[::2, 5].long()
    labels[249] = -1
    labels[399] = -1
    avoid = torch.zeros(M, dtype=torch.bool, device=DEV)
    avoid[100] = True
    kw = dict(kind="reference", temperature=T, vocab=Vc, alpha=2.0, labels=labels, avoid=avoid, seg=seg, n_seg=2)
    Hr, Wr = Hc.float().cpu().requires_grad_(), W.float().cpu().requires_grad_()
    ref, _ = head.distill_head_loss(Hr, Wr, ids.cpu(), u.cpu(), **{**kw, "labels": labels.cpu(), "avoid": avoid.cpu(),
                                                                   "seg": seg.cpu()})
    ref.backward()
    Hg, Wg = Hc.clone().requires_grad_(), W.clone().requires_grad_()
    got, logs = head.distill_head_loss(Hg, Wg, ids, u, **kw)
    got.backward()
    assert _lib.take_device_error() == 0
    assert abs(got.item() - ref.item()) <= 2e-2 * abs(ref.item()) + 1e-3
    assert (Hg.grad.float().cpu() - Hr.grad).abs().max() <= 5e-2 * Hr.grad.abs().max()
    assert (Wg.grad.float().cpu() - Wr.grad).abs().max() <= 5e-2 * Wr.grad.abs().max()
    assert set(dv.LOSS_KEYS) <= set(logs)
