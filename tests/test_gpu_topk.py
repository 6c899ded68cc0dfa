"""Exact top-K log-prob extraction, full log-prob rows, multi-teacher merge, collector, optimizer kernels on GPU."""
import numpy as np
import pytest
import torch

from llm_distillery_b200.collect.collector import TeacherCollector
from llm_distillery_b200.data.convo import ConvoTokenized
from llm_distillery_b200.engine.optim import FlatOptimizer, FlatParams
from llm_distillery_b200.models.llama import LlamaConfig, build_model
from llm_distillery_b200.ops import _lib, topk

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("rows,V,Vc,K", [(7, 1000, 1000, 10), (64, 32000, 32000, 200), (33, 5000, 4096, 400),
                                          (5, 300, 300, 300), (16, 128256, 128256, 128)])
def test_topk_logprob_exact(rows, V, Vc, K):
    torch.manual_seed(rows + K)
    x = torch.randn(rows, V, device=DEV) * 4
    x[:, ::7] = x[:, 1::7][:, : x[:, ::7].shape[1]]      # plenty of exact ties
    lp, ix = topk.topk_logprob(x, Vc, K)
    assert _lib.take_device_error() == 0
    ref_lp, ref_ix = topk.topk_logprob(x.cpu(), Vc, K)
    assert torch.equal(ix.cpu(), ref_ix)                  # ties broken by lower index, like a stable sort
    assert torch.allclose(lp.float().cpu(), ref_lp.float(), atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("case", ["one bin", "masked", "all equal", "few distinct"])
def test_topk_logprob_rows_that_defeat_the_histogram(case):
    """Rows whose K-th element shares its 11-bit histogram bin with thousands of others (the candidates no longer fit
    shared memory and the kernel narrows the threshold over the row instead), rows with masked (-inf) entries, and
    rows with more equal values at the threshold than the tie list holds."""
    torch.manual_seed(5)
    rows, V, K = 9, 20000, 200
    if case == "one bin":
        x = 1.0 + 0.1 * torch.rand(rows, V, device=DEV)            # every value in [1.0, 1.1): one bin
    elif case == "masked":
        x = torch.randn(rows, V, device=DEV) * 3
        x[:, 5000:] = float("-inf")
        x[3, 150:] = float("-inf")                                  # fewer finite values than K
    elif case == "all equal":
        x = torch.full((rows, V), 0.25, device=DEV)
        x[1, 17] = 3.0
    else:
        x = torch.randint(0, 3, (rows, V), device=DEV).float()      # ~6700 ties at the threshold
    lp, ix = topk.topk_logprob(x, V, K)
    assert _lib.take_device_error() == 0
    ref_lp, ref_ix = topk.topk_logprob(x.cpu(), V, K)
    assert torch.equal(ix.cpu(), ref_ix)
    got, want = lp.float().cpu(), ref_lp.float()
    finite = torch.isfinite(want)
    assert torch.equal(torch.isfinite(got), finite)
    assert torch.allclose(got[finite], want[finite], atol=2e-3, rtol=1e-3)


def test_logprob_full_and_merge():
    torch.manual_seed(0)
    x = torch.randn(50, 777, device=DEV) * 3
    full = topk.logprob_full(x, 700)
    assert torch.allclose(full.float().cpu(), torch.log_softmax(x[:, :700].cpu(), -1), atol=3e-3, rtol=2e-3)
    K = 40
    a = torch.log_softmax(torch.randn(60, 500, device=DEV) * 3, -1)
    b = torch.log_softmax(torch.randn(60, 500, device=DEV) * 3, -1)
    av, ai = a.topk(K, -1)
    bv, bi = b.topk(K, -1)
    lp, ids = topk.topk_merge(av, ai.int(), bv, bi.int())
    rlp, rids = topk.topk_merge(av.cpu(), ai.int().cpu(), bv.cpu(), bi.int().cpu())
    assert torch.allclose(lp.cpu(), rlp, atol=1e-4, rtol=1e-4)
    same = (ids.cpu() == rids).float().mean().item()
    assert same > 0.99          # order may differ only between exactly equal probabilities


def test_merge_keeps_the_mass_of_token_zero_beside_empty_slots():
    """Empty slots are (id 0, -inf); a real token 0 in both lists must come out with both probabilities."""
    ninf = float("-inf")
    a_lp = torch.tensor([[0.5, 0.2, 0.0, 0.0, 0.0, 0.0]], device=DEV).log()
    a_id = torch.tensor([[0, 7, 0, 0, 0, 0]], device=DEV, dtype=torch.int32)
    b_lp = torch.tensor([[0.3, 0.25, 0.1, 0.0, 0.0, 0.0]], device=DEV).log()
    b_id = torch.tensor([[0, 9, 7, 0, 0, 0]], device=DEV, dtype=torch.int32)
    lp, ids = topk.topk_merge(a_lp, a_id, b_lp, b_id)
    assert ids[0, :3].tolist() == [0, 7, 9]
    assert torch.allclose(lp[0, :3].exp().cpu(), torch.tensor([0.8, 0.3, 0.25]), atol=1e-5)
    assert ids[0, 3:].tolist() == [0, 0, 0] and bool((lp[0, 3:] == ninf).all())
    rlp, rids = topk.topk_merge(a_lp.cpu(), a_id.cpu(), b_lp.cpu(), b_id.cpu())
    assert rids[0, :3].tolist() == [0, 7, 9] and torch.allclose(rlp[0, :3].exp(), torch.tensor([0.8, 0.3, 0.25]), atol=1e-5)


def test_collector_matches_full_logits_path():
    torch.manual_seed(1)
    cfg = LlamaConfig(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256)
    model = build_model(cfg, dtype=torch.bfloat16, device=DEV, seed=3)
    rng = np.random.default_rng(0)
    convos, toks = [], []
    for i, (length, ranges) in enumerate([(100, [(2, 40), (50, 100)]), (77, [(0, 77)]), (128, [(10, 20)])]):
        t = np.zeros(128, dtype=np.int64)
        t[:length] = rng.integers(0, 2000, length)
        convos.append(ConvoTokenized(t, ranges, 128 - length, False, i))
        toks.append(t)
    tokens = np.stack(toks)
    col = TeacherCollector(model, topk=32, crop_to_size=2000, enable_topk=True)
    rows = col.collect_batch(tokens, convos)
    assert _lib.take_device_error() == 0
    with torch.no_grad():   # oracle: fp32 logits from the same bf16 hidden states and weights
        hs = model.hidden_states(torch.from_numpy(tokens).to(DEV)).float()
        logits = (hs @ model.lm_head.float().t()).reshape(3, 128, -1)[:, :, :2000]
    lp = torch.log_softmax(logits, -1).cpu()
    for r, c in zip(rows, convos):
        ci = c.content_indices()
        ci = ci[ci < c.length]
        assert r.values.shape == (len(ci), 32) and r.indices.shape == (len(ci), 32)
        ref_v, ref_i = lp[c.origin_convo_id, ci].topk(32, -1)
        agree = (torch.from_numpy(r.indices) == ref_i).float().mean().item()
        assert agree > 0.97     # only exact-tie order may differ
        assert torch.allclose(torch.from_numpy(r.values).float()[:, :4], ref_v[:, :4], atol=3e-2, rtol=2e-2)
    full = TeacherCollector(model, topk=0, crop_to_size=2000, enable_topk=False).collect_batch(tokens, convos)
    assert full[1].indices is None and full[1].values.shape == (77, 2000)


@pytest.mark.parametrize("name", ["adamw", "adam", "adamw8bit", "sgd", "rmsprop", "adagrad"])
def test_optimizer_kernels_match_torch_restatement(name):
    torch.manual_seed(2)
    w = torch.nn.Parameter(torch.randn(300, 70, device=DEV).bfloat16())
    w_cpu = torch.nn.Parameter(w.detach().float().cpu())
    fg = FlatParams([w])
    fc = FlatParams([w_cpu])
    fc.master.copy_(fg.master.cpu())
    og = FlatOptimizer(fg, name, lr=1e-2, weight_decay=0.01)
    oc = FlatOptimizer(fc, name, lr=1e-2, weight_decay=0.01)
    for _ in range(4):
        g = torch.randn(300, 70)
        w.grad_slot.buf.copy_(g.to(DEV))
        w_cpu.grad_slot.buf.copy_(g)
        og.step(grad_scale=0.5)
        oc.step(grad_scale=0.5)
    tol = 3e-2 if name == "adamw8bit" else 1e-4
    assert torch.allclose(fg.master.cpu(), fc.master, atol=tol, rtol=tol), (fg.master.cpu() - fc.master).abs().max()
    assert torch.allclose(w.detach().float().cpu(), fg.master.cpu()[: w.numel()].view(300, 70), atol=2e-2, rtol=2e-2)
