"""DistillEngine on CPU (fp32): loss goes down for every loss kind and optimizer family; schedules; flat buffers."""
import math

import pytest
import torch

from llm_distillery_b200.engine.optim import FlatOptimizer, FlatParams
from llm_distillery_b200.engine.schedule import LRSchedule
from llm_distillery_b200.engine.trainer import DistillEngine, synthetic_batch
from llm_distillery_b200.models.llama import LlamaConfig, build_model


def _model():
    cfg = LlamaConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=32)
    return build_model(cfg, dtype=torch.float32, seed=0)


@pytest.mark.parametrize("kind", ["kl", "rkl", "jsd", "reference"])
def test_loss_decreases(kind):
    m = _model()
    eng = DistillEngine(m, loss=kind, temperature=2.0 if kind == "kl" else 1.0, optimizer="adamw", lr=3e-3, grad_accum=2)
    hbs = [synthetic_batch(128, 2, 16, 8, seed=s, reference_fields=True) for s in (1, 2)]
    losses = [eng.train_step(hbs).item() for _ in range(12)]
    assert all(math.isfinite(x) for x in losses)
    assert losses[-1] < losses[0]


@pytest.mark.parametrize("name", ["adam", "adamw8bit", "paged_adamw32bit", "sgd", "rmsprop", "adagrad"])
def test_optimizer_names_step(name):
    m = _model()
    eng = DistillEngine(m, loss="kl", optimizer=name, lr=1e-2 if name in ("sgd", "adagrad") else 1e-3)
    hb = synthetic_batch(128, 2, 16, 8, seed=3)
    l0 = eng.train_step([hb]).item()
    for _ in range(8):
        l1 = eng.train_step([hb]).item()
    assert l1 < l0


def test_flat_params_alias_model_and_match_torch_adamw():
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(10, 7))
    b = torch.nn.Parameter(torch.randn(5))
    w2, b2 = torch.nn.Parameter(w.detach().clone()), torch.nn.Parameter(b.detach().clone())
    flat = FlatParams([w, b])
    opt = FlatOptimizer(flat, "adamw", lr=1e-2, betas=(0.9, 0.99), weight_decay=0.1)
    ref = torch.optim.AdamW([w2, b2], lr=1e-2, betas=(0.9, 0.99), weight_decay=0.1, eps=1e-8)
    for step in range(5):
        gw, gb = torch.randn(10, 7), torch.randn(5)
        w.grad_slot.buf.copy_(gw); b.grad_slot.buf.copy_(gb)
        w2.grad, b2.grad = gw.clone(), gb.clone()
        opt.step()
        ref.step()
    assert torch.allclose(w.data, w2.data, atol=1e-6) and torch.allclose(b.data, b2.data, atol=1e-6)
    assert w.data.data_ptr() == flat.model.data_ptr()


def test_wsd_shape():
    """Warmup-stable-decay (reference: utils/finetuning_utils.py:16-43; that class no longer constructs on this
    torch - LRScheduler lost its ``verbose`` argument - so the expected values are written out)."""
    mine = LRSchedule("wsd", 1e-3, 50, 7, 0.8, 5e-7)
    assert mine.lr_at(0) == pytest.approx(0.0, abs=1e-12)
    assert mine.lr_at(3) == pytest.approx(1e-3 * 0.5 * (1 + math.cos(math.pi + 3 / 7 * math.pi)))
    for s in range(7, 41):
        assert mine.lr_at(s) == pytest.approx(1e-3)
    assert mine.lr_at(45) == pytest.approx(1e-3 * (1 - 0.5 * (1 - 5e-7 / 1e-3)))
    assert mine.lr_at(50) == pytest.approx(5e-7) and mine.lr_at(1000) == pytest.approx(5e-7)
    lrs = [mine.lr] + [mine.step() for _ in range(5)]
    assert lrs == [mine.lr_at(i) for i in range(6)]


@pytest.mark.parametrize("name", ["cosine", "linear", "constant", "constant_with_warmup"])
def test_hf_named_schedules(name):
    from transformers import get_scheduler
    p = torch.nn.Parameter(torch.zeros(1))
    o = torch.optim.SGD([p], lr=2e-3)
    hs = get_scheduler(name, o, num_warmup_steps=5, num_training_steps=40)
    mine = LRSchedule(name, 2e-3, 40, 5)
    for _ in range(40):
        assert abs(o.param_groups[0]["lr"] - mine.lr) < 1e-9, name
        o.step(); hs.step(); mine.step()
