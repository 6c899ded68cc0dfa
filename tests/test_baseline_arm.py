"""The library baseline of the benchmark (baseline/hf_baseline.py) computes the same losses as this package: forward KL,
reverse KL and JSD of a tiny model on CPU, step for step, and gradient accumulation averages as the engine does."""
import pytest
import torch

from llm_distillery_b200.engine.trainer import DistillEngine, synthetic_batch
from llm_distillery_b200.models.llama import LlamaConfig, build_model

tr = pytest.importorskip("transformers")


@pytest.mark.parametrize("loss", ["kl", "rkl", "jsd"])
def test_baseline_losses_equal_the_engine_losses(loss):
    from baseline.hf_baseline import BaselineRunner
    cfg = LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=136, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=128)
    dev = torch.device("cpu")
    runner = BaselineRunner(cfg, dev, 1, temperature=2.0, topk=8, loss=loss, grad_accum=2)
    runner.model.float()
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=0)
    model.load_hf_state_dict({k: v.detach().clone() for k, v in runner.model.state_dict().items()}, strict=False)
    eng = DistillEngine(model, loss=loss, temperature=2.0, optimizer="adamw", lr=1e-3, crop_to_size=cfg.vocab_size)
    hb = synthetic_batch(cfg.vocab_size, 2, 32, 8, seed=1)
    ours, _ = eng.micro_step(hb.to_device(dev), last=True)
    theirs = runner._micro(hb.to_device(dev), step=False)
    assert torch.allclose(torch.as_tensor(float(ours)), theirs.float(), rtol=2e-4, atol=1e-5), (float(ours), float(theirs))
