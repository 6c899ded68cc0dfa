"""Frozen low-bit base weights (``training_precision`` 4bit / 8bit): quantisation oracles on CPU, the frozen-layer
mechanics of the model, and (on a GPU) the dequantisation kernels against the PyTorch restatement."""
import pytest
import torch

from llm_distillery_b200.engine.trainer import DistillEngine, synthetic_batch
from llm_distillery_b200.models.llama import LlamaConfig, build_model
from llm_distillery_b200.ops import quant


def _cfg():
    return LlamaConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=3,
                       num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)


def test_nf4_round_trip_picks_the_nearest_code_of_each_block():
    torch.manual_seed(0)
    w = torch.randn(96, 128) * 0.05
    q = quant.quantize_nf4(w)
    assert q["packed"].numel() == w.numel() // 2 and q["absmax_code"].numel() == w.numel() // 64
    back = quant.dequantize_reference(q)
    blocks = w.reshape(-1, 64)
    absmax = blocks.abs().amax(1)
    # the stored block maximum is within the second-level quantisation step of the true one
    stored = q["absmax_code"].float() * q["absmax_scale"].repeat_interleave(256)[: absmax.numel()] + q["offset"]
    assert torch.all((stored - absmax).abs() <= q["absmax_scale"].max() * 0.5 + 1e-7)
    # every value lands on the code nearest to it (oracle: brute-force search over the 16 codes)
    nearest = quant.NF4[(blocks[:, :, None] / absmax[:, None, None] - quant.NF4[None, None, :]).abs().argmin(-1)]
    assert torch.allclose(back.reshape(-1, 64), nearest * stored[:, None], atol=1e-7)
    assert (back - w).abs().max() <= 0.17 * absmax.max()       # the widest gap between neighbouring codes is 0.30


def test_int8_round_trip_is_within_half_a_step_per_row():
    torch.manual_seed(1)
    w = torch.randn(40, 64) * torch.rand(40, 1)
    q = quant.quantize_int8(w)
    back = quant.dequantize_reference(q)
    assert torch.all((back - w).abs() <= q["row_scale"][:, None] * 0.5 + 1e-7)


@pytest.mark.parametrize("kind", ["nf4", "int8"])
def test_frozen_quantised_layers_compute_with_the_dequantised_weights_and_do_not_train(kind):
    cfg = _cfg()
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=3)
    ref = build_model(cfg, dtype=torch.float32, device="cpu", seed=3)
    model.quantize_frozen_linears(kind)
    quantize = quant.quantize_nf4 if kind == "nf4" else quant.quantize_int8
    with torch.no_grad():
        for layer in ref.layers:
            for name in quant.LINEARS:
                p = getattr(layer, name)
                p.copy_(quant.dequantize_reference(quantize(p.data)))
    ids = torch.randint(0, cfg.vocab_size, (2, 32))
    with torch.no_grad():
        assert torch.equal(model.hidden_states(ids), ref.hidden_states(ids))
    trainable = {n for n, p in model.named_parameters() if p.requires_grad}
    assert trainable == {"embed_tokens", "norm", "lm_head"} | {f"layers.{i}.{n}" for i in range(3)
                                                                for n in ("input_layernorm", "post_attention_layernorm")}
    eng = DistillEngine(model, loss="kl", temperature=1.0, optimizer="adamw", lr=1e-2)
    before = {n: t.clone() for n, t in model.to_hf_state_dict().items()}
    hb = synthetic_batch(cfg.vocab_size, 2, 32, 8, seed=5)
    l0 = float(eng.train_step([hb]))
    l1 = float(eng.train_step([hb]))
    assert l1 < l0
    after = model.to_hf_state_dict()
    moved = {n for n in before if not torch.equal(before[n], after[n])}
    assert moved and all(("proj" not in n) for n in moved), moved       # no decoder matrix changed
    assert torch.equal(after["model.layers.1.mlp.down_proj.weight"], ref.layers[1].down_proj.data)
    # gradient checkpointing re-reads the weights in backward: the rotating buffers must hold the right layer again
    model.grad_checkpointing = True
    l2 = float(eng.train_step([hb]))
    assert l2 < l1


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["nf4", "int8"])
def test_dequant_kernels_match_the_restatement_and_training_runs(kind):
    torch.manual_seed(2)
    w = (torch.randn(1024, 512, device="cuda") * 0.03).bfloat16()
    q = (quant.quantize_nf4 if kind == "nf4" else quant.quantize_int8)(w)
    out = torch.empty_like(w)
    quant.dequantize_into(q, out)
    assert torch.equal(out, quant.dequantize_reference(q, torch.bfloat16))
    cfg = LlamaConfig(vocab_size=2048, hidden_size=512, intermediate_size=1408, num_hidden_layers=3,
                      num_attention_heads=8, num_key_value_heads=2, max_position_embeddings=512)
    model = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=3).quantize_frozen_linears(kind)
    eng = DistillEngine(model, loss="kl", temperature=2.0, optimizer="adamw", lr=1e-3)
    hb = synthetic_batch(cfg.vocab_size, 2, 256, 32, seed=1)
    losses = [float(eng.train_step([hb])) for _ in range(3)]
    assert losses[2] < losses[0]
    from llm_distillery_b200.ops import _lib
    assert _lib.take_device_error() == 0
