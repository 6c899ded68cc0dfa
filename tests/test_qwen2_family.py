"""Qwen2-style attention (bias on the q/k/v projections): the fused-QKV model equals HuggingFace's Qwen2ForCausalLM in
logits and gradients, round-trips through the HF checkpoint layout, and trains through the engine."""
import pytest
import torch

from llm_distillery_b200.ckpt.hf import load_hf_model, save_hf_model
from llm_distillery_b200.engine.trainer import DistillEngine, synthetic_batch
from llm_distillery_b200.models.llama import LlamaConfig, build_model

CFG = LlamaConfig(vocab_size=320, hidden_size=64, intermediate_size=136, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, max_position_embeddings=64, rope_theta=1e6, rms_norm_eps=1e-6,
                  attention_bias=True, model_type="qwen2", tie_word_embeddings=False)


def _hf_twin(model):
    tr = pytest.importorskip("transformers")
    hf_cfg = tr.Qwen2Config(vocab_size=CFG.vocab_size, hidden_size=CFG.hidden_size, intermediate_size=CFG.intermediate_size,
                            num_hidden_layers=CFG.num_hidden_layers, num_attention_heads=CFG.num_attention_heads,
                            num_key_value_heads=CFG.num_key_value_heads, max_position_embeddings=64, rope_theta=1e6,
                            rms_norm_eps=1e-6, tie_word_embeddings=False, use_sliding_window=False,
                            attn_implementation="eager")
    hf = tr.Qwen2ForCausalLM(hf_cfg).float()
    missing = hf.load_state_dict({k: v.clone() for k, v in model.to_hf_state_dict().items()}, strict=False)
    assert not [k for k in missing.missing_keys if "rotary" not in k], missing
    return hf


def test_logits_and_gradients_match_huggingface_qwen2():
    torch.manual_seed(0)
    model = build_model(CFG, dtype=torch.float32, device="cpu", seed=3)
    hf = _hf_twin(model)
    x = torch.randint(0, CFG.vocab_size, (2, 24))
    ours = model(x)
    ref = hf(x).logits
    assert torch.allclose(ours, ref, atol=2e-4, rtol=1e-3), (ours - ref).abs().max()
    ours.square().mean().backward()
    ref.square().mean().backward()
    b = model.layers[1].qkv_bias.grad
    q = CFG.q_size
    assert torch.allclose(b[:q], hf.model.layers[1].self_attn.q_proj.bias.grad, atol=1e-6, rtol=1e-3)
    assert torch.allclose(b[q + CFG.kv_size:], hf.model.layers[1].self_attn.v_proj.bias.grad, atol=1e-6, rtol=1e-3)
    w = model.layers[0].qkv_proj.grad
    assert torch.allclose(w[:q], hf.model.layers[0].self_attn.q_proj.weight.grad, atol=1e-6, rtol=1e-3)


def test_checkpoint_round_trip_and_config_say_qwen2(tmp_path):
    model = build_model(CFG, dtype=torch.float32, device="cpu", seed=4)
    save_hf_model(model, str(tmp_path / "m"))
    import json
    c = json.load(open(tmp_path / "m" / "config.json"))
    assert c["model_type"] == "qwen2" and c["architectures"] == ["Qwen2ForCausalLM"]
    back = load_hf_model(str(tmp_path / "m"), dtype=torch.float32)
    assert back.cfg.attention_bias and torch.equal(back.layers[1].qkv_bias, model.layers[1].qkv_bias)
    tr = pytest.importorskip("transformers")
    hf = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "m"), torch_dtype=torch.float32)
    x = torch.randint(0, CFG.vocab_size, (1, 10))
    assert torch.allclose(hf(x).logits, model(x), atol=2e-4, rtol=1e-3)


def test_engine_trains_the_bias():
    model = build_model(CFG, dtype=torch.float32, device="cpu", seed=5)
    before = model.layers[0].qkv_bias.detach().clone()
    eng = DistillEngine(model, loss="kl", temperature=1.0, optimizer="adamw", lr=1e-2)
    hb = synthetic_batch(CFG.vocab_size, 2, 32, 8, seed=1)
    l0 = float(eng.train_step([hb]))
    for _ in range(5):
        l1 = float(eng.train_step([hb]))
    assert l1 < l0 and not torch.equal(model.layers[0].qkv_bias, before)


@pytest.mark.gpu
@pytest.mark.parametrize("variant", ["qwen2", "qwen3", "llama with biases", "plain llama, long batch", "granite",
                                     "plain partial rotary, long batch", "olmo2", "glm4, long batch",
                                     "hunyuan", "gemma3, heads of 256", "mistral beyond its window"])
def test_gpu_kernels_follow_the_cpu_model(variant):
    """bf16 kernels (GEMMs with their epilogues, bias add, per-head norms, RoPE, flash attention ...) against the fp32 CPU
    statement of the same model, for the layer variants: q/k/v bias (Qwen2), per-head q/k norms (Qwen3), biases on every
    projection (Llama with attention_bias / mlp_bias), a plain layer with enough rows for the fused epilogues, Granite's
    multipliers, heads of which three quarters rotate (the fused rotary epilogues must step aside), and the general
    layer node with norms behind the branches (OLMo 2 with q/k norms over the whole projections; GLM-4)."""
    kw = dict(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, max_position_embeddings=1024, rope_theta=1e6, rms_norm_eps=1e-6)
    if variant == "qwen2":
        kw.update(attention_bias=True, model_type="qwen2")
    elif variant == "qwen3":
        kw.update(qk_norm=True, model_type="qwen3")
    elif variant == "llama with biases":
        kw.update(attention_bias=True, o_bias=True, mlp_bias=True)
    elif "partial rotary" in variant:
        kw.update(partial_rotary_factor=0.75)
    elif variant.startswith("gemma3"):        # heads of 256: PyTorch's attention and per-head norms; GeGLU; two rotary bases
        kw.update(model_type="gemma3_text", num_attention_heads=2, num_key_value_heads=1, head_dim_override=256,
                  hidden_size=256, mlp_act="gelu_tanh", norm_plus_one=True, embedding_multiplier=16.0,
                  embedding_multiplier_rounded=True, post_norm=True, qk_norm=True, sliding_window=64,
                  window_layers=[1, 0], rope_local_theta=10000.0, tie_word_embeddings=True)
    elif variant.startswith("mistral"):
        kw.update(model_type="mistral", sliding_window=48)
    elif variant == "hunyuan":
        kw.update(model_type="hunyuan_v1_dense", qk_norm=True, qk_norm_after_rope=True)
    elif variant == "olmo2":
        kw.update(model_type="olmo2", pre_norm=False, post_norm=True, qk_norm_full=True)
    elif variant.startswith("glm4"):
        kw.update(model_type="glm4", post_norm=True, attention_bias=True, partial_rotary_factor=0.5, rope_interleaved=True)
    elif variant == "granite":
        kw.update(model_type="granite", embedding_multiplier=6.0, attention_multiplier=0.09, residual_multiplier=0.3,
                  logits_scaling=4.0, attention_bias=True, o_bias=True, mlp_bias=True)
    cfg = LlamaConfig(**kw)
    cpu = build_model(cfg, dtype=torch.float32, device="cpu", seed=7)
    with torch.no_grad():
        g = torch.Generator().manual_seed(3)
        for n, p in cpu.named_parameters():
            if n.endswith("_bias"):
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
            elif n.endswith("q_norm") or n.endswith("k_norm") or n.endswith("_out_norm"):
                p.copy_(torch.empty(p.shape).uniform_(0.5, 1.5, generator=g))
    gpu = build_model(cfg, dtype=torch.bfloat16, device="cuda", seed=7)
    with torch.no_grad():
        for a, b in zip(gpu.parameters(), cpu.parameters()):
            a.copy_(b.to(torch.bfloat16))
            b.copy_(a.float().cpu())          # both sides hold the bf16-rounded weights
    x = torch.randint(0, cfg.vocab_size, (2, 640 if "long batch" in variant else 128))
    lc = cpu(x)
    lg = gpu(x.cuda())
    assert torch.allclose(lg.float().cpu(), lc, atol=6e-2, rtol=5e-2), (lg.float().cpu() - lc).abs().max()
    lc.square().mean().backward()
    lg.float().square().mean().backward()
    for (n, pg), (_, pc) in zip(gpu.named_parameters(), cpu.named_parameters()):
        gg, gc = pg.grad.float().cpu(), pc.grad
        assert torch.isfinite(gg).all(), n
        assert (gg - gc).abs().max() <= 0.06 * gc.abs().max() + 2e-4, (n, (gg - gc).abs().max(), gc.abs().max())
