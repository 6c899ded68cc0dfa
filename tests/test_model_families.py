"""Checkpoint-level compatibility beyond plain Llama: Llama 3.1 / 3.2 rope scaling, the Phi-3 family (fused projections
in the checkpoint), Mistral's attention window, and config keys that must survive a load / save round trip."""
import json

import pytest
import torch

from llm_distillery_b200.ckpt.hf import load_hf_model, load_tp_weights, save_hf_model
from llm_distillery_b200.models.llama import LlamaConfig, build_model
from llm_distillery_b200.ops import basic

tr = pytest.importorskip("transformers")

ROPE3 = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
         "original_max_position_embeddings": 64}


def _base(**kw):
    d = dict(vocab_size=320, hidden_size=64, intermediate_size=136, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, max_position_embeddings=256, rope_theta=10000.0, rms_norm_eps=1e-6)
    d.update(kw)
    return d


def test_llama3_rope_scaling_matches_huggingface():
    cfg = LlamaConfig(**_base(rope_scaling=ROPE3))
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=1)
    hf_cfg = tr.LlamaConfig(**_base(), rope_scaling=dict(ROPE3), attn_implementation="eager", tie_word_embeddings=False)
    hf = tr.LlamaForCausalLM(hf_cfg).float()
    hf.load_state_dict({k: v.clone() for k, v in model.to_hf_state_dict().items()}, strict=False)
    x = torch.randint(0, 320, (2, 200))          # beyond original_max_position_embeddings: the scaled band matters
    ours, ref = model(x), hf(x).logits
    assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (ours - ref).abs().max()
    plain = build_model(LlamaConfig(**_base()), dtype=torch.float32, device="cpu", seed=1)
    assert (plain(x) - ref).abs().max() > 2e-3    # and it is not a no-op (ten times the tolerance above)
    # linear scaling: every frequency divided by the factor
    c1, s1 = basic.rope_tables(32, 16, 10000.0, "cpu", {"type": "linear", "factor": 4.0})
    c0, s0 = basic.rope_tables(128, 16, 10000.0, "cpu")
    assert torch.allclose(c1[4::4], c0[1:8], atol=1e-6) and torch.allclose(s1[4::4], s0[1:8], atol=1e-6)
    with pytest.raises(NotImplementedError):
        basic.rope_tables(8, 16, 10000.0, "cpu", {"rope_type": "ntk-by-parts", "factor": 2.0})


def test_phi3_checkpoint_layout_matches_huggingface(tmp_path):
    cfg = LlamaConfig(**_base(model_type="phi3", pad_token_id=0, bos_token_id=1, eos_token_id=2))
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=2)
    sd = model.to_hf_state_dict()
    assert "model.layers.0.self_attn.qkv_proj.weight" in sd and "model.layers.1.mlp.gate_up_proj.weight" in sd
    assert not any("q_proj" in k or "gate_proj" in k for k in sd)
    hf_cfg = tr.Phi3Config(**_base(), pad_token_id=0, bos_token_id=1, eos_token_id=2, attn_implementation="eager",
                           tie_word_embeddings=False, sliding_window=None)
    hf = tr.Phi3ForCausalLM(hf_cfg).float()
    missing = hf.load_state_dict({k: v.clone() for k, v in sd.items()}, strict=False)
    assert not [k for k in missing.missing_keys if "rotary" not in k] and not missing.unexpected_keys, missing
    x = torch.randint(0, 320, (2, 40))
    ours, ref = model(x), hf(x).logits
    assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (ours - ref).abs().max()
    # save -> HuggingFace reads it; HuggingFace saves -> this loader reads it
    save_hf_model(model, str(tmp_path / "ours"))
    c = json.load(open(tmp_path / "ours" / "config.json"))
    assert c["model_type"] == "phi3" and c["architectures"] == ["Phi3ForCausalLM"] and c["pad_token_id"] == 0
    hf2 = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ours"), torch_dtype=torch.float32,
                                                  attn_implementation="eager")
    assert torch.allclose(hf2(x).logits, ref, atol=3e-4, rtol=1e-3)
    hf.save_pretrained(str(tmp_path / "theirs"), safe_serialization=True)
    back = load_hf_model(str(tmp_path / "theirs"), dtype=torch.float32)
    assert back.cfg.model_type == "phi3"
    assert torch.allclose(back(x), ref, atol=3e-4, rtol=1e-3)
    # tensor-parallel slices come out of the fused tensors
    _, w0 = load_tp_weights(str(tmp_path / "theirs"), 0, 2, dtype=torch.float32)
    _, w1 = load_tp_weights(str(tmp_path / "theirs"), 1, 2, dtype=torch.float32)
    q, kv, f = cfg.q_size, cfg.kv_size, cfg.intermediate_size
    full = back.layers[0].qkv_proj.data
    want0 = torch.cat([full[: q // 2], full[q: q + kv // 2], full[q + kv: q + kv + kv // 2]])
    want1 = torch.cat([full[q // 2: q], full[q + kv // 2: q + kv], full[q + kv + kv // 2:]])
    assert torch.equal(w0["layers.0.qkv_proj"], want0) and torch.equal(w1["layers.0.qkv_proj"], want1)
    gu = back.layers[1].gate_up_proj.data
    assert torch.equal(w1["layers.1.gate_up_proj"], torch.cat([gu[f // 2: f], gu[f + f // 2:]]))


def test_config_keys_survive_a_round_trip_and_unbuilt_variants_are_refused(tmp_path):
    src = dict(_base(), model_type="mistral", architectures=["MistralForCausalLM"], sliding_window=128, bos_token_id=5,
               eos_token_id=[6, 7], pad_token_id=9, rope_scaling=None, attention_dropout=0.0, initializer_range=0.02,
               transformers_version="4.40.0", hidden_act="silu", tie_word_embeddings=False, some_future_key={"a": 1})
    cfg = LlamaConfig.from_hf_dict(src)
    assert cfg.sliding_window == 128 and cfg.extra["some_future_key"] == {"a": 1} and cfg.eos_token_id == [6, 7]
    out = cfg.to_hf_dict()
    for k in ("sliding_window", "bos_token_id", "eos_token_id", "pad_token_id", "attention_dropout", "initializer_range",
              "some_future_key", "model_type"):
        assert out[k] == src[k], k
    assert out["architectures"] == ["MistralForCausalLM"]
    assert cfg.layer_window(0, 128) is None and cfg.layer_window(1, 129) == 128    # inside the window: plain causal
    for bad in (dict(model_type="gemma2"), dict(hidden_act="gelu_pytorch_tanh"), dict(head_dim=20),
                dict(rope_scaling={"rope_type": "ntk-by-parts", "factor": 4.0})):
        with pytest.raises(NotImplementedError):
            LlamaConfig.from_hf_dict(dict(_base(), **bad))
    # Qwen2 carries a window that is switched off
    q = LlamaConfig.from_hf_dict(dict(_base(), model_type="qwen2", sliding_window=64, use_sliding_window=False))
    assert q.sliding_window is None and q.attention_bias


def test_yarn_rope_scaling_and_explicit_head_dim_match_huggingface():
    yarn = {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64, "beta_fast": 32, "beta_slow": 1}
    cfg = LlamaConfig.from_hf_dict(dict(_base(), model_type="llama", rope_scaling=dict(yarn)))
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=3)
    hf = tr.LlamaForCausalLM(tr.LlamaConfig(**_base(), rope_scaling=dict(yarn), attn_implementation="eager",
                                            tie_word_embeddings=False)).float()
    hf.load_state_dict({k: v.clone() for k, v in model.to_hf_state_dict().items()}, strict=False)
    x = torch.randint(0, 320, (2, 200))
    ours, ref = model(x), hf(x).logits
    assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (ours - ref).abs().max()
    plain = build_model(LlamaConfig(**_base()), dtype=torch.float32, device="cpu", seed=3)
    assert (plain(x) - ref).abs().max() > 2e-3
    # the mscale pair of DeepSeek-style configs and an explicit attention factor
    c1, s1 = basic.rope_tables(16, 16, 10000.0, "cpu", dict(yarn, mscale=1.0, mscale_all_dim=0.5), model_max_pos=256)
    c0, s0 = basic.rope_tables(16, 16, 10000.0, "cpu", dict(yarn, attention_factor=1.0), model_max_pos=256)
    import math
    want = (0.1 * math.log(4.0) + 1.0) / (0.05 * math.log(4.0) + 1.0)
    assert torch.allclose(c1, c0 * want, atol=1e-6) and torch.allclose(s1, s0 * want, atol=1e-6)

    # head_dim that is not hidden_size / heads (Mistral-Nemo style): 64 hidden, 4 heads of 32
    d = dict(_base(), model_type="llama", head_dim=32)
    cfg2 = LlamaConfig.from_hf_dict(d)
    assert cfg2.head_dim == 32 and cfg2.q_size == 128 and cfg2.to_hf_dict()["head_dim"] == 32
    m2 = build_model(cfg2, dtype=torch.float32, device="cpu", seed=4)
    assert m2.layers[0].o_proj.shape == (64, 128)
    hf2 = tr.LlamaForCausalLM(tr.LlamaConfig(**_base(), head_dim=32, attn_implementation="eager",
                                             tie_word_embeddings=False)).float()
    res = hf2.load_state_dict({k: v.clone() for k, v in m2.to_hf_state_dict().items()}, strict=False)
    assert not res.unexpected_keys
    x2 = torch.randint(0, 320, (2, 50))
    assert torch.allclose(m2(x2), hf2(x2).logits, atol=3e-4, rtol=1e-3)
    with pytest.raises(NotImplementedError):
        LlamaConfig.from_hf_dict(dict(_base(), model_type="llama", head_dim=20))


def test_qwen3_head_norms_match_huggingface(tmp_path):
    """Qwen3: no projection bias, RMSNorm over every query and key head before the rotation, explicit head_dim."""
    d = dict(_base(), model_type="qwen3", head_dim=32, use_sliding_window=False, attention_bias=False)
    cfg = LlamaConfig.from_hf_dict(d)
    assert cfg.qk_norm and cfg.head_dim == 32 and not cfg.attention_bias
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=6)
    with torch.no_grad():
        for l in model.layers:
            l.q_norm.uniform_(0.5, 1.5)
            l.k_norm.uniform_(0.5, 1.5)
    hf = tr.Qwen3ForCausalLM(tr.Qwen3Config(**_base(), head_dim=32, attn_implementation="eager", tie_word_embeddings=False,
                                            use_sliding_window=False, attention_bias=False)).float()
    res = hf.load_state_dict({k: v.clone() for k, v in model.to_hf_state_dict().items()}, strict=False)
    assert not res.unexpected_keys and not [k for k in res.missing_keys if "rotary" not in k], res
    x = torch.randint(0, 320, (2, 48))
    ours, ref = model(x), hf(x).logits
    assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (ours - ref).abs().max()
    tgt = torch.randint(0, 320, (2 * 48,))
    torch.nn.functional.cross_entropy(ours.reshape(-1, 320), tgt).backward()
    torch.nn.functional.cross_entropy(ref.reshape(-1, 320), tgt).backward()
    hf_grads = {n: p.grad for n, p in hf.named_parameters()}
    for n, p, sl in model.named_hf_parameters():
        g = p.grad if sl is None else p.grad[sl]
        assert torch.allclose(g, hf_grads[n], atol=2e-5, rtol=2e-3), (n, (g - hf_grads[n]).abs().max())
    # gradient checkpointing and the chunked inference path take the same norms
    g0 = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    model.grad_checkpointing = True
    torch.nn.functional.cross_entropy(model(x).reshape(-1, 320), tgt).backward()
    for n, p in model.named_parameters():
        assert torch.allclose(p.grad, g0[n], atol=1e-6, rtol=1e-5), n
    with torch.no_grad():
        assert torch.allclose(model.hidden_states(x), model.hidden_states_chunked(x, 16), atol=2e-5, rtol=1e-4)
    # both checkpoint directions
    save_hf_model(model, str(tmp_path / "ours"))
    c = json.load(open(tmp_path / "ours" / "config.json"))
    assert c["model_type"] == "qwen3" and c["architectures"] == ["Qwen3ForCausalLM"] and c["head_dim"] == 32
    hf2 = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ours"), dtype=torch.float32, attn_implementation="eager")
    assert torch.allclose(hf2(x).logits, ref, atol=3e-4, rtol=1e-3)
    hf.save_pretrained(str(tmp_path / "theirs"), safe_serialization=True)
    back = load_hf_model(str(tmp_path / "theirs"), dtype=torch.float32)
    assert back.cfg.qk_norm and torch.allclose(back(x), ref, atol=3e-4, rtol=1e-3)
    _, w0 = load_tp_weights(str(tmp_path / "theirs"), 0, 2, dtype=torch.float32)      # the norms are replicated
    assert torch.equal(w0["layers.1.q_norm"], back.layers[1].q_norm.data) and w0["layers.0.k_norm"].shape == (32,)
    with pytest.raises(NotImplementedError):
        LlamaConfig.from_hf_dict(dict(d, num_experts=8))


def test_rope_parameters_dict_of_newer_huggingface_configs_is_read(tmp_path):
    """transformers 5 writes ``rope_parameters = {rope_theta, rope_type, ...}`` instead of ``rope_theta`` / ``rope_scaling``."""
    hf_cfg = tr.LlamaConfig(**_base(rope_theta=500000.0), rope_scaling=dict(ROPE3), attn_implementation="eager",
                            tie_word_embeddings=False)
    hf = tr.LlamaForCausalLM(hf_cfg).float()
    hf.save_pretrained(str(tmp_path / "m"), safe_serialization=True)
    saved = json.load(open(tmp_path / "m" / "config.json"))
    back = load_hf_model(str(tmp_path / "m"), dtype=torch.float32)
    assert back.cfg.rope_theta == 500000.0
    assert (back.cfg.rope_scaling or {}).get("rope_type") == "llama3", (saved, back.cfg.rope_scaling)
    x = torch.randint(0, 320, (1, 150))
    assert torch.allclose(back(x), hf(x).logits, atol=3e-4, rtol=1e-3)


def test_phi3_longrope_matches_huggingface():
    """Phi-3 long-context checkpoints: per-frequency short / long factors chosen by the sequence length."""
    torch.manual_seed(0)
    short = (1.0 + 0.2 * torch.rand(8)).tolist()
    long = (1.5 + 2.0 * torch.rand(8)).tolist()
    scaling = {"type": "longrope", "short_factor": short, "long_factor": long}
    d = dict(_base(max_position_embeddings=256), model_type="phi3", pad_token_id=0, rope_scaling=scaling,
             original_max_position_embeddings=64)
    cfg = LlamaConfig.from_hf_dict(d)
    assert cfg.rope_scaling["original_max_position_embeddings"] == 64
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=8)
    hf_cfg = tr.Phi3Config(**_base(max_position_embeddings=256), pad_token_id=0, attn_implementation="eager",
                           tie_word_embeddings=False, sliding_window=None, original_max_position_embeddings=64,
                           rope_scaling=dict(scaling))
    hf = tr.Phi3ForCausalLM(hf_cfg).float()
    res = hf.load_state_dict({k: v.clone() for k, v in model.to_hf_state_dict().items()}, strict=False)
    assert not res.unexpected_keys
    for L in (48, 200, 40):          # short regime, long regime, short again (the cached tables must follow)
        x = torch.randint(0, 320, (2, L))
        ours, ref = model(x), hf(x).logits
        assert torch.allclose(ours, ref, atol=4e-4, rtol=1e-3), (L, (ours - ref).abs().max())
    same = LlamaConfig.from_hf_dict(dict(d, rope_scaling=dict(scaling, type="su")))
    assert same.rope_scaling["rope_type"] == "longrope"


def test_partial_rotary_matches_huggingface(tmp_path):
    """Phi-4-mini's layout: three quarters of every head rotate, the rest passes through; longrope factors cover the
    rotated part only; tied embeddings."""
    torch.manual_seed(1)
    base = _base(max_position_embeddings=256)
    rot_half = int(base["hidden_size"] // base["num_attention_heads"] * 0.75) // 2
    scaling = {"type": "longrope", "short_factor": (1.0 + 0.2 * torch.rand(rot_half)).tolist(),
               "long_factor": (1.5 + 2.0 * torch.rand(rot_half)).tolist()}
    hf_cfg = tr.Phi3Config(**base, pad_token_id=0, attn_implementation="eager", tie_word_embeddings=True,
                           sliding_window=None, original_max_position_embeddings=64, partial_rotary_factor=0.75,
                           rope_scaling=dict(scaling))
    hf = tr.Phi3ForCausalLM(hf_cfg).float()
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    model = load_hf_model(str(tmp_path / "hf"), dtype=torch.float32)
    cfg = model.cfg
    assert cfg.partial_rotary_factor == 0.75 and cfg.rotary_dim == 2 * rot_half < cfg.head_dim
    assert model.rope("cpu", 48)[0].shape[1] == rot_half
    for L in (48, 200):
        x = torch.randint(0, 320, (2, L))
        ours, ref = model(x), hf(x).logits
        assert torch.allclose(ours, ref, atol=4e-4, rtol=1e-3), (L, (ours - ref).abs().max())
    full = build_model(LlamaConfig.from_hf_dict(dict(cfg.to_hf_dict(), partial_rotary_factor=1.0, rope_scaling=None)),
                       dtype=torch.float32, device="cpu", seed=0)
    full.load_state_dict(model.state_dict())
    assert (full(x) - ref).abs().max() > 4e-3             # the factor is not a no-op
    # gradients through the inverse rotation of the rotated part only
    tgt = torch.randint(0, 320, (2 * 200,))
    torch.nn.functional.cross_entropy(model(x).view(-1, 320), tgt).backward()
    torch.nn.functional.cross_entropy(hf(x).logits.view(-1, 320), tgt).backward()
    g_hf = hf.model.layers[0].self_attn.qkv_proj.weight.grad
    assert torch.allclose(model.layers[0].qkv_proj.grad, g_hf, atol=2e-5, rtol=2e-3)
    # the factor survives a save and HuggingFace reads it back
    save_hf_model(model, str(tmp_path / "ours"))
    hf2 = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ours"), torch_dtype=torch.float32,
                                                  attn_implementation="eager")
    assert torch.allclose(hf2(x).logits, ref, atol=4e-4, rtol=1e-3)
    # the standalone op: elements past the rotary width are untouched, and the inverse undoes the rotation
    cos, sin = basic.rope_tables(64, 24, 10000.0, "cpu")
    v = torch.randn(10, 3 * 32)
    pos = torch.arange(10, dtype=torch.int32)
    r = basic.rope_(v.clone(), pos, cos, sin, 3, 32)
    assert torch.equal(r.view(10, 3, 32)[..., 24:], v.view(10, 3, 32)[..., 24:])
    assert not torch.allclose(r.view(10, 3, 32)[1:, :, :24], v.view(10, 3, 32)[1:, :, :24])
    assert torch.allclose(basic.rope_(r, pos, cos, sin, 3, 32, inverse=True), v, atol=1e-5)


@pytest.mark.parametrize("family", ["mistral", "qwen2 with windowed upper layers", "phi3"])
def test_sliding_window_attention_matches_huggingface(tmp_path, family):
    """Sequences longer than the window: a query sees the last ``sliding_window`` positions - logits, gradients (with and
    without recomputation) and the chunked inference path against HuggingFace; inside the window nothing changes."""
    torch.manual_seed(7)
    if family == "mistral":
        hf = tr.MistralForCausalLM(tr.MistralConfig(**_base(), sliding_window=32, attn_implementation="eager",
                                                    tie_word_embeddings=False)).float()
        flags = None
    elif family == "phi3":
        hf = tr.Phi3ForCausalLM(tr.Phi3Config(**_base(), sliding_window=32, pad_token_id=0, attn_implementation="eager",
                                              tie_word_embeddings=False)).float()
        flags = None
    else:
        hf = tr.Qwen2ForCausalLM(tr.Qwen2Config(**_base(num_hidden_layers=3), sliding_window=32, use_sliding_window=True,
                                                max_window_layers=1, attn_implementation="eager",
                                                tie_word_embeddings=False)).float()
        flags = [0, 1, 1]
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    model = load_hf_model(str(tmp_path / "hf"), dtype=torch.float32)
    cfg = model.cfg
    assert cfg.sliding_window == 32 and cfg.window_layers == flags
    for L, recompute in ((24, False), (100, False), (100, True)):
        model.grad_checkpointing = recompute
        model.zero_grad()
        hf.zero_grad()
        x = torch.randint(1, 320, (2, L))
        ours, ref = model(x), hf(x).logits
        assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (L, (ours - ref).abs().max())
        tgt = torch.randint(0, 320, (2 * L,))
        torch.nn.functional.cross_entropy(ours.reshape(-1, 320), tgt).backward()
        torch.nn.functional.cross_entropy(ref.reshape(-1, 320), tgt).backward()
        hf_g = {n: p.grad for n, p in hf.named_parameters()}
        for n, p, sl in model.named_hf_parameters():
            g = p.grad if sl is None else p.grad[sl]
            assert torch.allclose(g, hf_g[n], atol=2e-5, rtol=2e-3), (L, n, (g - hf_g[n]).abs().max())
    model.grad_checkpointing = False
    with torch.no_grad():
        hs = model.hidden_states_chunked(x, 16)
        assert torch.allclose(torch.nn.functional.linear(hs, model.lm_head).view(2, 100, -1), ref, atol=3e-4, rtol=1e-3)
        plain = build_model(LlamaConfig.from_hf_dict(dict(cfg.to_hf_dict(), sliding_window=None, use_sliding_window=False)),
                            dtype=torch.float32, device="cpu", seed=0)
        plain.load_state_dict(model.state_dict())
        assert (plain(x) - ref).abs().max() > 3e-3            # the window is not a no-op at this length
    save_hf_model(model, str(tmp_path / "ours"))
    hf2 = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ours"), torch_dtype=torch.float32,
                                                  attn_implementation="eager")
    assert torch.allclose(hf2(x).logits, ref, atol=3e-4, rtol=1e-3)


def test_dynamic_ntk_rope_scaling_matches_huggingface():
    """Inside the model's context nothing changes; beyond it the base follows the sequence length."""
    sc = {"rope_type": "dynamic", "factor": 3.0}
    cfg = LlamaConfig.from_hf_dict(dict(_base(max_position_embeddings=64), model_type="llama", rope_scaling=dict(sc)))
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=6)
    plain = build_model(LlamaConfig(**_base(max_position_embeddings=64)), dtype=torch.float32, device="cpu", seed=6)
    for L in (48, 200, 120, 40):          # a fresh HuggingFace model per length: its tables remember earlier lengths
        hf = tr.LlamaForCausalLM(tr.LlamaConfig(**_base(max_position_embeddings=64), rope_scaling=dict(sc),
                                                attn_implementation="eager", tie_word_embeddings=False)).float()
        hf.load_state_dict({k: v.clone() for k, v in model.to_hf_state_dict().items()}, strict=False)
        x = torch.randint(0, 320, (2, L))
        ours, ref = model(x), hf(x).logits
        assert torch.allclose(ours, ref, atol=4e-4, rtol=1e-3), (L, (ours - ref).abs().max())
        assert ((plain(x) - ref).abs().max() > 3e-3) == (L > 64), L
    # HunYuan's form: a fixed alpha instead of the length
    c, s_ = basic.rope_tables(16, 16, 10000.0, "cpu", {"rope_type": "dynamic", "alpha": 1000.0, "factor": 1.0})
    c2, s2 = basic.rope_tables(16, 16, 10000.0 * 1000.0 ** (16 / 14), "cpu")
    assert torch.allclose(c, c2) and torch.allclose(s_, s2)


def test_smollm3_layers_without_rotation_match_huggingface(tmp_path):
    """SmolLM3: Llama blocks of which every n-th applies no rotary embedding (the flags come from the interval when
    the config does not list them)."""
    base = _base(num_hidden_layers=4)
    hf_cfg = tr.SmolLM3Config(**base, pad_token_id=0, attn_implementation="eager", tie_word_embeddings=True,
                              no_rope_layer_interval=2)
    assert hf_cfg.no_rope_layers == [1, 0, 1, 0]
    hf = tr.SmolLM3ForCausalLM(hf_cfg).float()
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    model = load_hf_model(str(tmp_path / "hf"), dtype=torch.float32)
    assert model.cfg.model_type == "smollm3" and model.cfg.no_rope_layers == [1, 0, 1, 0]
    x = torch.randint(0, 320, (2, 64))
    ours, ref = model(x), hf(x).logits
    assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (ours - ref).abs().max()
    every = build_model(LlamaConfig.from_hf_dict(dict(model.cfg.to_hf_dict(), no_rope_layers=[1, 1, 1, 1])),
                        dtype=torch.float32, device="cpu", seed=0)
    every.load_state_dict(model.state_dict())
    assert (every(x) - ref).abs().max() > 3e-3                  # the flags matter
    # from the interval alone
    d = dict(model.cfg.to_hf_dict())
    d.pop("no_rope_layers")
    assert LlamaConfig.from_hf_dict(dict(d, no_rope_layer_interval=3)).no_rope_layers == [1, 1, 0, 1]
    # gradients, with recomputation in backward, and the chunked inference path
    model.grad_checkpointing = True
    tgt = torch.randint(0, 320, (2 * 64,))
    torch.nn.functional.cross_entropy(model(x).view(-1, 320), tgt).backward()
    torch.nn.functional.cross_entropy(hf(x).logits.view(-1, 320), tgt).backward()
    for li in (0, 1):
        want = torch.cat([getattr(hf.model.layers[li].self_attn, n).weight.grad for n in ("q_proj", "k_proj", "v_proj")])
        assert torch.allclose(model.layers[li].qkv_proj.grad, want, atol=2e-5, rtol=2e-3), li
    with torch.no_grad():
        hs = model.hidden_states_chunked(x, 16)
        assert torch.allclose(torch.nn.functional.linear(hs, model.lm_head).view(2, 64, -1), ref, atol=3e-4, rtol=1e-3)
    save_hf_model(model, str(tmp_path / "ours"))
    hf2 = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ours"), torch_dtype=torch.float32,
                                                  attn_implementation="eager")
    assert hf2.config.no_rope_layers == [1, 0, 1, 0] and torch.allclose(hf2(x).logits, ref, atol=3e-4, rtol=1e-3)
    with pytest.raises(ValueError, match="lists 3 layers"):
        LlamaConfig.from_hf_dict(dict(model.cfg.to_hf_dict(), no_rope_layers=[1, 0, 1]))
    # other model types ignore the key
    assert LlamaConfig.from_hf_dict(dict(_base(), model_type="llama", no_rope_layers=[0, 0])).no_rope_layers is None


_MORE = {   # family: (HuggingFace model, config, extra config keys, (pre_norm, post_norm, qk_norm_full, qk_norm), general node)
    "olmo2": ("Olmo2ForCausalLM", "Olmo2Config", {}, (False, True, True, False), True),
    "olmo3": ("Olmo3ForCausalLM", "Olmo3Config", dict(sliding_window=24, layer_types=["sliding_attention", "full_attention"]),
              (False, True, True, False), True),
    "ministral": ("MinistralForCausalLM", "MinistralConfig",
                  dict(head_dim=16, sliding_window=24, layer_types=["sliding_attention", "full_attention"]),
                  (True, False, False, False), False),
    "glm": ("GlmForCausalLM", "GlmConfig", dict(head_dim=16), (True, False, False, False), False),
    "glm4": ("Glm4ForCausalLM", "Glm4Config", dict(head_dim=16), (True, True, False, False), True),
    "exaone4": ("Exaone4ForCausalLM", "Exaone4Config", dict(sliding_window=None, layer_types=["full_attention"] * 2),
                (False, True, False, True), True),
    "exaone4 hybrid": ("Exaone4ForCausalLM", "Exaone4Config", dict(sliding_window=64, sliding_window_pattern=2),
                       (False, True, False, True), True),
    "helium": ("HeliumForCausalLM", "HeliumConfig", dict(head_dim=16), (True, False, False, False), False),
    "ernie4_5": ("Ernie4_5ForCausalLM", "Ernie4_5Config", dict(head_dim=32), (True, False, False, False), False),
    "hunyuan_v1_dense": ("HunYuanDenseV1ForCausalLM", "HunYuanDenseV1Config",
                         dict(head_dim=16, rope_parameters={"rope_type": "dynamic", "alpha": 50.0, "factor": 1.0,
                                                            "rope_theta": 10000.0}),
                         (True, False, False, True), True),
    "gemma": ("GemmaForCausalLM", "GemmaConfig", dict(head_dim=32), (True, False, False, False), True),
    "gemma3_text": ("Gemma3ForCausalLM", "Gemma3TextConfig",
                    dict(head_dim=32, sliding_window=24, sliding_window_pattern=2, query_pre_attn_scalar=48),
                    (True, True, False, True), True),
    "seed_oss": ("SeedOssForCausalLM", "SeedOssConfig", dict(head_dim=32, attention_dropout=0.0, residual_dropout=0.0),
                 (True, False, False, False), False),
}


@pytest.mark.parametrize("family,recompute", [("olmo2", False), ("olmo2", True), ("glm", False), ("glm4", False),
                                              ("glm4", True), ("exaone4", False), ("exaone4 hybrid", True),
                                              ("helium", False), ("ernie4_5", False), ("seed_oss", False),
                                              ("hunyuan_v1_dense", False), ("hunyuan_v1_dense", True),
                                              ("gemma", False), ("gemma3_text", False), ("gemma3_text", True),
                                              ("olmo3", False), ("olmo3", True), ("ministral", False)])
def test_more_decoder_families_match_huggingface(tmp_path, family, recompute):
    """OLMo 2 (norms behind the branches only, q/k norms over the whole projections), EXAONE 4 (the same placement with
    per-head q/k norms; hybrid checkpoints: windowed layers rotate, global ones do not), GLM (half of each head rotates,
    rotary pairs neighbours in the checkpoint, fused gate/up tensor, q/k/v bias), GLM-4 0414 (GLM with norms behind
    the branches as well), Helium and ERNIE 4.5 (Llama layers, rotary pairs neighbours), Seed-OSS (q/k/v bias and an
    explicit head_dim), HunYuan (per-head q/k norms behind the rotation, a base scaled by a fixed alpha), Gemma (GeGLU,
    norm weights stored minus one, scaled embeddings) and Gemma 3 text (Gemma with four norms per layer, per-head q/k
    norms, windowed layers with a rotary base of their own - the 48 positions are twice its window): logits, every gradient, the chunked inference path and checkpoints both ways."""
    cls_n, ccls_n, extra, flags, general = _MORE[family]
    cls, ccls = getattr(tr, cls_n), getattr(tr, ccls_n)
    mt = family.split()[0]
    torch.manual_seed(4)
    hf = cls(ccls(**{k: v for k, v in _base().items() if k != "rope_theta"}, **extra, pad_token_id=0,
                  attn_implementation="eager", tie_word_embeddings=False)).float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.uniform_(0.5, 1.5)
            elif n.endswith("bias"):
                p.normal_(0, 0.05)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    model = load_hf_model(str(tmp_path / "hf"), dtype=torch.float32)
    cfg = model.cfg
    assert cfg.model_type == mt and cfg.sandwich == general
    assert (cfg.pre_norm, cfg.post_norm, cfg.qk_norm_full, cfg.qk_norm) == flags
    if mt in ("glm", "glm4"):
        assert cfg.rope_interleaved and cfg.partial_rotary_factor == 0.5 and cfg.attention_bias and not cfg.o_bias
    if mt in ("helium", "ernie4_5"):
        assert cfg.rope_interleaved and cfg.partial_rotary_factor == 1.0 and not cfg.attention_bias
    if mt == "seed_oss":
        assert cfg.attention_bias and not cfg.o_bias and cfg.head_dim == 32 and not cfg.rope_interleaved
    if mt == "gemma3_text":
        assert cfg.window_layers == [1, 0] and cfg.sliding_window == 24 and cfg.rope_local_theta == 10000.0
        assert cfg.rope_theta == 1e6 and abs(cfg.attention_multiplier - 48 ** -0.5) < 1e-12
    if mt in ("gemma", "gemma3_text"):
        assert cfg.mlp_act == "gelu_tanh" and cfg.norm_plus_one and cfg.embedding_multiplier == 8.0
    if family == "exaone4 hybrid":
        assert cfg.no_rope_layers == [1, 0] and cfg.sliding_window == 64
    elif mt == "exaone4":
        assert cfg.no_rope_layers is None and cfg.sliding_window is None
    assert sum(p.numel() for p in model.parameters()) == cfg.num_params() == sum(p.numel() for p in hf.parameters())
    model.grad_checkpointing = recompute
    x = torch.randint(1, 320, (2, 48))          # not the padding id: HuggingFace's embedding gives it no gradient
    ours, ref = model(x), hf(x).logits
    assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (ours - ref).abs().max()
    tgt = torch.randint(0, 320, (2 * 48,))
    torch.nn.functional.cross_entropy(ours.reshape(-1, 320), tgt).backward()
    torch.nn.functional.cross_entropy(ref.reshape(-1, 320), tgt).backward()
    ours_g = {n: (p.grad if sl is None else p.grad[sl]) for n, p, sl in model.named_hf_parameters()}
    if cfg.rope_interleaved:
        ours_g = model._permute_rotary_rows(ours_g, to_checkpoint=True)
    hf_g = {n: p.grad for n, p in hf.named_parameters()}
    assert set(ours_g) == set(hf_g)
    for n, g in ours_g.items():
        assert torch.allclose(g, hf_g[n], atol=2e-5, rtol=2e-3), (n, (g - hf_g[n]).abs().max())
    model.grad_checkpointing = False
    with torch.no_grad():
        hs = model.hidden_states_chunked(x, 16)
        assert torch.allclose(torch.nn.functional.linear(hs, model.lm_head).view(2, 48, -1), ref, atol=3e-4, rtol=1e-3)
    save_hf_model(model, str(tmp_path / "ours"))
    hf2 = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ours"), torch_dtype=torch.float32,
                                                  attn_implementation="eager")
    assert type(hf2) is cls and torch.allclose(hf2(x).logits, ref, atol=3e-4, rtol=1e-3)
    if family == "olmo2":
        with pytest.raises(NotImplementedError, match="o_proj"):
            LlamaConfig.from_hf_dict(dict(cfg.to_hf_dict(), attention_bias=True))
    if family == "exaone4 hybrid":           # beyond the window the windowed layer sees the last 64 positions only
        assert cfg.window_layers == [1, 0] and cfg.layer_window(0, 100) == 64 and cfg.layer_window(1, 100) is None
        x = torch.randint(1, 320, (2, 100))
        assert torch.allclose(model(x), hf(x).logits, atol=3e-4, rtol=1e-3)


def test_llama_with_attention_and_mlp_biases_matches_huggingface(tmp_path):
    """HuggingFace's Llama with attention_bias (q, k, v and o) and mlp_bias (gate, up, down) - the Granite code models."""
    d = dict(_base(), model_type="llama", attention_bias=True, mlp_bias=True)
    cfg = LlamaConfig.from_hf_dict(d)
    assert cfg.attention_bias and cfg.o_bias and cfg.mlp_bias
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=12)
    hf = tr.LlamaForCausalLM(tr.LlamaConfig(**_base(), attention_bias=True, mlp_bias=True, attn_implementation="eager",
                                            tie_word_embeddings=False)).float()
    res = hf.load_state_dict({k: v.clone() for k, v in model.to_hf_state_dict().items()}, strict=False)
    assert not res.unexpected_keys and not [k for k in res.missing_keys if "rotary" not in k], res
    x = torch.randint(0, 320, (2, 48))
    ours, ref = model(x), hf(x).logits
    assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (ours - ref).abs().max()
    tgt = torch.randint(0, 320, (2 * 48,))
    torch.nn.functional.cross_entropy(ours.reshape(-1, 320), tgt).backward()
    torch.nn.functional.cross_entropy(ref.reshape(-1, 320), tgt).backward()
    hf_grads = {n: p.grad for n, p in hf.named_parameters()}
    seen = 0
    for n, p, sl in model.named_hf_parameters():
        g = p.grad if sl is None else p.grad[sl]
        assert torch.allclose(g, hf_grads[n], atol=2e-5, rtol=2e-3), (n, (g - hf_grads[n]).abs().max())
        seen += n.endswith(".bias")
    assert seen == 2 * 7                                   # q, k, v, o, gate, up, down per layer
    g0 = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    model.grad_checkpointing = True
    torch.nn.functional.cross_entropy(model(x).reshape(-1, 320), tgt).backward()
    for n, p in model.named_parameters():
        assert torch.allclose(p.grad, g0[n], atol=1e-6, rtol=1e-5), n
    with torch.no_grad():
        assert torch.allclose(model.hidden_states(x), model.hidden_states_chunked(x, 16), atol=2e-5, rtol=1e-4)
    save_hf_model(model, str(tmp_path / "ours"))
    c = json.load(open(tmp_path / "ours" / "config.json"))
    assert c["model_type"] == "llama" and c["attention_bias"] is True and c["mlp_bias"] is True
    back = load_hf_model(str(tmp_path / "ours"), dtype=torch.float32)
    assert torch.equal(back(x), model(x))
    with pytest.raises(NotImplementedError):
        load_tp_weights(str(tmp_path / "ours"), 0, 2, dtype=torch.float32)
    # the engine's flat gradient slots take the bias gradients too
    from llm_distillery_b200.engine.trainer import DistillEngine, synthetic_batch
    eng = DistillEngine(back, loss="kl", temperature=1.0, optimizer="adamw", lr=1e-2)
    b0 = back.layers[0].down_bias.detach().clone()
    hb = synthetic_batch(cfg.vocab_size, 2, 32, 8, seed=0)
    l0 = eng.train_step([hb]); l1 = eng.train_step([hb])
    assert l1 < l0 and not torch.equal(back.layers[0].down_bias, b0)


def test_granite_multipliers_match_huggingface(tmp_path):
    """Granite: fixed multipliers on the embedding output, the attention scores, each branch and the logits (and
    optionally biases on every projection)."""
    mult = dict(embedding_multiplier=6.0, attention_multiplier=0.09, residual_multiplier=0.3, logits_scaling=4.0)
    d = dict(_base(), model_type="granite", attention_bias=True, mlp_bias=True, **mult)
    cfg = LlamaConfig.from_hf_dict(d)
    assert cfg.residual_multiplier == 0.3 and cfg.logits_scaling == 4.0 and cfg.o_bias and cfg.mlp_bias
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=13)
    hf = tr.GraniteForCausalLM(tr.GraniteConfig(**_base(), attention_bias=True, mlp_bias=True, **mult,
                                                attn_implementation="eager", tie_word_embeddings=False)).float()
    res = hf.load_state_dict({k: v.clone() for k, v in model.to_hf_state_dict().items()}, strict=False)
    assert not res.unexpected_keys and not [k for k in res.missing_keys if "rotary" not in k], res
    x = torch.randint(0, 320, (2, 48))
    ours, ref = model(x), hf(x).logits
    assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (ours - ref).abs().max()
    plain = build_model(LlamaConfig.from_hf_dict(dict(_base(), model_type="llama", attention_bias=True, mlp_bias=True)),
                        dtype=torch.float32, device="cpu", seed=13)
    assert (plain(x) - ref).abs().max() > 1e-2            # the multipliers matter
    tgt = torch.randint(0, 320, (2 * 48,))
    torch.nn.functional.cross_entropy(ours.reshape(-1, 320), tgt).backward()
    torch.nn.functional.cross_entropy(ref.reshape(-1, 320), tgt).backward()
    hf_grads = {n: p.grad for n, p in hf.named_parameters()}
    for n, p, sl in model.named_hf_parameters():
        g = p.grad if sl is None else p.grad[sl]
        assert torch.allclose(g, hf_grads[n], atol=3e-5, rtol=3e-3), (n, (g - hf_grads[n]).abs().max())
    g0 = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    model.grad_checkpointing = True
    torch.nn.functional.cross_entropy(model(x).reshape(-1, 320), tgt).backward()
    for n, p in model.named_parameters():
        assert torch.allclose(p.grad, g0[n], atol=1e-6, rtol=1e-5), n
    with torch.no_grad():
        assert torch.allclose(model.hidden_states(x), model.hidden_states_chunked(x, 16), atol=2e-5, rtol=1e-4)
    save_hf_model(model, str(tmp_path / "ours"))
    c = json.load(open(tmp_path / "ours" / "config.json"))
    assert c["model_type"] == "granite" and c["residual_multiplier"] == 0.3 and c["logits_scaling"] == 4.0
    hf2 = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ours"), dtype=torch.float32, attn_implementation="eager")
    assert torch.allclose(hf2(x).logits, ref, atol=3e-4, rtol=1e-3)
    back = load_hf_model(str(tmp_path / "ours"), dtype=torch.float32)
    assert torch.equal(back(x), model(x))
    with pytest.raises(NotImplementedError):
        load_tp_weights(str(tmp_path / "ours"), 0, 2, dtype=torch.float32)
    # a Llama config that happens to carry such keys is not affected by them
    assert LlamaConfig.from_hf_dict(dict(_base(), model_type="llama", residual_multiplier=0.5)).residual_multiplier == 1.0


def test_every_model_type_survives_config_round_trips():
    """to_hf_dict -> from_hf_dict gives the same configuration for every model type that is read, and every type in
    the list of known types is exercised here."""
    import dataclasses
    moe = dict(num_local_experts=4, num_experts_per_tok=2)
    cases = {
        "llama": {}, "mistral": dict(sliding_window=128),
        "qwen2": dict(attention_bias=True, sliding_window=64, window_layers=[0, 1]),
        "phi3": dict(partial_rotary_factor=0.75), "mixtral": moe,
        "qwen3": dict(qk_norm=True, head_dim_override=32),
        "qwen3_moe": dict(moe, qk_norm=True, moe_renormalize=False),
        "qwen2_moe": dict(moe, attention_bias=True, shared_expert_intermediate_size=80, moe_renormalize=False),
        "granite": dict(embedding_multiplier=6.0, attention_multiplier=0.2, residual_multiplier=0.4, logits_scaling=3.0),
        "granitemoe": dict(moe, residual_multiplier=0.4, attention_multiplier=0.2, shared_expert_gated=False),
        "granitemoeshared": dict(moe, residual_multiplier=0.4, attention_multiplier=0.2, shared_expert_gated=False,
                                 shared_expert_intermediate_size=80),
        "smollm3": dict(no_rope_layers=[1, 0]),
        "olmo2": dict(pre_norm=False, post_norm=True, qk_norm_full=True),
        "olmoe": dict(moe, qk_norm_full=True, moe_renormalize=False),
        "ministral": dict(sliding_window=24, window_layers=[1, 0]),
        "olmo3": dict(pre_norm=False, post_norm=True, qk_norm_full=True, sliding_window=24, window_layers=[1, 0]),
        "glm": dict(attention_bias=True, partial_rotary_factor=0.5, rope_interleaved=True),
        "glm4": dict(attention_bias=True, partial_rotary_factor=0.5, rope_interleaved=True, post_norm=True),
        "exaone4": dict(pre_norm=False, post_norm=True, qk_norm=True, no_rope_layers=[1, 0], window_layers=[1, 0],
                        sliding_window=128),
        "helium": dict(rope_interleaved=True), "ernie4_5": dict(rope_interleaved=True),
        "seed_oss": dict(attention_bias=True, head_dim_override=32),
        "gemma": dict(mlp_act="gelu_tanh", norm_plus_one=True, embedding_multiplier_rounded=True, embedding_multiplier=8.0,
                      head_dim_override=32),
        "gemma3_text": dict(mlp_act="gelu_tanh", norm_plus_one=True, embedding_multiplier_rounded=True,
                            embedding_multiplier=8.0, head_dim_override=32, post_norm=True, qk_norm=True,
                            sliding_window=24, window_layers=[1, 0], rope_local_theta=10000.0,
                            attention_multiplier=48 ** -0.5),
        "hunyuan_v1_dense": dict(qk_norm=True, qk_norm_after_rope=True,
                                 rope_scaling={"rope_type": "dynamic", "alpha": 1000.0, "factor": 1.0}),
    }
    assert set(cases) == set(LlamaConfig._KNOWN_TYPES)
    for mt, kw in cases.items():
        cfg = LlamaConfig(**_base(), model_type=mt, **kw)
        back = LlamaConfig.from_hf_dict(cfg.to_hf_dict())
        a, b = dataclasses.asdict(cfg), dataclasses.asdict(back)
        a.pop("extra"), b.pop("extra")
        if a["attention_multiplier"] is None and b["attention_multiplier"] is not None:     # written out as 1 / sqrt(d)
            assert abs(b["attention_multiplier"] - cfg.head_dim ** -0.5) < 1e-12
            b["attention_multiplier"] = None
        assert a == b, (mt, {k: (a[k], b[k]) for k in a if a[k] != b[k]})
        again = LlamaConfig.from_hf_dict(back.to_hf_dict())
        assert dataclasses.asdict(again) == dataclasses.asdict(back), mt


# config.json contents as published for these checkpoints (keys that matter here; long factor lists shortened)
_PUBLISHED = {
 "llama-3.1-8b": {"architectures":["LlamaForCausalLM"],"attention_bias":False,"attention_dropout":0.0,"bos_token_id":128000,"eos_token_id":[128001,128008,128009],"hidden_act":"silu","hidden_size":4096,"initializer_range":0.02,"intermediate_size":14336,"max_position_embeddings":131072,"mlp_bias":False,"model_type":"llama","num_attention_heads":32,"num_hidden_layers":32,"num_key_value_heads":8,"pretraining_tp":1,"rms_norm_eps":1e-05,"rope_scaling":{"factor":8.0,"low_freq_factor":1.0,"high_freq_factor":4.0,"original_max_position_embeddings":8192,"rope_type":"llama3"},"rope_theta":500000.0,"tie_word_embeddings":False,"torch_dtype":"bfloat16","use_cache":True,"vocab_size":128256},
 "qwen2.5-7b": {"architectures":["Qwen2ForCausalLM"],"attention_dropout":0.0,"bos_token_id":151643,"eos_token_id":151645,"hidden_act":"silu","hidden_size":3584,"initializer_range":0.02,"intermediate_size":18944,"max_position_embeddings":32768,"max_window_layers":28,"model_type":"qwen2","num_attention_heads":28,"num_hidden_layers":28,"num_key_value_heads":4,"rms_norm_eps":1e-06,"rope_theta":1000000.0,"sliding_window":131072,"tie_word_embeddings":False,"torch_dtype":"bfloat16","use_cache":True,"use_sliding_window":False,"vocab_size":152064},
 "qwen3-8b": {"architectures":["Qwen3ForCausalLM"],"attention_bias":False,"attention_dropout":0.0,"head_dim":128,"hidden_act":"silu","hidden_size":4096,"intermediate_size":12288,"max_position_embeddings":40960,"max_window_layers":36,"model_type":"qwen3","num_attention_heads":32,"num_hidden_layers":36,"num_key_value_heads":8,"rms_norm_eps":1e-06,"rope_scaling":None,"rope_theta":1000000,"sliding_window":None,"tie_word_embeddings":False,"use_sliding_window":False,"vocab_size":151936},
 "mistral-7b-v0.1": {"architectures":["MistralForCausalLM"],"bos_token_id":1,"eos_token_id":2,"hidden_act":"silu","hidden_size":4096,"initializer_range":0.02,"intermediate_size":14336,"max_position_embeddings":32768,"model_type":"mistral","num_attention_heads":32,"num_hidden_layers":32,"num_key_value_heads":8,"rms_norm_eps":1e-05,"rope_theta":10000.0,"sliding_window":4096,"tie_word_embeddings":False,"vocab_size":32000},
 "mistral-nemo": {"architectures":["MistralForCausalLM"],"head_dim":128,"hidden_act":"silu","hidden_size":5120,"intermediate_size":14336,"max_position_embeddings":1024000,"model_type":"mistral","num_attention_heads":32,"num_hidden_layers":40,"num_key_value_heads":8,"rms_norm_eps":1e-05,"rope_theta":1000000.0,"sliding_window":None,"vocab_size":131072},
 "phi-4-mini": {"architectures":["Phi3ForCausalLM"],"attention_bias":False,"bos_token_id":199999,"embd_pdrop":0.0,"eos_token_id":199999,"full_attn_mod":1,"hidden_act":"silu","hidden_size":3072,"intermediate_size":8192,"interpolate_factor":1,"lm_head_bias":False,"max_position_embeddings":131072,"mlp_bias":False,"model_type":"phi3","num_attention_heads":24,"num_hidden_layers":32,"num_key_value_heads":8,"original_max_position_embeddings":4096,"pad_token_id":199999,"partial_rotary_factor":0.75,"resid_pdrop":0.0,"rms_norm_eps":1e-05,"rope_scaling":{"long_factor":[1.0]*48,"short_factor":[1.0]*48,"type":"longrope"},"rope_theta":10000.0,"sliding_window":262144,"tie_word_embeddings":True,"vocab_size":200064},
 "mixtral-8x7b": {"architectures":["MixtralForCausalLM"],"hidden_act":"silu","hidden_size":4096,"intermediate_size":14336,"max_position_embeddings":32768,"model_type":"mixtral","num_attention_heads":32,"num_experts_per_tok":2,"num_hidden_layers":32,"num_key_value_heads":8,"num_local_experts":8,"output_router_logits":False,"rms_norm_eps":1e-05,"rope_theta":1000000.0,"router_aux_loss_coef":0.02,"sliding_window":None,"vocab_size":32000},
 "olmo2-7b": {"architectures":["Olmo2ForCausalLM"],"attention_bias":False,"hidden_act":"silu","hidden_size":4096,"intermediate_size":11008,"max_position_embeddings":4096,"model_type":"olmo2","num_attention_heads":32,"num_hidden_layers":32,"num_key_value_heads":32,"rms_norm_eps":1e-06,"rope_scaling":None,"rope_theta":500000,"tie_word_embeddings":False,"vocab_size":100352},
 "glm-4-9b-chat-hf": {"architectures":["GlmForCausalLM"],"attention_bias":True,"head_dim":128,"hidden_act":"silu","hidden_size":4096,"intermediate_size":13696,"max_position_embeddings":131072,"model_type":"glm","num_attention_heads":32,"num_hidden_layers":40,"num_key_value_heads":2,"partial_rotary_factor":0.5,"rms_norm_eps":1.5625e-07,"rope_theta":10000.0,"tie_word_embeddings":False,"vocab_size":151552},
 "smollm3-3b": {"architectures":["SmolLM3ForCausalLM"],"attention_bias":False,"hidden_act":"silu","hidden_size":2048,"intermediate_size":11008,"max_position_embeddings":65536,"mlp_bias":False,"model_type":"smollm3","no_rope_layer_interval":4,"no_rope_layers":[1,1,1,0]*9,"num_attention_heads":16,"num_hidden_layers":36,"num_key_value_heads":4,"rms_norm_eps":1e-06,"rope_scaling":None,"rope_theta":5000000.0,"sliding_window":None,"use_sliding_window":False,"tie_word_embeddings":True,"vocab_size":128256},
 "granite-3.1-1b-a400m": {"architectures":["GraniteMoeForCausalLM"],"attention_bias":False,"attention_multiplier":0.015625,"embedding_multiplier":12.0,"hidden_act":"silu","hidden_size":1024,"intermediate_size":512,"logits_scaling":6.0,"max_position_embeddings":131072,"model_type":"granitemoe","num_attention_heads":16,"num_experts_per_tok":8,"num_hidden_layers":24,"num_key_value_heads":8,"num_local_experts":32,"output_router_logits":False,"residual_multiplier":0.22,"rms_norm_eps":1e-06,"rope_scaling":None,"rope_theta":10000000.0,"router_aux_loss_coef":0.0,"tie_word_embeddings":True,"vocab_size":49155},
 "gemma-2": {"model_type":"gemma2","hidden_size":2304},
}


def test_published_configs_parse_to_the_published_sizes():
    want = {"llama-3.1-8b": 8.03, "qwen2.5-7b": 7.62, "qwen3-8b": 8.19, "mistral-7b-v0.1": 7.24, "mistral-nemo": 12.25,
            "phi-4-mini": 3.84, "mixtral-8x7b": 46.70, "olmo2-7b": 7.30, "glm-4-9b-chat-hf": 9.40, "smollm3-3b": 3.08,
            "granite-3.1-1b-a400m": 1.33}
    for name, d in _PUBLISHED.items():
        if name not in want:
            with pytest.raises(NotImplementedError, match="model_type"):
                LlamaConfig.from_hf_dict(d)
            continue
        cfg = LlamaConfig.from_hf_dict(d)
        assert abs(cfg.num_params() / 1e9 - want[name]) < 0.006, (name, cfg.num_params())
        assert cfg.head_dim in (64, 128) and cfg.rotary_dim % 16 == 0, name       # what the flash kernels take
        assert LlamaConfig.from_hf_dict(cfg.to_hf_dict()).num_params() == cfg.num_params()
    g = LlamaConfig.from_hf_dict({"architectures": ["Gemma3ForCausalLM"], "attention_bias": False, "head_dim": 256,
                                  "hidden_activation": "gelu_pytorch_tanh", "hidden_size": 1152, "intermediate_size": 6912,
                                  "max_position_embeddings": 32768, "model_type": "gemma3_text", "num_attention_heads": 4,
                                  "num_hidden_layers": 26, "num_key_value_heads": 1, "query_pre_attn_scalar": 256,
                                  "rms_norm_eps": 1e-06, "rope_local_base_freq": 10000, "rope_scaling": None,
                                  "rope_theta": 1000000, "sliding_window": 512, "sliding_window_pattern": 6,
                                  "vocab_size": 262144, "final_logit_softcapping": None, "attn_logit_softcapping": None})
    assert abs(g.num_params() / 1e9 - 1.00) < 0.006 and g.window_layers.count(0) == 4 and g.rope_local_theta == 10000.0
    g.check_gpu_kernels()                                        # heads of 256 run, on PyTorch's attention
    assert LlamaConfig.from_hf_dict(_PUBLISHED["phi-4-mini"]).rotary_dim == 96
    assert LlamaConfig.from_hf_dict(_PUBLISHED["mistral-7b-v0.1"]).sliding_window == 4096
    assert LlamaConfig.from_hf_dict(_PUBLISHED["qwen2.5-7b"]).sliding_window is None
    assert LlamaConfig.from_hf_dict(_PUBLISHED["smollm3-3b"]).no_rope_layers.count(0) == 9


def test_shapes_outside_the_gpu_kernels_are_named_before_any_launch():
    LlamaConfig(**_base(hidden_size=256, num_attention_heads=4)).check_gpu_kernels()                  # head_dim 64
    LlamaConfig(**_base(hidden_size=256, num_attention_heads=2, partial_rotary_factor=0.75)).check_gpu_kernels()
    with pytest.raises(NotImplementedError, match="rotary width 8"):
        LlamaConfig(**_base(partial_rotary_factor=0.5)).check_gpu_kernels()
    with pytest.raises(NotImplementedError, match="head_dim 24.*rotary width 24"):
        LlamaConfig(**_base(hidden_size=96)).check_gpu_kernels()
    LlamaConfig(**_base(hidden_size=1024, head_dim_override=256)).check_gpu_kernels()     # PyTorch's attention
    with pytest.raises(NotImplementedError, match="intermediate_size 100"):
        LlamaConfig(**_base(hidden_size=256, num_attention_heads=4, intermediate_size=100)).check_gpu_kernels()


def test_gemma3_multimodal_wrapper_loads_as_its_language_model(tmp_path):
    """A Gemma 3 checkpoint with a vision tower: the text_config block (which lists only what differs from
    HuggingFace's defaults) and the language model's tensors are read; the result is a text-only Gemma 3."""
    text = dict(hidden_size=64, intermediate_size=136, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                head_dim=32, vocab_size=320, sliding_window=24, sliding_window_pattern=2, max_position_embeddings=256,
                rope_scaling={"rope_type": "linear", "factor": 8.0})
    vision = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2, image_size=28,
                  patch_size=14)
    torch.manual_seed(9)
    hf = tr.Gemma3ForConditionalGeneration(tr.Gemma3Config(text_config=text, vision_config=vision, mm_tokens_per_image=4,
                                                           attn_implementation="eager")).float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.uniform_(-0.3, 0.3)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    hf.eval()
    model = load_hf_model(str(tmp_path / "hf"), dtype=torch.float32)
    cfg = model.cfg
    assert cfg.model_type == "gemma3_text" and cfg.head_dim == 32 and cfg.window_layers == [1, 0]
    assert cfg.rope_scaling["factor"] == 8.0 and cfg.rope_local_theta == 10000.0 and cfg.rope_theta == 1e6
    x = torch.randint(1, 320, (2, 60))
    with torch.no_grad():
        ref = hf(input_ids=x).logits
        assert torch.allclose(model(x), ref, atol=4e-4, rtol=1e-3), (model(x) - ref).abs().max()
    # a published text_config names only a few keys: the rest are HuggingFace's defaults, not this model's
    big = LlamaConfig.from_hf_dict({"model_type": "gemma3", "text_config": {
        "hidden_size": 2560, "intermediate_size": 10240, "model_type": "gemma3_text", "num_hidden_layers": 34,
        "rope_scaling": {"factor": 8.0, "rope_type": "linear"}, "sliding_window": 1024}})
    assert (big.vocab_size, big.num_attention_heads, big.num_key_value_heads, big.head_dim) == (262208, 8, 4, 256)
    assert big.window_layers.count(0) == 5 and big.embedding_multiplier == 2560 ** 0.5 and big.tie_word_embeddings
    assert abs(big.num_params() / 1e9 - 3.88) < 0.01             # the 4B checkpoint's language model
    save_hf_model(model, str(tmp_path / "ours"))
    hf2 = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ours"), torch_dtype=torch.float32,
                                                  attn_implementation="eager")
    assert type(hf2) is tr.Gemma3ForCausalLM and torch.allclose(hf2(x).logits, ref, atol=4e-4, rtol=1e-3)


@pytest.mark.parametrize("family", ["seed_oss", "smollm3", "qwen3", "phi3 with partial rotation"])
def test_tensor_parallel_slice_loader_agrees_with_slicing_the_whole_model(tmp_path, family):
    """The types the tensor-parallel teacher takes: what ``load_tp_weights`` reads from a saved folder rank by rank is
    what ``shard_llama_weights`` cuts out of the whole model; the types it does not take are refused by name."""
    from llm_distillery_b200.parallel.tp import shard_llama_weights
    kw = {"seed_oss": dict(model_type="seed_oss", attention_bias=True, head_dim_override=32),
          "smollm3": dict(model_type="smollm3", no_rope_layers=[1, 0]), "qwen3": dict(model_type="qwen3", qk_norm=True),
          "phi3 with partial rotation": dict(model_type="phi3", partial_rotary_factor=0.5)}[family]
    cfg = LlamaConfig(**_base(), **kw)
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=1)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("_bias"):
                p.normal_(0, 0.1)
    save_hf_model(model, str(tmp_path / "m"))
    sd = {k: v.detach() for k, v in model.state_dict().items()}
    for rank in range(2):
        got_cfg, got = load_tp_weights(str(tmp_path / "m"), rank, 2, dtype=torch.float32)
        want = shard_llama_weights(cfg, sd, rank, 2, None)
        assert got_cfg.model_type == cfg.model_type and got_cfg.rotary_dim == cfg.rotary_dim
        for k, v in want.items():
            if torch.is_tensor(v):
                assert torch.equal(v, got[k]), (rank, k)
    for other in (dict(model_type="olmo2", pre_norm=False, post_norm=True, qk_norm_full=True),
                  dict(model_type="glm", attention_bias=True, partial_rotary_factor=0.5, rope_interleaved=True),
                  dict(model_type="gemma", mlp_act="gelu_tanh", norm_plus_one=True, head_dim_override=32)):
        save_hf_model(build_model(LlamaConfig(**_base(), **other), dtype=torch.float32, device="cpu", seed=1),
                      str(tmp_path / other["model_type"]))
        with pytest.raises(NotImplementedError, match="tp_size = 1"):
            load_tp_weights(str(tmp_path / other["model_type"]), 0, 2)


def test_mistral3_wrapper_loads_as_its_language_model(tmp_path):
    """Mistral Small 3.1 style checkpoints: a vision tower around a Mistral text model."""
    text = dict(_base(), model_type="mistral", head_dim=32, sliding_window=None)
    vision = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2, image_size=28,
                  patch_size=14, head_dim=16)
    torch.manual_seed(11)
    hf = tr.Mistral3ForConditionalGeneration(tr.Mistral3Config(text_config=text, vision_config=vision,
                                                               attn_implementation="eager")).float().eval()
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    model = load_hf_model(str(tmp_path / "hf"), dtype=torch.float32)
    assert model.cfg.model_type == "mistral" and model.cfg.head_dim == 32
    x = torch.randint(1, 320, (2, 40))
    with torch.no_grad():
        ref = hf(input_ids=x).logits
        assert torch.allclose(model(x), ref, atol=3e-4, rtol=1e-3), (model(x) - ref).abs().max()
    # the tensor-parallel loader reads the wrapped tensors through the same names
    from llm_distillery_b200.parallel.tp import shard_llama_weights
    sd = {k: v.detach() for k, v in model.state_dict().items()}
    for rank in range(2):
        _, got = load_tp_weights(str(tmp_path / "hf"), rank, 2, dtype=torch.float32)
        want = shard_llama_weights(model.cfg, sd, rank, 2, None)
        assert all(torch.equal(v, got[k]) for k, v in want.items() if torch.is_tensor(v))
    with pytest.raises(ValueError, match="does not name"):
        LlamaConfig.from_hf_dict({"model_type": "mistral3", "text_config": {"model_type": "mistral", "hidden_size": 64}})
    with pytest.raises(NotImplementedError, match="language model"):
        LlamaConfig.from_hf_dict({"model_type": "qwen2_vl", "text_config": {"model_type": "qwen2_vl_text"}})
