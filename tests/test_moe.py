"""Mixtral-style sparse mixture-of-experts decoder (models/moe.py) against HuggingFace's own Mixtral modules on CPU:
logits, every parameter's gradient, checkpoint names both ways, gradient checkpointing, the engine's flat gradient
slots, and the reference's default ``freeze_layers`` entry (the router)."""
import json

import pytest
import torch

from llm_distillery_b200.ckpt.hf import load_hf_model, save_hf_model
from llm_distillery_b200.engine.trainer import DistillEngine, synthetic_batch
from llm_distillery_b200.models.llama import LlamaConfig, build_model

tr = pytest.importorskip("transformers")


def _base(**kw):
    d = dict(vocab_size=320, hidden_size=64, intermediate_size=136, num_hidden_layers=2, num_attention_heads=4,
             num_key_value_heads=2, max_position_embeddings=256, rope_theta=10000.0, rms_norm_eps=1e-6)
    d.update(kw)
    return d


def _pair(seed=3, experts=4, k=2):
    cfg = LlamaConfig(**_base(model_type="mixtral", num_local_experts=experts, num_experts_per_tok=k))
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=seed)
    with torch.no_grad():       # spread the router so that the experts' shares differ
        for l in model.layers:
            l.router.mul_(30.0)
    hf_cfg = tr.MixtralConfig(**_base(), num_local_experts=experts, num_experts_per_tok=k, attn_implementation="eager",
                              tie_word_embeddings=False, sliding_window=None, router_jitter_noise=0.0)
    hf = tr.MixtralForCausalLM(hf_cfg).float()
    return cfg, model, hf


def _load_into_hf(hf, sd):
    """Our HF-named tensors into a HuggingFace Mixtral, whatever this transformers version calls its expert tensors."""
    own = hf.state_dict()
    if all(k in own for k in sd):
        return hf.load_state_dict({k: v.clone() for k, v in sd.items()}, strict=False)
    # newer releases stack the experts: experts.gate_up_proj [E, 2f, h] / experts.down_proj [E, h, f]
    out = {k: v.clone() for k, v in sd.items() if "block_sparse_moe.experts" not in k}
    layers = sorted({k.split(".")[2] for k in sd if "block_sparse_moe.experts" in k}, key=int)
    for li in layers:
        pre = f"model.layers.{li}.block_sparse_moe.experts."
        E = 1 + max(int(k[len(pre):].split(".")[0]) for k in sd if k.startswith(pre))
        gu = torch.stack([torch.cat([sd[f"{pre}{e}.w1.weight"], sd[f"{pre}{e}.w3.weight"]]) for e in range(E)])
        dn = torch.stack([sd[f"{pre}{e}.w2.weight"] for e in range(E)])
        cand_gu = [k for k in own if k.startswith(f"model.layers.{li}.") and k.endswith("experts.gate_up_proj")]
        cand_dn = [k for k in own if k.startswith(f"model.layers.{li}.") and k.endswith("experts.down_proj")]
        assert cand_gu and cand_dn, [k for k in own if f"layers.{li}." in k]
        out[cand_gu[0]] = gu if own[cand_gu[0]].shape == gu.shape else gu.transpose(1, 2).contiguous()
        out[cand_dn[0]] = dn if own[cand_dn[0]].shape == dn.shape else dn.transpose(1, 2).contiguous()
    renamed = {}
    for k, v in out.items():       # the router may live under another name as well
        if k not in own and k.endswith("block_sparse_moe.gate.weight"):
            alt = [o for o in own if o.startswith(k.rsplit("block_sparse_moe", 1)[0]) and "gate" in o and "experts" not in o]
            assert alt, k
            renamed[alt[0]] = v
        else:
            renamed[k] = v
    return hf.load_state_dict(renamed, strict=False)


def test_logits_and_gradients_match_huggingface_mixtral():
    cfg, model, hf = _pair()
    res = _load_into_hf(hf, model.to_hf_state_dict())
    assert not [k for k in res.missing_keys if "rotary" not in k], res.missing_keys
    x = torch.randint(0, 320, (2, 48))
    ours, ref = model(x), hf(x).logits
    assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (ours - ref).abs().max()
    tgt = torch.randint(0, 320, (2, 48))
    torch.nn.functional.cross_entropy(ours.reshape(-1, 320), tgt.reshape(-1)).backward()
    torch.nn.functional.cross_entropy(ref.reshape(-1, 320), tgt.reshape(-1)).backward()
    hf_grads = {n: p.grad for n, p in hf.named_parameters()}
    stacked = any(n.endswith("experts.gate_up_proj") for n in hf_grads)     # newer releases stack the experts
    checked = 0
    for n, p, sl in model.named_hf_parameters():
        g = p.grad if sl is None else p.grad[sl]
        if n in hf_grads:
            want = hf_grads[n]
        elif n.endswith("block_sparse_moe.gate.weight"):
            want = hf_grads[n.replace("block_sparse_moe.gate", "mlp.gate")]
        elif stacked and ".experts." in n:
            pre, rest = n.split("block_sparse_moe.experts.")
            e, which = int(rest.split(".")[0]), rest.split(".")[1]
            f = cfg.intermediate_size
            if which == "w2":
                want = hf_grads[pre + "mlp.experts.down_proj"][e]
            else:
                gu = hf_grads[pre + "mlp.experts.gate_up_proj"][e]
                want = gu[:f] if which == "w1" else gu[f:]
        else:
            raise AssertionError(f"no counterpart for {n}")
        assert torch.allclose(g, want, atol=2e-5, rtol=2e-3), (n, (g - want).abs().max())
        checked += 1
    assert checked == 3 + 2 * (7 + 3 * 4)
    # every expert received rows, and their gradients are finite and not all zero
    for l in model.layers:
        assert torch.isfinite(l.gate_up_proj.grad).all() and (l.gate_up_proj.grad.abs().amax(dim=(1, 2)) > 0).all()


def test_gradient_checkpointing_and_inference_paths_agree():
    cfg, model, _ = _pair(seed=5)
    x = torch.randint(0, 320, (2, 40))
    a = model(x)
    a.square().mean().backward()
    g0 = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad()
    model.grad_checkpointing = True
    b = model(x)
    b.square().mean().backward()
    assert torch.allclose(a, b, atol=1e-6)
    for n, p in model.named_parameters():
        assert torch.allclose(p.grad, g0[n], atol=1e-6, rtol=1e-5), n
    with torch.no_grad():
        full = model.hidden_states(x)
        chunked = model.hidden_states_chunked(x, 16)
    assert torch.allclose(full, chunked, atol=2e-5, rtol=1e-4)


def test_checkpoint_round_trip_and_router_freeze(tmp_path):
    cfg, model, hf = _pair(seed=7)
    save_hf_model(model, str(tmp_path / "ours"))
    c = json.load(open(tmp_path / "ours" / "config.json"))
    assert c["model_type"] == "mixtral" and c["num_local_experts"] == 4 and c["architectures"] == ["MixtralForCausalLM"]
    back = load_hf_model(str(tmp_path / "ours"), dtype=torch.float32)
    x = torch.randint(0, 320, (1, 24))
    assert torch.equal(back(x), model(x))
    # HuggingFace reads what this repository wrote, and this repository reads what HuggingFace writes
    hf2 = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ours"), dtype=torch.float32, attn_implementation="eager")
    assert torch.allclose(hf2(x).logits, model(x), atol=3e-4, rtol=1e-3)
    hf2.save_pretrained(str(tmp_path / "theirs"), safe_serialization=True)
    again = load_hf_model(str(tmp_path / "theirs"), dtype=torch.float32)
    assert torch.allclose(again(x), model(x), atol=1e-6)
    names = set(model.to_hf_state_dict())
    assert "model.layers.1.block_sparse_moe.gate.weight" in names
    assert "model.layers.0.block_sparse_moe.experts.3.w2.weight" in names
    # the reference's shipped freeze_layers entry names the router
    frozen = model.apply_freeze(["block_sparse_moe.gate"])
    assert len(frozen) == 2 and not model.layers[0].router.requires_grad and model.layers[0].gate_up_proj.requires_grad
    eng = DistillEngine(model, loss="kl", temperature=1.0, optimizer="adamw", lr=1e-3)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    hb = synthetic_batch(cfg.vocab_size, 2, 32, 8, seed=0)
    l0 = eng.train_step([hb])
    l1 = eng.train_step([hb])
    assert l1 < l0
    assert torch.equal(model.layers[0].router, before["layers.0.router"])
    assert not torch.equal(model.layers[0].gate_up_proj, before["layers.0.gate_up_proj"])
    with pytest.raises(NotImplementedError):
        model.quantize_frozen_linears("nf4")


def test_dense_configs_refuse_experts_and_mixtral_needs_them():
    with pytest.raises(NotImplementedError):
        LlamaConfig.from_hf_dict(dict(_base(), model_type="llama", num_local_experts=4))
    with pytest.raises(ValueError):
        LlamaConfig.from_hf_dict(dict(_base(), model_type="mixtral"))
    cfg = LlamaConfig.from_hf_dict(dict(_base(), model_type="mixtral", num_local_experts=8, num_experts_per_tok=2,
                                        router_aux_loss_coef=0.02))
    assert cfg.num_local_experts == 8 and cfg.extra["router_aux_loss_coef"] == 0.02
    assert cfg.num_params() > LlamaConfig(**_base()).num_params() * 3


def test_command_line_with_a_mixtral_student_and_teacher(tmp_path):
    """Collect from a dense and a mixture-of-experts teacher, train a mixture-of-experts student with the router frozen
    (the reference's shipped ``freeze_layers``), end to end through the command line on CPU."""
    import os
    from llm_distillery_b200 import cli
    from llm_distillery_b200.ckpt.hf import load_hf_state_dict
    from llm_distillery_b200.models.llama import preset
    from llm_distillery_b200.utils import synthetic
    root = str(tmp_path)
    os.environ["B200_NO_PROGRESS"] = "1"
    tok = os.path.join(root, "tok")
    synthetic.make_tokenizer(tok, 400)
    kw = dict(vocab_size=512, hidden_size=64, intermediate_size=176, max_position_embeddings=512)
    moe = dict(kw, model_type="mixtral", num_local_experts=4, num_experts_per_tok=2, intermediate_size=88)
    synthetic.make_model_dir(os.path.join(root, "teachers", "dense"), preset("plumbing-teacher", **kw), tok, seed=1, batch_size=4)
    synthetic.make_model_dir(os.path.join(root, "teachers", "sparse"), preset("plumbing-teacher", **moe), tok, seed=5, batch_size=3)
    synthetic.make_model_dir(os.path.join(root, "student"), preset("plumbing-student", **moe), tok, seed=2)
    synthetic.make_dataset(os.path.join(root, "train.jsonl"), 7, seed=3)
    synthetic.make_dataset(os.path.join(root, "val.jsonl"), 2, seed=4)
    conf = {"dataset_path": os.path.join(root, "train.jsonl"), "validation_dataset_path": os.path.join(root, "val.jsonl"),
            "teacher_models_folder": os.path.join(root, "teachers"), "student_path": os.path.join(root, "student"),
            "cache_folder": os.path.join(root, "cache"), "context_len": 96, "crop_distr_to_size": 400, "save_topK": 20,
            "enable_topK": True, "device": "cpu", "num_epochs": 1, "num_warmup_steps": 1, "batch_size": 2,
            "grad_accum_batches": 1, "lr": 1e-3, "optimizer": "adamw", "data_order": "sorted",
            "training_precision": "fp32", "freeze_layers": ["block_sparse_moe.gate"], "loss": "reference",
            "max_cache_size_gb": 320}
    path = os.path.join(root, "config.json")
    with open(path, "w") as f:
        json.dump(conf, f)
    out = cli.main(["--config", path])
    assert out["trained_samples"] == 7 and out["tokens_collected"] > 0
    trained = os.path.join(root, "cache", "student", "trained")
    final = [d for d in os.listdir(trained) if d.endswith("final")][0]
    sd, init = load_hf_state_dict(os.path.join(trained, final)), load_hf_state_dict(os.path.join(root, "student"))
    moved = {k: float((sd[k].float() - init[k].float()).abs().max()) for k in init}
    assert all(m == 0.0 for k, m in moved.items() if "block_sparse_moe.gate" in k)
    assert any(m > 0 for k, m in moved.items() if ".experts." in k)
    assert json.load(open(os.path.join(trained, final, "config.json")))["model_type"] == "mixtral"


def test_the_console_reports_what_the_workers_are_busy_with():
    """The status postfixes of the reference's progress bars (classes/student/model.py:81-85 and its call sites,
    classes/teacher/model.py:81-99): the command-line run above went through all of them."""
    from llm_distillery_b200.obs import console
    seen = console.status_history()
    for text in ("Loading model...", "Generating...", "Writing rows...", "Saving model at step final...",
                 "Unloading model..."):
        assert text in seen, (text, seen[-20:])
    assert any(t.startswith("Loading dense") or t.startswith("Loading sparse") for t in seen)
    assert console.last_status() == ""


@pytest.mark.parametrize("renorm", [False, True])
def test_qwen3_moe_matches_huggingface(tmp_path, renorm):
    """Qwen3-MoE: per-head q/k norms, experts of their own width, router weights with or without renormalisation."""
    d = dict(_base(), model_type="qwen3_moe", head_dim=32, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=48,
             norm_topk_prob=renorm, decoder_sparse_step=1, mlp_only_layers=[], use_sliding_window=False)
    cfg = LlamaConfig.from_hf_dict(d)
    assert cfg.num_local_experts == 4 and cfg.intermediate_size == 48 and cfg.qk_norm and cfg.moe_renormalize == renorm
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=9)
    with torch.no_grad():
        for l in model.layers:
            l.router.mul_(30.0)
            l.q_norm.uniform_(0.5, 1.5)
    hf_kw = {k: v for k, v in d.items() if k != "model_type"}
    hf = tr.Qwen3MoeForCausalLM(tr.Qwen3MoeConfig(**hf_kw, attn_implementation="eager", tie_word_embeddings=False)).float()
    sd = model.to_hf_state_dict()
    own = hf.state_dict()
    if not all(k in own for k in sd):          # newer releases stack the experts
        f = cfg.intermediate_size
        packed = {k: v for k, v in sd.items() if ".experts." not in k}
        for li in range(cfg.num_hidden_layers):
            pre = f"model.layers.{li}.mlp.experts."
            packed[pre + "gate_up_proj"] = torch.stack([torch.cat([sd[f"{pre}{e}.gate_proj.weight"],
                                                                   sd[f"{pre}{e}.up_proj.weight"]]) for e in range(4)])
            packed[pre + "down_proj"] = torch.stack([sd[f"{pre}{e}.down_proj.weight"] for e in range(4)])
        sd = packed
    res = hf.load_state_dict({k: v.clone() for k, v in sd.items()}, strict=False)
    assert not res.unexpected_keys and not [k for k in res.missing_keys if "rotary" not in k], res
    x = torch.randint(0, 320, (2, 48))
    ours, ref = model(x), hf(x).logits
    assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (ours - ref).abs().max()
    tgt = torch.randint(0, 320, (2 * 48,))
    torch.nn.functional.cross_entropy(ours.reshape(-1, 320), tgt).backward()
    torch.nn.functional.cross_entropy(ref.reshape(-1, 320), tgt).backward()
    hf_grads = {n: p.grad for n, p in hf.named_parameters()}
    f = cfg.intermediate_size
    for n, p, sl in model.named_hf_parameters():
        g = p.grad if sl is None else p.grad[sl]
        if n in hf_grads:
            want = hf_grads[n]
        else:
            pre, rest = n.split("mlp.experts.")
            e, which = int(rest.split(".")[0]), rest.split(".")[1]
            if which == "down_proj":
                want = hf_grads[pre + "mlp.experts.down_proj"][e]
            else:
                gu = hf_grads[pre + "mlp.experts.gate_up_proj"][e]
                want = gu[:f] if which == "gate_proj" else gu[f:]
        assert torch.allclose(g, want, atol=2e-5, rtol=2e-3), (n, (g - want).abs().max())
    # checkpoints both ways; the dense FFN width of the source config survives
    save_hf_model(model, str(tmp_path / "ours"))
    c = json.load(open(tmp_path / "ours" / "config.json"))
    assert c["model_type"] == "qwen3_moe" and c["num_experts"] == 4 and c["moe_intermediate_size"] == 48
    assert c["intermediate_size"] == 136 and c["norm_topk_prob"] == renorm and "num_local_experts" not in c
    hf2 = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ours"), dtype=torch.float32, attn_implementation="eager")
    assert torch.allclose(hf2(x).logits, ref, atol=3e-4, rtol=1e-3)
    hf.save_pretrained(str(tmp_path / "theirs"), safe_serialization=True)
    back = load_hf_model(str(tmp_path / "theirs"), dtype=torch.float32)
    assert back.cfg.model_type == "qwen3_moe" and torch.allclose(back(x), ref, atol=3e-4, rtol=1e-3)
    with pytest.raises(NotImplementedError):
        LlamaConfig.from_hf_dict(dict(d, mlp_only_layers=[0]))


@pytest.mark.parametrize("renorm,recompute", [(False, False), (True, True)])
def test_qwen2_moe_matches_huggingface(tmp_path, renorm, recompute):
    """Qwen2-MoE: Qwen2's attention (bias on q, k, v), routed experts and a dense shared expert whose output is scaled
    per token by a sigmoid gate - logits and every gradient against HuggingFace, with and without recomputation."""
    d = dict(_base(), model_type="qwen2_moe", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=48,
             shared_expert_intermediate_size=80, norm_topk_prob=renorm, decoder_sparse_step=1, mlp_only_layers=[],
             use_sliding_window=False)
    cfg = LlamaConfig.from_hf_dict(d)
    assert cfg.num_local_experts == 4 and cfg.intermediate_size == 48 and cfg.shared_expert_intermediate_size == 80
    assert cfg.attention_bias and not cfg.qk_norm and cfg.moe_renormalize == renorm
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=10)
    assert sum(p.numel() for p in model.parameters()) == cfg.num_params()
    with torch.no_grad():
        for l in model.layers:
            l.router.mul_(30.0)
            l.shared_expert_gate.mul_(40.0)        # gates away from one half
    model.grad_checkpointing = recompute
    hf_kw = {k: v for k, v in d.items() if k != "model_type"}
    hf = tr.Qwen2MoeForCausalLM(tr.Qwen2MoeConfig(**hf_kw, attn_implementation="eager", tie_word_embeddings=False)).float()
    sd = model.to_hf_state_dict()
    own = hf.state_dict()
    if not all(k in own for k in sd):          # newer releases stack the experts
        packed = {k: v for k, v in sd.items() if ".experts." not in k}
        for li in range(cfg.num_hidden_layers):
            pre = f"model.layers.{li}.mlp.experts."
            packed[pre + "gate_up_proj"] = torch.stack([torch.cat([sd[f"{pre}{e}.gate_proj.weight"],
                                                                   sd[f"{pre}{e}.up_proj.weight"]]) for e in range(4)])
            packed[pre + "down_proj"] = torch.stack([sd[f"{pre}{e}.down_proj.weight"] for e in range(4)])
        sd = packed
    res = hf.load_state_dict({k: v.clone() for k, v in sd.items()}, strict=False)
    assert not res.unexpected_keys and not [k for k in res.missing_keys if "rotary" not in k], res
    x = torch.randint(0, 320, (2, 48))
    ours, ref = model(x), hf(x).logits
    assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (ours - ref).abs().max()
    tgt = torch.randint(0, 320, (2 * 48,))
    torch.nn.functional.cross_entropy(ours.reshape(-1, 320), tgt).backward()
    torch.nn.functional.cross_entropy(ref.reshape(-1, 320), tgt).backward()
    hf_grads = {n: p.grad for n, p in hf.named_parameters()}
    f = cfg.intermediate_size
    seen_shared = 0
    for n, p, sl in model.named_hf_parameters():
        g = p.grad if sl is None else p.grad[sl]
        if n in hf_grads:
            want = hf_grads[n]
            seen_shared += "shared_expert" in n
        else:
            pre, rest = n.split("mlp.experts.")
            e, which = int(rest.split(".")[0]), rest.split(".")[1]
            if which == "down_proj":
                want = hf_grads[pre + "mlp.experts.down_proj"][e]
            else:
                gu = hf_grads[pre + "mlp.experts.gate_up_proj"][e]
                want = gu[:f] if which == "gate_proj" else gu[f:]
        assert torch.allclose(g, want, atol=2e-5, rtol=2e-3), (n, (g - want).abs().max())
    assert seen_shared == 4 * cfg.num_hidden_layers
    # the inference path (chunked prefill) runs the shared expert too
    model.grad_checkpointing = False
    with torch.no_grad():
        hs = model.hidden_states_chunked(x, 16)
        assert torch.allclose(torch.nn.functional.linear(hs, model.lm_head).view(2, 48, -1), ref, atol=3e-4, rtol=1e-3)
    # checkpoints both ways
    save_hf_model(model, str(tmp_path / "ours"))
    c = json.load(open(tmp_path / "ours" / "config.json"))
    assert c["model_type"] == "qwen2_moe" and c["num_experts"] == 4 and c["shared_expert_intermediate_size"] == 80
    assert c["intermediate_size"] == 136 and c["moe_intermediate_size"] == 48 and "num_local_experts" not in c
    hf2 = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ours"), dtype=torch.float32, attn_implementation="eager")
    assert torch.allclose(hf2(x).logits, ref, atol=3e-4, rtol=1e-3)
    hf.save_pretrained(str(tmp_path / "theirs"), safe_serialization=True)
    back = load_hf_model(str(tmp_path / "theirs"), dtype=torch.float32)
    assert back.cfg.model_type == "qwen2_moe" and torch.allclose(back(x), ref, atol=3e-4, rtol=1e-3)
    for bad in (dict(mlp_only_layers=[0]), dict(decoder_sparse_step=2), dict(qkv_bias=False)):
        with pytest.raises(NotImplementedError):
            LlamaConfig.from_hf_dict(dict(d, **bad))
    with pytest.raises(NotImplementedError):
        LlamaConfig.from_hf_dict(dict(_base(), model_type="llama", shared_expert_intermediate_size=64))


@pytest.mark.parametrize("recompute", [False, True])
def test_olmoe_matches_huggingface(tmp_path, recompute):
    """OLMoE: Llama layers whose q/k norms cover the whole projections, every MLP a mixture of experts without
    renormalised router weights."""
    torch.manual_seed(3)
    hf = tr.OlmoeForCausalLM(tr.OlmoeConfig(**{k: v for k, v in _base().items() if k != "rope_theta"}, num_experts=4,
                                            num_experts_per_tok=2, pad_token_id=0, attn_implementation="eager",
                                            tie_word_embeddings=False)).float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.uniform_(0.5, 1.5)
            elif n.endswith("mlp.gate.weight"):
                p.mul_(30.0)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    model = load_hf_model(str(tmp_path / "hf"), dtype=torch.float32)
    cfg = model.cfg
    assert cfg.model_type == "olmoe" and cfg.qk_norm_full and not cfg.sandwich and cfg.num_local_experts == 4
    assert not cfg.moe_renormalize
    assert sum(p.numel() for p in model.parameters()) == cfg.num_params() == sum(p.numel() for p in hf.parameters())
    model.grad_checkpointing = recompute
    x = torch.randint(1, 320, (2, 48))
    ours, ref = model(x), hf(x).logits
    assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (ours - ref).abs().max()
    tgt = torch.randint(0, 320, (2 * 48,))
    torch.nn.functional.cross_entropy(ours.reshape(-1, 320), tgt).backward()
    torch.nn.functional.cross_entropy(ref.reshape(-1, 320), tgt).backward()
    hf_grads = {n: p.grad for n, p in hf.named_parameters()}
    f = cfg.intermediate_size
    for n, p, sl in model.named_hf_parameters():
        g = p.grad if sl is None else p.grad[sl]
        if n in hf_grads:
            want = hf_grads[n]
        else:
            pre, rest = n.split("mlp.experts.")
            e, which = int(rest.split(".")[0]), rest.split(".")[1]
            if which == "down_proj":
                want = hf_grads[pre + "mlp.experts.down_proj"][e]
            else:
                gu = hf_grads[pre + "mlp.experts.gate_up_proj"][e]
                want = gu[:f] if which == "gate_proj" else gu[f:]
        assert torch.allclose(g, want, atol=2e-5, rtol=2e-3), (n, (g - want).abs().max())
    model.grad_checkpointing = False
    with torch.no_grad():
        hs = model.hidden_states_chunked(x, 16)
        assert torch.allclose(torch.nn.functional.linear(hs, model.lm_head).view(2, 48, -1), ref, atol=3e-4, rtol=1e-3)
    save_hf_model(model, str(tmp_path / "ours"))
    hf2 = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ours"), dtype=torch.float32, attn_implementation="eager")
    assert type(hf2) is tr.OlmoeForCausalLM and torch.allclose(hf2(x).logits, ref, atol=3e-4, rtol=1e-3)


@pytest.mark.parametrize("family,recompute", [("granitemoe", False), ("granitemoeshared", False), ("granitemoeshared", True)])
def test_granite_moe_matches_huggingface(tmp_path, family, recompute):
    """Granite MoE: Granite's four multipliers around Mixtral-style experts (stacked tensors in the checkpoint); the
    shared variant adds a dense MLP to every token's expert output, ungated."""
    cls, ccls = ((tr.GraniteMoeForCausalLM, tr.GraniteMoeConfig) if family == "granitemoe"
                 else (tr.GraniteMoeSharedForCausalLM, tr.GraniteMoeSharedConfig))
    extra = dict(shared_intermediate_size=80) if family == "granitemoeshared" else {}
    torch.manual_seed(5)
    hf = cls(ccls(**{k: v for k, v in _base().items() if k != "rope_theta"}, num_local_experts=4, num_experts_per_tok=2,
                  embedding_multiplier=6.0, attention_multiplier=0.2, residual_multiplier=0.4, logits_scaling=3.0,
                  pad_token_id=0, attn_implementation="eager", tie_word_embeddings=False, **extra)).float()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.uniform_(0.5, 1.5)
            elif "router" in n:
                p.mul_(30.0)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    model = load_hf_model(str(tmp_path / "hf"), dtype=torch.float32)
    cfg = model.cfg
    assert cfg.model_type == family and cfg.num_local_experts == 4 and cfg.residual_multiplier == 0.4
    assert cfg.shared_expert_intermediate_size == (80 if extra else 0) and not cfg.shared_expert_gated
    assert sum(p.numel() for p in model.parameters()) == cfg.num_params() == sum(p.numel() for p in hf.parameters())
    model.grad_checkpointing = recompute
    x = torch.randint(1, 320, (2, 48))
    ours, ref = model(x), hf(x).logits
    assert torch.allclose(ours, ref, atol=3e-4, rtol=1e-3), (ours - ref).abs().max()
    tgt = torch.randint(0, 320, (2 * 48,))
    torch.nn.functional.cross_entropy(ours.reshape(-1, 320), tgt).backward()
    torch.nn.functional.cross_entropy(ref.reshape(-1, 320), tgt).backward()
    hf_grads = {n: p.grad for n, p in hf.named_parameters()}
    ours_g = {n: (p.grad if sl is None else p.grad[sl]) for n, p, sl in model.named_hf_parameters()}
    assert set(ours_g) == set(hf_grads)
    for n, g in ours_g.items():
        assert torch.allclose(g, hf_grads[n], atol=2e-5, rtol=2e-3), (n, (g - hf_grads[n]).abs().max())
    model.grad_checkpointing = False
    with torch.no_grad():
        hs = model.hidden_states_chunked(x, 16)
        assert torch.allclose(torch.nn.functional.linear(hs, model.lm_head).view(2, 48, -1), ref, atol=3e-4, rtol=1e-3)
    save_hf_model(model, str(tmp_path / "ours"))
    hf2 = tr.AutoModelForCausalLM.from_pretrained(str(tmp_path / "ours"), dtype=torch.float32, attn_implementation="eager")
    assert type(hf2) is cls and torch.allclose(hf2(x).logits, ref, atol=3e-4, rtol=1e-3)
