"""The command line under many settings of its configuration keys, single process on CPU: every case collects, trains
and validates without error; a few are checked further (full-vocabulary rows, frozen tensors, saved files)."""
import json
import math
import os

import numpy as np
import pytest

from llm_distillery_b200 import cli
from llm_distillery_b200.ckpt.hf import load_hf_state_dict
from llm_distillery_b200.data.h5store import H5Store
from llm_distillery_b200.models.llama import preset
from llm_distillery_b200.utils import synthetic

CASES = {
    "full distributions": {"enable_topK": False},
    "full distributions, weighted reference loss": {"enable_topK": False, "loss": "reference"},
    "8-bit AdamW, cosine": {"optimizer": "adamw8bit", "lr_scheduler": "cosine"},
    "RMSprop, linear": {"optimizer": "rmsprop", "lr_scheduler": "linear"},
    "Adagrad, constant with warm-up": {"optimizer": "adagrad", "lr_scheduler": "constant_with_warmup"},
    "reverse KL at T = 3": {"loss": "rkl", "temperature": 3.0},
    "JSD": {"loss": "jsd"},
    "no validation set": {"validation_dataset_path": ""},
    "frozen MLPs": {"freeze_layers": [".mlp."]},
    "bf16 on CPU": {"training_precision": "bf16"},
    "4bit: frozen NF4 decoder matrices": {"training_precision": "4bit"},
    "8bit: frozen int8 decoder matrices": {"training_precision": "8bit"},
    # the combination the reference ships in its config.json (a router entry in freeze_layers matches nothing here)
    "4bit with the reference's shipped optimizer, schedule and freeze list": {
        "training_precision": "4bit", "optimizer": "adamw8bit", "lr_scheduler": "wsd", "decay_start": 0.9, "alpha": 2,
        "freeze_layers": [".block_sparse_moe.gate"], "loss": "reference", "grad_accum_batches": 2,
        "validate_every_n_epochs": 0.5},
    "shuffled, checkpointing, accumulation of 3": {"data_order": "shuffle", "grad_checkpointing": True, "grad_accum_batches": 3},
    "native order, context 48": {"data_order": "native", "context_len": 48},
    "top-K above the crop": {"save_topK": 600},
    "crop and top-K above the vocabulary": {"crop_distr_to_size": 32000, "save_topK": 600},
    "every range is content, one big batch": {"save_sys_range": True, "save_user_range": True, "batch_size": 64,
                                              "num_warmup_steps": 0},      # the single step is not a warm-up step
    "two epochs, checkpoint per epoch, final state": {"num_epochs": 2, "save_student_every_n_epochs": 1, "save_final_state": True},
}


@pytest.fixture(scope="module")
def world(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("variants"))
    os.environ["B200_NO_PROGRESS"] = "1"
    tok = os.path.join(root, "tok")
    synthetic.make_tokenizer(tok, 400)
    kw = dict(vocab_size=512, hidden_size=64, intermediate_size=176, max_position_embeddings=512)
    synthetic.make_model_dir(os.path.join(root, "teachers", "teacher_a"), preset("plumbing-teacher", **kw), tok, seed=1, batch_size=4)
    synthetic.make_model_dir(os.path.join(root, "teachers", "teacher_b"), preset("plumbing-teacher", **kw), tok, seed=5, batch_size=3)
    synthetic.make_model_dir(os.path.join(root, "student"), preset("plumbing-student", **kw), tok, seed=2)
    synthetic.make_dataset(os.path.join(root, "train.jsonl"), 9, seed=3)
    synthetic.make_dataset(os.path.join(root, "val.jsonl"), 3, seed=4)
    base = {"dataset_path": os.path.join(root, "train.jsonl"), "validation_dataset_path": os.path.join(root, "val.jsonl"),
            "teacher_models_folder": os.path.join(root, "teachers"), "student_path": os.path.join(root, "student"),
            "context_len": 96, "crop_distr_to_size": 400, "save_topK": 20, "enable_topK": True, "device": "cpu",
            "num_epochs": 1, "num_warmup_steps": 2, "batch_size": 2, "grad_accum_batches": 1, "lr": 1e-3,
            "optimizer": "adamw", "data_order": "sorted", "training_precision": "fp32", "freeze_layers": [], "loss": "kl",
            "max_cache_size_gb": 320}
    return root, base


@pytest.mark.parametrize("name", list(CASES))
def test_cli_case(world, name):
    root, base = world
    cache = os.path.join(root, "cache_" + "".join(ch if ch.isalnum() else "_" for ch in name))
    conf = dict(base, cache_folder=cache, **CASES[name])
    path = cache + ".json"
    with open(path, "w") as f:
        json.dump(conf, f)
    out = cli.main(["--config", path])
    assert out["trained_samples"] == 9 * conf["num_epochs"] and out["tokens_collected"] > 0
    val = out.get("last_validation") or {}
    if conf["validation_dataset_path"]:
        assert val and all(math.isfinite(v) for v in val.values()), val
    else:
        assert not val
    st = H5Store(os.path.join(cache, "dataset"))
    ids = st.get_dataset_ids()
    assert len(ids) == 9
    v, ix = st.load_id(ids[0])
    if conf["enable_topK"]:
        keep = min(conf["save_topK"], conf["crop_distr_to_size"], 512)      # never more values than the vocabulary has
        assert v.shape[1] == keep and ix is not None and ix.max() < min(conf["crop_distr_to_size"], 512)
        assert (np.exp(v).sum(-1) <= 2.0 + 1e-2).all()                   # two teachers' probabilities summed
    else:
        assert v.shape[1] == 400 and ix is None                          # whole cropped distribution, no index table
    st.close()
    trained = os.path.join(cache, "student", "trained")
    finals = [d for d in os.listdir(trained) if d.endswith("final")]
    assert len(finals) == 1
    sd, init = load_hf_state_dict(os.path.join(trained, finals[0])), load_hf_state_dict(os.path.join(root, "student"))
    moved = {k: float((sd[k].float() - init[k].float()).abs().max()) for k in init}
    assert max(moved.values()) > 1e-5
    if name[:4] in ("4bit", "8bit"):
        # the decoder matrices are frozen at their quantised values: what is saved differs from the checkpoint by the
        # quantisation error only, and embeddings / norms / head are what trained
        from llm_distillery_b200.ops import quant
        w0 = init["model.layers.0.mlp.down_proj.weight"].float()
        q = (quant.quantize_nf4 if name[0] == "4" else quant.quantize_int8)(w0)
        assert np.allclose(sd["model.layers.0.mlp.down_proj.weight"].float().numpy(),
                           quant.dequantize_reference(q).numpy(), atol=1e-6)
        assert moved["model.embed_tokens.weight"] > 1e-5 and moved["model.norm.weight"] > 0
    if name == "frozen MLPs":
        assert all(m == 0.0 for k, m in moved.items() if ".mlp." in k) and any(m > 0 for k, m in moved.items() if "self_attn" in k)
    if name.startswith("two epochs"):
        assert len(os.listdir(trained)) == 2                              # the epoch-1 checkpoint and the final one
        assert {"model_state.pt", "optimizer_state.pt", "scheduler_state.pt", "trainer_state.json"} <= set(
            os.listdir(os.path.join(cache, "student", "states")))


FAMILIES = {
    "qwen2_moe": dict(model_type="qwen2_moe", num_local_experts=4, num_experts_per_tok=2, intermediate_size=48,
                      shared_expert_intermediate_size=80, attention_bias=True, moe_renormalize=False),
    "qwen3_moe": dict(model_type="qwen3_moe", num_local_experts=4, num_experts_per_tok=2, intermediate_size=48,
                      qk_norm=True, head_dim_override=32),
    "olmoe": dict(model_type="olmoe", num_local_experts=4, num_experts_per_tok=2, intermediate_size=48,
                  qk_norm_full=True, moe_renormalize=False),
    "granitemoeshared": dict(model_type="granitemoeshared", num_local_experts=4, num_experts_per_tok=2,
                             intermediate_size=48, shared_expert_intermediate_size=80, shared_expert_gated=False,
                             embedding_multiplier=6.0, attention_multiplier=0.2, residual_multiplier=0.4, logits_scaling=3.0),
    "smollm3": dict(model_type="smollm3", no_rope_layers=[1, 0]),
    "phi3, three quarters of a head rotate": dict(model_type="phi3", partial_rotary_factor=0.75),
    "granite": dict(model_type="granite", embedding_multiplier=6.0, attention_multiplier=0.2, residual_multiplier=0.4,
                    logits_scaling=3.0),
    "qwen3": dict(model_type="qwen3", qk_norm=True),
    "olmo2": dict(model_type="olmo2", pre_norm=False, post_norm=True, qk_norm_full=True),
    "glm4": dict(model_type="glm4", post_norm=True, attention_bias=True, partial_rotary_factor=0.5, rope_interleaved=True,
                 head_dim_override=32),
    "glm": dict(model_type="glm", attention_bias=True, partial_rotary_factor=0.5, rope_interleaved=True),
    "exaone4, windowed and global layers": dict(model_type="exaone4", pre_norm=False, post_norm=True, qk_norm=True,
                                                no_rope_layers=[1, 0], window_layers=[1, 0], sliding_window=48),
    "mistral, window shorter than the context": dict(model_type="mistral", sliding_window=40),
    "gemma3_text": dict(model_type="gemma3_text", mlp_act="gelu_tanh", norm_plus_one=True, embedding_multiplier=8.0,
                        embedding_multiplier_rounded=True, post_norm=True, qk_norm=True, sliding_window=40,
                        window_layers=[1, 0], rope_local_theta=10000.0, head_dim_override=32, tie_word_embeddings=True),
    "helium": dict(model_type="helium", rope_interleaved=True),
    "ernie4_5": dict(model_type="ernie4_5", rope_interleaved=True),
    "seed_oss": dict(model_type="seed_oss", attention_bias=True, head_dim_override=32),
    "hunyuan_v1_dense": dict(model_type="hunyuan_v1_dense", qk_norm=True, qk_norm_after_rope=True,
                             rope_scaling={"rope_type": "dynamic", "alpha": 1000.0, "factor": 1.0}),
}


@pytest.mark.parametrize("family", list(FAMILIES))
def test_cli_with_teacher_and_student_of_a_model_family(tmp_path, family):
    """Collection, training, validation and the saved checkpoint with both models of one family; the saved student
    loads again and HuggingFace's config class for the family accepts its config.json."""
    import dataclasses
    import transformers as tr
    from llm_distillery_b200.ckpt.hf import load_hf_model
    root = str(tmp_path)
    os.environ["B200_NO_PROGRESS"] = "1"
    tok = os.path.join(root, "tok")
    synthetic.make_tokenizer(tok, 400)
    kw = dict(vocab_size=512, hidden_size=64, intermediate_size=176, max_position_embeddings=512, num_hidden_layers=2)
    fam = FAMILIES[family]
    t_cfg = dataclasses.replace(preset("plumbing-teacher", **kw), **fam)
    s_cfg = dataclasses.replace(preset("plumbing-student", **kw), **fam)
    synthetic.make_model_dir(os.path.join(root, "teachers", "teacher_a"), t_cfg, tok, seed=1, batch_size=4)
    synthetic.make_model_dir(os.path.join(root, "student"), s_cfg, tok, seed=2)
    synthetic.make_dataset(os.path.join(root, "train.jsonl"), 6, seed=3)
    synthetic.make_dataset(os.path.join(root, "val.jsonl"), 2, seed=4)
    cache = os.path.join(root, "cache")
    conf = {"dataset_path": os.path.join(root, "train.jsonl"), "validation_dataset_path": os.path.join(root, "val.jsonl"),
            "teacher_models_folder": os.path.join(root, "teachers"), "student_path": os.path.join(root, "student"),
            "context_len": 96, "crop_distr_to_size": 400, "save_topK": 20, "enable_topK": True, "device": "cpu",
            "num_epochs": 1, "num_warmup_steps": 1, "batch_size": 2, "grad_accum_batches": 1, "lr": 1e-3,
            "optimizer": "adamw", "data_order": "sorted", "training_precision": "fp32", "freeze_layers": [], "loss": "kl",
            "max_cache_size_gb": 320, "cache_folder": cache}
    path = os.path.join(root, "config.json")
    with open(path, "w") as f:
        json.dump(conf, f)
    out = cli.main(["--config", path])
    assert out["trained_samples"] == 6 and out["tokens_collected"] > 0
    assert all(math.isfinite(v) for v in out["last_validation"].values())
    trained = os.path.join(cache, "student", "trained")
    final = os.path.join(trained, [d for d in os.listdir(trained) if d.endswith("final")][0])
    back = load_hf_model(final, dtype=None)
    for k, v in fam.items():
        assert getattr(back.cfg, k) == v, (k, getattr(back.cfg, k))
    init = load_hf_state_dict(os.path.join(root, "student"))
    sd = load_hf_state_dict(final)
    assert set(sd) == set(init) and max(float((sd[k].float() - init[k].float()).abs().max()) for k in init) > 1e-5
    hf_cfg = tr.AutoConfig.from_pretrained(final)
    assert hf_cfg.model_type == fam["model_type"]
