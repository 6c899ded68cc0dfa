"""The whole command-line pipeline on one GPU in bf16: tokenise, collect the teacher's top-K rows into the HDF5 store,
train the student against them, validate, save the HuggingFace-layout checkpoint and the trainer state; a second run
finds nothing to collect and resumes from the saved state."""
import json
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_cli_collect_train_checkpoint_on_gpu(tmp_path, monkeypatch):
    from llm_distillery_b200 import cli
    from llm_distillery_b200.ckpt.hf import load_hf_state_dict
    from llm_distillery_b200.data.h5store import H5Store
    from llm_distillery_b200.models.llama import preset
    from llm_distillery_b200.ops import _lib
    from llm_distillery_b200.utils import synthetic
    monkeypatch.setenv("B200_NO_PROGRESS", "1")
    monkeypatch.delenv("WORLD_SIZE", raising=False)
    root = str(tmp_path)
    on_gpu = torch.cuda.is_available()      # the body also runs on a CPU box when the marker is selected by hand
    tok = os.path.join(root, "tok")
    synthetic.make_tokenizer(tok, 400)
    kw = dict(vocab_size=512, hidden_size=256, intermediate_size=688, max_position_embeddings=512)
    synthetic.make_model_dir(os.path.join(root, "teachers", "teacher_a"), preset("plumbing-teacher", **kw), tok, seed=1,
                             batch_size=4)
    synthetic.make_model_dir(os.path.join(root, "student"), preset("plumbing-student", **kw), tok, seed=2)
    synthetic.make_dataset(os.path.join(root, "train.jsonl"), 12, seed=3)
    synthetic.make_dataset(os.path.join(root, "val.jsonl"), 4, seed=4)
    conf = {"cache_folder": os.path.join(root, "cache"), "dataset_path": os.path.join(root, "train.jsonl"),
            "validation_dataset_path": os.path.join(root, "val.jsonl"), "teacher_models_folder": os.path.join(root, "teachers"),
            "student_path": os.path.join(root, "student"), "context_len": 128, "crop_distr_to_size": 400, "save_topK": 32,
            "enable_topK": True, "device": "cuda:0" if on_gpu else "cpu", "num_epochs": 3, "num_warmup_steps": 2, "batch_size": 2,
            "grad_accum_batches": 2, "temperature": 2.0, "lr": 2e-3, "optimizer": "adamw", "data_order": "sorted",
            "training_precision": "bf16" if on_gpu else "fp32", "validate_every_n_epochs": 1, "save_student_every_n_epochs": 1,
            "freeze_layers": [], "loss": "kl", "max_cache_size_gb": 320, "save_final_state": True}
    path = os.path.join(root, "config.json")
    with open(path, "w") as f:
        json.dump(conf, f)
    before = _lib.LAUNCH_COUNT[0]
    out = cli.main(["--config", path])
    if on_gpu:
        torch.cuda.synchronize()
        assert _lib.take_device_error() == 0
        assert _lib.LAUNCH_COUNT[0] - before > 200      # the native kernels ran, not a PyTorch fallback
    assert out["trained_samples"] == 36 and out["tokens_collected"] > 0, out
    store = H5Store(os.path.join(root, "cache", "dataset"))
    ids = store.get_dataset_ids()
    assert len(ids) == 12
    vals, idx = store.load_id(ids[0])
    assert vals.shape[1] == 32 and idx.shape == vals.shape and idx.max() < 400
    store.close()
    base = os.path.join(root, "cache", "student", "trained")
    final = [d for d in os.listdir(base) if d.endswith("final")]
    assert len(final) == 1
    trained = load_hf_state_dict(os.path.join(base, final[0]))
    init = load_hf_state_dict(os.path.join(root, "student"))
    assert all(torch.isfinite(v.float()).all() for v in trained.values())
    assert max((trained[k].float() - init[k].float()).abs().max().item() for k in init) > 1e-3
    with open(os.path.join(root, "cache", "metrics.jsonl")) as f:
        recs = [json.loads(line) for line in f if line.strip()]
    val = [r["Val Loss/custom loss"] for r in recs if "Val Loss/custom loss" in r]
    assert len(val) >= 2 and val[-1] < val[0], val      # the student moved towards the teacher
    # second run: nothing to collect; training is already complete
    out2 = cli.main(["--config", path])
    assert out2["tokens_collected"] == 0, out2


def test_two_teachers_are_merged_on_the_device(tmp_path, monkeypatch):
    """Two teachers of one vocabulary: the second teacher's rows are merged into the stored ones by the
    ``topk_merge`` kernel from the store's writer threads; the result equals the NumPy statement of the merge."""
    import numpy as np
    from llm_distillery_b200 import cli
    from llm_distillery_b200.data import h5store
    from llm_distillery_b200.data.h5store import H5Store
    from llm_distillery_b200.models.llama import preset
    from llm_distillery_b200.utils import synthetic
    monkeypatch.setenv("B200_NO_PROGRESS", "1")
    monkeypatch.delenv("WORLD_SIZE", raising=False)
    root = str(tmp_path)
    tok = os.path.join(root, "tok")
    synthetic.make_tokenizer(tok, 400)
    kw = dict(vocab_size=512, hidden_size=256, intermediate_size=688, max_position_embeddings=512)
    for name, seed in (("teacher_a", 1), ("teacher_b", 7)):
        synthetic.make_model_dir(os.path.join(root, "teachers", name), preset("plumbing-teacher", **kw), tok, seed=seed,
                                 batch_size=4)
    synthetic.make_model_dir(os.path.join(root, "student"), preset("plumbing-student", **kw), tok, seed=2)
    synthetic.make_dataset(os.path.join(root, "train.jsonl"), 8, seed=3)
    synthetic.make_dataset(os.path.join(root, "val.jsonl"), 2, seed=4)
    calls = {"device": 0, "host": 0, "pairs": []}
    real = h5store.merge_topk_on

    def spy(device, d_l, d_i, n_l, n_i):
        out = real(device, d_l, d_i, n_l, n_i)
        calls["device" if str(device).startswith("cuda") else "host"] += 1
        if len(calls["pairs"]) < 3:
            calls["pairs"].append((out, h5store.merge_topk(d_l, d_i, n_l, n_i)))
        return out
    monkeypatch.setattr(h5store, "merge_topk_on", spy)
    conf = {"cache_folder": os.path.join(root, "cache"), "dataset_path": os.path.join(root, "train.jsonl"),
            "validation_dataset_path": os.path.join(root, "val.jsonl"), "teacher_models_folder": os.path.join(root, "teachers"),
            "student_path": os.path.join(root, "student"), "context_len": 128, "crop_distr_to_size": 400, "save_topK": 32,
            "enable_topK": True, "device": "cuda:0", "num_epochs": 1, "num_warmup_steps": 0, "batch_size": 2,
            "grad_accum_batches": 1, "temperature": 1.0, "lr": 1e-3, "optimizer": "adamw", "data_order": "sorted",
            "training_precision": "bf16", "validate_every_n_epochs": 1, "save_student_every_n_epochs": 1,
            "freeze_layers": [], "loss": "kl", "max_cache_size_gb": 320}
    path = os.path.join(root, "config.json")
    with open(path, "w") as f:
        json.dump(conf, f)
    out = cli.main(["--config", path])
    assert out["trained_samples"] == 8
    assert calls["device"] >= 8 and calls["host"] == 0, calls          # every conversation of the second teacher
    for (gl, gi), (hl, hi) in calls["pairs"]:
        order_g, order_h = np.argsort(gi, axis=1), np.argsort(hi, axis=1)
        assert np.array_equal(np.take_along_axis(gi, order_g, 1), np.take_along_axis(hi, order_h, 1))
        a, b = np.take_along_axis(gl, order_g, 1), np.take_along_axis(hl, order_h, 1)
        fin = np.isfinite(a) & np.isfinite(b)
        assert np.array_equal(np.isfinite(a), np.isfinite(b))
        worst = np.unravel_index(np.argmax(np.where(fin, np.abs(a - b), 0)), a.shape)
        assert np.allclose(a[fin], b[fin], atol=2e-3), (worst, a[worst], b[worst], np.take_along_axis(gi, order_g, 1)[worst],
                                                        a.shape, gl.dtype, hl.dtype)
    store = H5Store(os.path.join(root, "cache", "dataset"))
    v, ix = store.load_id(store.get_dataset_ids()[0])
    assert v.shape[1] == 32 and np.isfinite(v).all()
    store.close()
