"""End-to-end CPU plumbing run: synthetic tokenizer + random-init teacher (2 layers) and student (4 layers),
collect top-K into HDF5, train a few optimizer steps, checkpoint; rerun collects nothing and resumes."""
import json
import os

import numpy as np
import pytest
import torch

from llm_distillery_b200 import cli
from llm_distillery_b200.ckpt.hf import load_hf_model
from llm_distillery_b200.data.h5store import H5Store
from llm_distillery_b200.models.llama import preset
from llm_distillery_b200.utils import synthetic


@pytest.fixture(scope="module")
def workspace(tmp_path_factory):
    root = tmp_path_factory.mktemp("plumbing")
    tok = str(root / "tok")
    synthetic.make_tokenizer(tok, 400)
    tcfg = preset("plumbing-teacher", vocab_size=512, hidden_size=64, intermediate_size=176, max_position_embeddings=128)
    scfg = preset("plumbing-student", vocab_size=512, hidden_size=64, intermediate_size=176, max_position_embeddings=128)
    synthetic.make_model_dir(str(root / "teachers" / "teacher_a"), tcfg, tok, seed=1, batch_size=4)
    synthetic.make_model_dir(str(root / "student"), scfg, tok, seed=2)
    synthetic.make_dataset(str(root / "train.jsonl"), 24, seed=3)
    synthetic.make_dataset(str(root / "val.jsonl"), 6, seed=4)
    conf = {"cache_folder": str(root / "cache"), "dataset_path": str(root / "train.jsonl"),
            "validation_dataset_path": str(root / "val.jsonl"), "teacher_models_folder": str(root / "teachers"),
            "student_path": str(root / "student"), "context_len": 96, "crop_distr_to_size": 400, "save_topK": 20,
            "enable_topK": True, "device": "cpu", "num_epochs": 2, "num_warmup_steps": 4, "batch_size": 2,
            "grad_accum_batches": 2, "temperature": 1.0, "lr": 2e-3, "optimizer": "adamw", "data_order": "sorted",
            "training_precision": "fp32", "validate_every_n_epochs": 1, "save_student_every_n_epochs": 1,
            "freeze_layers": [], "loss": "reference", "max_cache_size_gb": 320}
    with open(root / "config.json", "w") as f:
        json.dump(conf, f)
    return root


def test_collect_train_checkpoint_then_rerun_skips_collection(workspace):
    os.environ["B200_NO_PROGRESS"] = "1"
    out = cli.main(["--config", str(workspace / "config.json")])
    assert out["trained_samples"] == 48 and out["tokens_collected"] > 0
    st = H5Store(str(workspace / "cache" / "dataset"))
    ids = st.get_dataset_ids()
    assert len(ids) == 24 and st.get_topk() == 20 and st.get_vocab_family() == "Unknown"
    v, ix = st.load_id(ids[0])
    assert v.shape[1] == 20 and ix.max() < 400 and (np.diff(v, axis=1) <= 1e-3).all()     # sorted descending
    assert abs(np.exp(v[0]).sum()) <= 1.0 + 1e-2
    st.close()
    trained = workspace / "cache" / "student" / "trained"
    folders = sorted(os.listdir(trained))
    assert "student_step_final" in folders and any(f.startswith("student_step_24") for f in folders)
    m = load_hf_model(str(trained / "student_step_final"), dtype=torch.float32)
    m0 = load_hf_model(str(workspace / "student"), dtype=torch.float32)
    assert not torch.equal(m.lm_head, m0.lm_head)
    lines = [json.loads(x) for x in open(workspace / "cache" / "metrics.jsonl") if "step" in x]
    val = [r["Val Loss/custom loss"] for r in lines if "Val Loss/custom loss" in r]
    assert len(val) >= 3 and val[-1] < val[0]
    assert any("Learning Rate" in r for r in lines) and any("Loss/kl_div" in r for r in lines)
    # HF transformers reads the checkpoint folder
    from transformers import AutoModelForCausalLM
    hf = AutoModelForCausalLM.from_pretrained(str(trained / "student_step_final"), torch_dtype=torch.float32)
    x = torch.randint(0, 400, (1, 12))
    assert torch.allclose(hf(x).logits, m(x), atol=2e-4, rtol=1e-3)

    # rerun: nothing to collect (SHA sync), training runs from the data on disk
    out2 = cli.main(["--config", str(workspace / "config.json"), "--num_epochs", "1", "--loss", "kl"])
    assert out2["tokens_collected"] == 0 and out2["trained_samples"] == 24


def test_chunked_mode_and_dataset_edit(workspace):
    os.environ["B200_NO_PROGRESS"] = "1"
    # drop two samples and add one: the store renames / removes / collects only what changed
    rows = [json.loads(x) for x in open(workspace / "train.jsonl")]
    rows = rows[2:] + [{"init": "", "conversations": [{"from": "human", "value": "brand new sample about foxes"},
                                                     {"from": "gpt", "value": "and wizards too"}], "source": "s", "tags": []}]
    with open(workspace / "train2.jsonl", "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    out = cli.main(["--config", str(workspace / "config.json"), "--dataset_path", str(workspace / "train2.jsonl"),
                    "--num_epochs", "1", "--loss", "kl"])
    assert out["tokens_collected"] > 0 and out["trained_samples"] == 23
    st = H5Store(str(workspace / "cache" / "dataset"))
    assert sorted(st.get_dataset_ids()) == list(range(23))
    st.close()
    # tiny cache limit: alternate collect-chunk / train-chunk, trainer state handed over between chunks
    out = cli.main(["--config", str(workspace / "config.json"), "--dataset_path", str(workspace / "train2.jsonl"),
                    "--max_cache_size_gb", "0.00002", "--num_epochs", "1", "--loss", "jsd",
                    "--cache_folder", str(workspace / "cache_chunked")])
    assert out["trained_samples"] == 23
    assert os.path.exists(workspace / "cache_chunked" / "student" / "states" / "trainer_state.json")


def test_stop_request_saves_state_and_the_rerun_ends_like_an_undisturbed_run(tmp_path, monkeypatch):
    """SIGTERM in the middle of training: the step is finished, the trainer state saved, the command returns; the same
    command again takes the run up in the middle of its epoch and ends with the weights of a run that was never
    stopped. A signal outside training still ends the process the old way (not exercised here)."""
    import json
    import signal
    from llm_distillery_b200 import cli
    from llm_distillery_b200.ckpt.hf import load_hf_state_dict
    from llm_distillery_b200.models.llama import preset
    from llm_distillery_b200.models.student import StudentModel
    from llm_distillery_b200.utils import synthetic
    monkeypatch.setenv("B200_NO_PROGRESS", "1")
    root = str(tmp_path)
    tok = os.path.join(root, "tok")
    synthetic.make_tokenizer(tok, 400)
    kw = dict(vocab_size=512, hidden_size=64, intermediate_size=176, max_position_embeddings=512)
    synthetic.make_model_dir(os.path.join(root, "teachers", "teacher_a"), preset("plumbing-teacher", **kw), tok, seed=1, batch_size=4)
    synthetic.make_model_dir(os.path.join(root, "student"), preset("plumbing-student", **kw), tok, seed=2)
    synthetic.make_dataset(os.path.join(root, "train.jsonl"), 8, seed=3)
    synthetic.make_dataset(os.path.join(root, "val.jsonl"), 2, seed=4)
    conf = {"dataset_path": os.path.join(root, "train.jsonl"), "validation_dataset_path": os.path.join(root, "val.jsonl"),
            "teacher_models_folder": os.path.join(root, "teachers"), "student_path": os.path.join(root, "student"),
            "context_len": 96, "crop_distr_to_size": 400, "save_topK": 20, "enable_topK": True, "device": "cpu",
            "num_epochs": 2, "num_warmup_steps": 4, "batch_size": 2, "grad_accum_batches": 1, "lr": 1e-3,
            "optimizer": "adamw", "data_order": "sorted", "training_precision": "fp32", "freeze_layers": [], "loss": "kl"}
    for name in ("stopped", "whole"):
        with open(os.path.join(root, f"{name}.json"), "w") as f:
            json.dump(dict(conf, cache_folder=os.path.join(root, "cache_" + name)), f)
    real, count = StudentModel._optimizer_step, [0]

    def step(self):
        real(self)
        count[0] += 1
        if count[0] == 5:                       # the signal arrives during the fifth of eight steps (second epoch)
            cli.handle_termination(signal.SIGTERM, None)
    monkeypatch.setattr(StudentModel, "_optimizer_step", step)
    out = cli.main(["--config", os.path.join(root, "stopped.json")])
    assert out == {"stopped": True, "trained_samples": 10}
    states = os.listdir(os.path.join(root, "cache_stopped", "student", "states"))
    assert {"model_state.pt", "optimizer_state.pt", "trainer_state.json"} <= set(states)
    monkeypatch.setattr(StudentModel, "_optimizer_step", real)
    out = cli.main(["--config", os.path.join(root, "stopped.json")])
    assert out["trained_samples"] == 16 and out["tokens_collected"] == 0
    out = cli.main(["--config", os.path.join(root, "whole.json")])
    assert out["trained_samples"] == 16

    def final(cache):
        base = os.path.join(root, cache, "student", "trained")
        return load_hf_state_dict(os.path.join(base, [d for d in os.listdir(base) if d.endswith("final")][0]))
    a, b = final("cache_stopped"), final("cache_whole")
    for k in b:
        assert (a[k].float() - b[k].float()).abs().max().item() < 1e-6, k


@pytest.mark.parametrize("teachers,kill_at", [(1, 4), (2, 10)])
def test_collection_killed_half_way_is_continued_not_repeated(tmp_path, monkeypatch, teachers, kill_at):
    """The process dies during collection (here: an exception out of the third batch). What had reached the HDF5 file
    stays; the same command again collects only the conversations that are missing and the store equals a fresh one.
    With two teachers the kill comes while the SECOND is merging: the conversations it had not reached carry the first
    teacher's rows under a marked SHA, are seen as changed by the next run and collected again by both teachers."""
    import json
    from llm_distillery_b200 import cli
    from llm_distillery_b200.collect.collector import TeacherCollector
    from llm_distillery_b200.models.llama import preset
    from llm_distillery_b200.utils import synthetic
    monkeypatch.setenv("B200_NO_PROGRESS", "1")
    root = str(tmp_path)
    tok = os.path.join(root, "tok")
    synthetic.make_tokenizer(tok, 400)
    kw = dict(vocab_size=512, hidden_size=64, intermediate_size=176, max_position_embeddings=512)
    synthetic.make_model_dir(os.path.join(root, "teachers", "teacher_a"), preset("plumbing-teacher", **kw), tok, seed=1, batch_size=2)
    if teachers == 2:
        synthetic.make_model_dir(os.path.join(root, "teachers", "teacher_b"), preset("plumbing-teacher", **kw), tok, seed=7,
                                 batch_size=2)
    synthetic.make_model_dir(os.path.join(root, "student"), preset("plumbing-student", **kw), tok, seed=2)
    synthetic.make_dataset(os.path.join(root, "train.jsonl"), 10, seed=3)
    synthetic.make_dataset(os.path.join(root, "val.jsonl"), 2, seed=4)
    conf = {"dataset_path": os.path.join(root, "train.jsonl"), "validation_dataset_path": os.path.join(root, "val.jsonl"),
            "teacher_models_folder": os.path.join(root, "teachers"), "student_path": os.path.join(root, "student"),
            "context_len": 96, "crop_distr_to_size": 400, "save_topK": 20, "enable_topK": True, "device": "cpu",
            "num_epochs": 1, "num_warmup_steps": 0, "batch_size": 2, "grad_accum_batches": 1, "lr": 1e-3,
            "optimizer": "adamw", "data_order": "sorted", "training_precision": "fp32", "freeze_layers": [], "loss": "kl"}
    for name in ("killed", "fresh"):
        with open(os.path.join(root, f"{name}.json"), "w") as f:
            json.dump(dict(conf, cache_folder=os.path.join(root, "cache_" + name)), f)
    real, calls = TeacherCollector.collect_batch, [0]

    def dying(self, *a, **k):
        calls[0] += 1
        if calls[0] == kill_at:    # one teacher: validation batch + two training batches are through; two teachers:
            # both validation batches, the first teacher's five batches and two of the second teacher's
            raise KeyboardInterrupt("killed")
        return real(self, *a, **k)
    monkeypatch.setattr(TeacherCollector, "collect_batch", dying)
    with pytest.raises(KeyboardInterrupt):
        cli.main(["--config", os.path.join(root, "killed.json")])
    cli.handle_termination(None, None)                       # what the signal handler does on the way out
    monkeypatch.setattr(TeacherCollector, "collect_batch", real)
    partial = H5Store(os.path.join(root, "cache_killed", "dataset"))
    have = len(partial.get_dataset_ids())
    partial.close()
    assert (0 < have < 10) if teachers == 1 else have == 10
    if teachers == 2:
        from llm_distillery_b200.data.convo import PARTIAL_SHA_PREFIX
        partial = H5Store(os.path.join(root, "cache_killed", "dataset"))
        marked = [c for c, sha in partial.get_available_shas().items() if sha.startswith(PARTIAL_SHA_PREFIX)]
        partial.close()
        assert len(marked) == 6                               # four conversations got the second teacher's rows
    out = cli.main(["--config", os.path.join(root, "killed.json")])
    fresh = cli.main(["--config", os.path.join(root, "fresh.json")])
    assert out["trained_samples"] == fresh["trained_samples"] == 10
    assert 0 < out["tokens_collected"] < fresh["tokens_collected"]
    a, b = H5Store(os.path.join(root, "cache_killed", "dataset")), H5Store(os.path.join(root, "cache_fresh", "dataset"))
    assert sorted(a.get_dataset_ids()) == sorted(b.get_dataset_ids()) == list(range(10))
    for cid in range(10):
        va, ia = a.load_id(cid)
        vb, ib = b.load_id(cid)
        assert a.get_sha(cid) == b.get_sha(cid) and np.array_equal(va, vb) and np.array_equal(ia, ib), cid
    a.close()
    b.close()
