"""The CPU plumbing configuration, at its stated sizes: random-init Llama-style teacher (2 layers) and student
(4 layers), hidden 256, 4 heads, FFN 688, vocab 32000, token ids uniform in [0, 32000), 64 samples of 256 tokens in
batches of 2; teacher top-200 log-probs stored fp16 + indices in HDF5; forward KL at T = 1, AdamW 1e-4, 10 steps,
fp32, single process, seeded. Checks: 64 groups of [255, 200] rows, loss goes down, a rerun is bit-identical, the
checkpoint reloads, and collecting again finds nothing to do."""
import numpy as np
import torch

from llm_distillery_b200.ckpt.hf import load_hf_model, save_hf_model
from llm_distillery_b200.collect.collector import TeacherCollector
from llm_distillery_b200.data.convo import ConvoTokenized
from llm_distillery_b200.data.h5store import H5Store
from llm_distillery_b200.engine.trainer import DistillEngine, HostBatch
from llm_distillery_b200.loss.head import sort_teacher_rows
from llm_distillery_b200.models.llama import build_model, preset

N, L, K, B = 64, 256, 200, 2


def _convos(seed=0):
    rng = np.random.default_rng(seed)
    return [ConvoTokenized(rng.integers(0, 32000, L).astype(np.int64), [(0, L - 1)], 0, False, i, "s") for i in range(N)]


def _collect(store, convos):
    teacher = build_model(preset("plumbing-teacher"), dtype=torch.float32, device="cpu", seed=1)
    col = TeacherCollector(teacher, topk=K, crop_to_size=32000)
    todo = [c for c in convos if store.get_sha(c.origin_convo_id) != c.content_sha]
    for i in range(0, len(todo), B):
        part = todo[i:i + B]
        store.write_batch(col.collect_batch(np.stack([c.tokenized for c in part]), part))
    store.wait()
    return len(todo)


def _train(store, convos, steps=10):
    student = build_model(preset("plumbing-student"), dtype=torch.float32, device="cpu", seed=2)
    eng = DistillEngine(student, loss="kl", temperature=1.0, optimizer="adamw", lr=1e-4)
    losses = []
    first = None
    for s in range(steps + 1):
        part = convos[(s * B) % N:(s * B) % N + B] if s < steps else convos[:B]
        vals, idxs = zip(*[store.load_id(c.origin_convo_id) for c in part])
        ids, logp = sort_teacher_rows(torch.from_numpy(np.concatenate(idxs).astype(np.int64)),
                                      torch.from_numpy(np.concatenate(vals).astype(np.float32)))
        rows = torch.cat([torch.arange(L - 1) + b * L for b in range(B)])
        seg = torch.arange(B).repeat_interleave(L - 1)
        hb = HostBatch(torch.from_numpy(np.stack([c.tokenized for c in part])), ids, logp, seg, B, rows=rows, n_tokens=B * L)
        if s < steps:
            losses.append(float(eng.train_step([hb])))
        else:
            losses.append(float(eng.eval_batch(hb)[0]))     # the first batch again, after the 10 updates
    return student, losses


def test_config1_collect_train_checkpoint_rerun(tmp_path):
    torch.manual_seed(0)
    convos = _convos()
    store = H5Store(str(tmp_path / "ds"))
    assert _collect(store, convos) == N
    ids = store.get_dataset_ids()
    assert len(ids) == N
    v, ix = store.load_id_raw(ids[3])                       # as stored: fp16 values, 32-bit indices
    assert v.shape == (L - 1, K) and v.dtype == np.float16 and ix.shape == (L - 1, K) and ix.max() < 32000
    assert ix.dtype.itemsize == 4
    assert (np.diff(v.astype(np.float32), axis=1) <= 1e-3).all()
    student, losses = _train(store, convos)
    # losses[0] is the first batch before any update, losses[-1] the same batch after the 10 updates
    assert losses[-1] < losses[0], losses
    _, losses2 = _train(store, convos)
    assert losses == losses2                               # seeded, single process: bit-identical rerun
    save_hf_model(student, str(tmp_path / "ckpt"))
    back = load_hf_model(str(tmp_path / "ckpt"), dtype=torch.float32)
    assert torch.equal(back.lm_head, student.lm_head) and torch.equal(back.layers[3].qkv_proj, student.layers[3].qkv_proj)
    assert _collect(store, convos) == 0                     # everything is on disk with matching content hashes
    store.close()
