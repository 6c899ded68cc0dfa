"""Cross-tokenizer alignment: byte trie, vocabulary map, position pairing, mass remap, two-teacher end-to-end run."""
import json
import os

import numpy as np
import pytest
import torch

from llm_distillery_b200 import cli
from llm_distillery_b200.align import aligner as al
from llm_distillery_b200.data.h5store import H5Store
from llm_distillery_b200.models.llama import preset
from llm_distillery_b200.ops import topk
from llm_distillery_b200.utils import synthetic


@pytest.fixture(scope="module")
def toks(tmp_path_factory):
    root = tmp_path_factory.mktemp("toks")
    a = synthetic.make_tokenizer(str(root / "a"), 400, seed=0)
    b = synthetic.make_tokenizer(str(root / "b"), 700, seed=5, extra_merges_text="quartz sphinx wizard " * 50)
    return root, a, b


def test_trie_and_vocab_map(toks):
    _, a, b = toks
    t = al.ByteTrie()
    for i, k in enumerate([b"a", b"ab", b"abc", b"b", b"abd"]):
        t.insert(k, i)
    assert t.longest_prefix(b"abcd") == 2 and t.longest_prefix(b"abx") == 1 and t.longest_prefix(b"zz") == -1
    ident = al.build_vocab_map(a, a)
    tb = al.token_bytes(a)
    real = [i for i, x in enumerate(tb) if x]
    dup = {}
    for i in real:
        dup.setdefault(tb[i], i)
    assert all(ident[i] == dup[tb[i]] for i in real)                  # same vocabulary -> identity (lowest id of equal strings)
    m = al.build_vocab_map(b, a)
    sb, tbb = al.token_bytes(a), al.token_bytes(b)
    for t_id in np.random.default_rng(0).choice(len(tbb), 200):
        if not tbb[t_id]:
            assert m[t_id] == -1
            continue
        assert m[t_id] >= 0                                            # byte fallback: every token has an image
        img = sb[m[t_id]]
        assert tbb[t_id].startswith(img)
        assert not any(tbb[t_id].startswith(x) and len(x) > len(img) for x in sb if x)   # and it is the longest


def test_remap_conserves_mass_and_matches_bruteforce(toks):
    _, a, b = toks
    table = torch.from_numpy(al.build_vocab_map(b, a))
    g = torch.Generator().manual_seed(0)
    V, K = len(table), 40
    lp, ids = torch.log_softmax(torch.randn(30, V, generator=g) * 3, -1).topk(K, -1)
    o_lp, o_id = topk.remap_topk(lp, ids.int(), table, K)
    for r in range(30):
        acc = {}
        for l, i in zip(lp[r].tolist(), ids[r].tolist()):
            s = int(table[i])
            if s >= 0:
                acc[s] = acc.get(s, 0.0) + float(np.exp(l))
        got = {int(i): float(np.exp(l)) for l, i in zip(o_lp[r].tolist(), o_id[r].tolist()) if np.isfinite(l)}
        assert got.keys() == acc.keys()
        assert all(abs(got[k] - acc[k]) < 1e-5 for k in acc)
        assert abs(sum(got.values()) - sum(acc.values())) < 1e-5 and sum(got.values()) <= lp[r].exp().sum() + 1e-5
        vals = o_lp[r][torch.isfinite(o_lp[r])]
        assert (vals[:-1] >= vals[1:] - 1e-6).all()


def test_position_alignment_on_shared_text(toks):
    _, a, b = toks
    from llm_distillery_b200.data.tokenize import TokenizeSpec, encode_prompt_format, tokenize_sample
    from llm_distillery_b200.data.convo import ConvoTokenized
    from llm_distillery_b200.config import DEFAULT_PROMPT_FORMAT
    item = {"init": "", "conversations": [{"from": "human", "value": "the quick brown fox jumps over wizard quartz 42"},
                                          {"from": "gpt", "value": "sphinx of black quartz judge my vow"}], "tags": []}
    convs = []
    for tk in (a, b):
        spec = TokenizeSpec(128, model_student=True, model_add_bos=True, bos_token_id=1)
        _, t, ranges, n, empty = tokenize_sample(0, item, tk, encode_prompt_format(DEFAULT_PROMPT_FORMAT, tk), spec)
        convs.append(ConvoTokenized(t, ranges, 128 - n, False, 0))
    s, t = convs
    sb, tb = al.token_bytes(a), al.token_bytes(b)
    pos = al.align_positions(s, t, sb, tb)
    so, to = al.start_offsets(s.tokenized, s.length, sb), al.start_offsets(t.tokenized, t.length, tb)
    assert so[-1] == to[-1]                                   # both token streams spell the same bytes
    ci = s.content_indices(); ci = ci[ci < s.length]
    assert (pos >= 0).mean() > 0.2       # the finer tokenizer has many boundaries the coarser one lacks
    for r, p in enumerate(pos):
        if p >= 0:
            assert so[ci[r] + 1] == to[p + 1]


def test_two_teachers_one_with_another_tokenizer(toks, tmp_path):
    root, a, b = toks
    os.environ["B200_NO_PROGRESS"] = "1"
    cfg_t = preset("plumbing-teacher", vocab_size=768, hidden_size=64, intermediate_size=176, max_position_embeddings=128)
    cfg_s = preset("plumbing-student", vocab_size=512, hidden_size=64, intermediate_size=176, max_position_embeddings=128,
                   num_hidden_layers=2)
    synthetic.make_model_dir(str(tmp_path / "teachers" / "t_same"), preset("plumbing-teacher", vocab_size=512, hidden_size=64,
                             intermediate_size=176, max_position_embeddings=128), str(root / "a"), seed=1, batch_size=4, add_bos=False)
    synthetic.make_model_dir(str(tmp_path / "teachers" / "t_other"), cfg_t, str(root / "b"), seed=2, batch_size=4, add_bos=False)
    synthetic.make_model_dir(str(tmp_path / "student"), cfg_s, str(root / "a"), seed=3)
    synthetic.make_dataset(str(tmp_path / "train.jsonl"), 10, seed=3)
    synthetic.make_dataset(str(tmp_path / "val.jsonl"), 3, seed=4)
    conf = {"cache_folder": str(tmp_path / "cache"), "dataset_path": str(tmp_path / "train.jsonl"),
            "validation_dataset_path": str(tmp_path / "val.jsonl"), "teacher_models_folder": str(tmp_path / "teachers"),
            "student_path": str(tmp_path / "student"), "context_len": 96, "crop_distr_to_size": 400, "save_topK": 16,
            "device": "cpu", "num_epochs": 1, "batch_size": 2, "grad_accum_batches": 1, "lr": 1e-3, "optimizer": "adamw",
            "training_precision": "fp32", "freeze_layers": [], "loss": "jsd", "cross_tokenizer": True}
    (tmp_path / "config.json").write_text(json.dumps(conf))
    with pytest.raises(ValueError):
        cli.main(["--config", str(tmp_path / "config.json"), "--cross_tokenizer", "false"])
    out = cli.main(["--config", str(tmp_path / "config.json")])
    assert out["trained_samples"] == 10
    st = H5Store(str(tmp_path / "cache" / "dataset"))
    v, ix = st.load_id(st.get_dataset_ids()[0])
    mass = np.exp(v).sum(-1)
    assert ix.max() < 400 and (mass > 0.03).all() and (mass <= 2.0 + 1e-2).all()
    st.close()
    # the other-vocabulary teacher alone: aligned rows carry remapped mass on student ids, unaligned rows are empty
    conf2 = dict(conf, teacher_models_folder=str(tmp_path / "teachers" / "t_other"), cache_folder=str(tmp_path / "cache2"),
                 loss="kl")
    (tmp_path / "config2.json").write_text(json.dumps(conf2))
    out = cli.main(["--config", str(tmp_path / "config2.json")])
    assert out["trained_samples"] == 10 and np.isfinite(out["last_validation"]["kl_div"])
    st = H5Store(str(tmp_path / "cache2" / "dataset"))
    got_rows = empty_rows = 0
    for cid in st.get_dataset_ids():
        v, ix = st.load_id(cid)
        fin = np.isfinite(v)
        got_rows += int(fin.any(1).sum())
        empty_rows += int((~fin.any(1)).sum())
        assert ix[fin].max() < 400 and (np.exp(v[fin.any(1)]).sum(-1) <= 1.0 + 1e-2).all()
    assert got_rows > 0 and empty_rows > 0
    st.close()


def _random_vocabularies(seed, n_student=3000, n_teacher=4000):
    """Byte-fallback style vocabularies: all 256 single bytes plus random multi-byte strings over a small alphabet
    (so that prefixes collide often), some strings in both."""
    import random
    rng = random.Random(seed)
    alpha = b"abcde \xc3\xa9"
    def words(n):
        return [bytes(rng.choice(alpha) for _ in range(rng.randint(1, 9))) for _ in range(n)]
    student = [bytes([b]) for b in range(256)] + words(n_student) + [b""]
    teacher = [b"", bytes([7])] + words(n_teacher) + student[300:600] + [b"\xff\xfe\xfd" * 5]
    return teacher, student


def test_flattened_trie_walk_equals_the_dictionary_trie():
    import numpy as np
    from llm_distillery_b200.align.aligner import ByteTrie, vocab_map_from_bytes
    from llm_distillery_b200.ops.topk import trie_walk
    teacher, student = _random_vocabularies(0, 400, 500)
    trie = ByteTrie()
    for i, b in enumerate(student):
        if b:
            trie.insert(b, i)
    want = np.asarray([trie.longest_prefix(b) if b else -1 for b in teacher])
    got, got_len = trie_walk(trie.flatten(), teacher, "cpu")
    assert np.array_equal(got.numpy(), want)
    for t, (sid, n) in enumerate(zip(got.tolist(), got_len.tolist())):
        if sid >= 0:
            assert student[sid] == teacher[t][:n] and n == len(student[sid])
        else:
            assert n == 0
    # byte-fallback student vocabulary: every non-empty teacher token has an image
    assert all(s >= 0 for s, b in zip(got.tolist(), teacher) if b)
    assert np.array_equal(vocab_map_from_bytes(teacher, student), want)
    # a vocabulary limit removes the longer tokens: images fall back to shorter prefixes, never disappear
    lim = vocab_map_from_bytes(teacher, student, student_vocab_limit=256)
    assert all(0 <= s < 256 for s, b in zip(lim.tolist(), teacher) if b)


@pytest.mark.gpu
def test_trie_walk_kernel_equals_the_dictionary_trie():
    import numpy as np
    from llm_distillery_b200.align.aligner import ByteTrie, vocab_map_from_bytes
    from llm_distillery_b200.ops import _lib
    from llm_distillery_b200.ops.topk import trie_walk
    for seed, (ns, nt) in enumerate([(3000, 4000), (20000, 50000), (5, 3)]):
        teacher, student = _random_vocabularies(seed, ns, nt)
        trie = ByteTrie()
        for i, b in enumerate(student):
            if b:
                trie.insert(b, i)
        want = np.asarray([trie.longest_prefix(b) if b else -1 for b in teacher])
        got, got_len = trie_walk(trie.flatten(), teacher, "cuda")
        torch.cuda.synchronize()
        assert _lib.take_device_error() == 0
        assert np.array_equal(got.cpu().numpy(), want)
        lens = got_len.cpu().tolist()
        assert all((n == len(student[s])) if s >= 0 else n == 0 for s, n in zip(want.tolist(), lens))
        assert np.array_equal(vocab_map_from_bytes(teacher, student, device="cuda"), want)
    # a student vocabulary without any token: nothing has an image
    empty = ByteTrie().flatten()
    got, _ = trie_walk(empty, [b"abc", b""], "cuda")
    assert got.cpu().tolist() == [-1, -1]


def test_native_trie_builder_equals_the_dictionary_trie():
    import time
    from llm_distillery_b200.align.aligner import ByteTrie, flat_trie
    from llm_distillery_b200.ops import _lib
    try:
        _lib.host().b200_trie_build
    except (OSError, AttributeError):
        pytest.skip("host library not built")
    for seed, (ns, nt) in enumerate([(400, 10), (20000, 10), (0, 1)]):
        _, student = _random_vocabularies(seed, ns, nt)
        student = student + student[300:320]              # duplicates: the lowest id stays
        for limit in (None, 256, 1000):
            trie = ByteTrie()
            for i, b in enumerate(student):
                if b and (limit is None or i < limit):
                    trie.insert(b, i)
            want, got = trie.flatten(), flat_trie(student, limit)
            assert sorted(want) == sorted(got)
            for k in want:
                assert got[k].dtype == want[k].dtype and np.array_equal(got[k], want[k]), (seed, limit, k)
    empty = flat_trie([], None)
    assert empty["node_value"].tolist() == [-1] and empty["edge_start"].tolist() == [0, 0]
    # and it is the fast way: a 100k-token vocabulary
    import random
    rng = random.Random(1)
    big = [bytes(rng.randrange(97, 123) for _ in range(rng.randint(2, 12))) for _ in range(100000)]
    t0 = time.perf_counter()
    ft = flat_trie(big)
    native_s = time.perf_counter() - t0
    assert ft["node_value"].max() == 99999 or len(set(big)) < len(big)
    assert native_s < 1.5, native_s
