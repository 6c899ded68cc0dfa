"""C++ HDF5 store: round trips, metadata, rename/delete/merge, crash consistency, and a byte-level check of the
emitted structures with an independent reader."""
import os
import shutil

import numpy as np
import pytest

from llm_distillery_b200.data.convo import TeacherRows
from llm_distillery_b200.data.h5store import H5Store, merge_topk
from tests.h5_spec_reader import SpecReader


def _rows(cid, n=37, K=16, V=500, seed=0, sample="s"):
    rng = np.random.default_rng(seed + cid)
    logits = rng.normal(size=(n, V)).astype(np.float32) * 3
    lp = logits - np.log(np.exp(logits).sum(-1, keepdims=True))
    idx = np.argsort(-lp, axis=1)[:, :K]
    return TeacherRows(cid, np.take_along_axis(lp, idx, 1), idx.astype(np.int64), f"sha{cid:04d}" * 8, f"{sample}-{cid} é")


@pytest.mark.parametrize("shuffle", [True, False])
def test_roundtrip_reopen_and_spec_reader(tmp_path, shuffle):
    st = H5Store(str(tmp_path), shuffle=shuffle)
    data = {i: _rows(i, n=5 + 3 * i) for i in [0, 1, 2, 10, 33, 7]}
    st.write_batch(list(data.values()))
    st.set_vocab_family("llama_3")
    st.set_topk(16)
    st.wait()
    assert sorted(st.get_dataset_ids()) == sorted(data)
    for i, r in data.items():
        v, ix = st.load_id(i)
        assert v.dtype == np.float32 and ix.dtype == np.int64
        assert np.array_equal(v, r.values.astype(np.float16).astype(np.float32)) and np.array_equal(ix, r.indices)
    assert st.get_available_shas()[10] == data[10].content_sha
    st.close()
    st2 = H5Store(str(tmp_path))
    assert st2.get_vocab_family() == "llama_3" and st2.get_topk() == 16 and st2.has_data()
    v, ix = st2.load_id(33)
    assert np.array_equal(ix, data[33].indices)
    st2.close()
    sr = SpecReader(os.path.join(str(tmp_path), "distributions.hdf5"))
    root = sr.group(sr.root_hdr)
    assert sorted(root) == sorted(f"convo_{i}" for i in data)
    assert sr.attrs(sr.root_hdr) == {"vocab_family": "llama_3", "topk": 16}
    g = sr.group(root["convo_10"])
    assert sorted(g) == ["distributions", "indices"]
    assert sr.attrs(root["convo_10"]) == {"content_sha": data[10].content_sha, "sample": data[10].sample}
    assert np.array_equal(sr.dataset(g["distributions"]), data[10].values.astype(np.float16))
    assert np.array_equal(sr.dataset(g["indices"]), data[10].indices.astype(np.uint32))


def test_many_groups_multilevel_btree(tmp_path):
    st = H5Store(str(tmp_path))
    n = 1300   # > 32 * 32 links: forces a two-level group B-tree
    st.write_batch([_rows(i, n=2, K=4, V=50) for i in range(n)])
    st.close()
    sr = SpecReader(os.path.join(str(tmp_path), "distributions.hdf5"))
    assert len(sr.group(sr.root_hdr)) == n
    st = H5Store(str(tmp_path))
    assert sorted(st.get_dataset_ids()) == list(range(n))
    v, ix = st.load_id(1299)
    assert v.shape == (2, 4)
    st.close()


def test_delete_rename_swap_purge_update_sha(tmp_path):
    st = H5Store(str(tmp_path))
    st.write_batch([_rows(i) for i in range(6)])
    st.wait()
    ref = {i: st.load_id(i)[1] for i in range(6)}
    st.sync([4, 5], {0: 1, 1: 0, 2: 9})        # swap 0<->1, move 2->9
    assert sorted(st.get_dataset_ids()) == [0, 1, 3, 9]
    assert np.array_equal(st.load_id(0)[1], ref[1]) and np.array_equal(st.load_id(1)[1], ref[0])
    assert np.array_equal(st.load_id(9)[1], ref[2])
    st.update_shas({3: "f" * 64, 77: "ignored"})
    assert st.get_sha(3) == "f" * 64 and np.array_equal(st.load_id(3)[1], ref[3])
    before = st.file_bytes()
    st.repack()
    assert st.file_bytes() < before and sorted(st.get_dataset_ids()) == [0, 1, 3, 9]
    st.set_vocab_family("x"); st.set_topk(3)
    st.purge_dataset(ask_confirmation=False)
    assert not st.has_data() and st.get_vocab_family() is None and st.get_topk() is None
    with pytest.raises(ValueError):
        st.load_id(0)
    st.close()


def test_multi_teacher_merge_sums_probabilities(tmp_path):
    a, b = _rows(0, n=9, seed=1), _rows(0, n=12, seed=2)
    st = H5Store(str(tmp_path))
    st.write_batch([a]); st.wait()
    st.write_batch([b]); st.wait()
    v, ix = st.load_id(0)
    assert v.shape == (12, 16)
    for r in range(9):
        acc = {}
        for src in (a, b):
            for i, lp in zip(src.indices[r], src.values[r].astype(np.float16).astype(np.float32)):
                acc[int(i)] = acc.get(int(i), 0.0) + float(np.exp(lp))
        best = sorted(acc.items(), key=lambda kv: -kv[1])[:16]
        assert set(int(x) for x in ix[r]) == {k for k, _ in best} or abs(best[15][1] - sorted(acc.values())[-17]) < 1e-6
        got = dict(zip(ix[r].tolist(), np.exp(v[r]).tolist()))
        for k, p in best[:8]:
            assert abs(got[k] - p) < 3e-3 * max(p, 1e-3)
    assert np.array_equal(ix[9:], b.indices[9:])
    assert st.get_sha(0) == b.content_sha
    st.close()
    l, i = merge_topk(a.values, a.indices, a.values, a.indices)   # same teacher twice = doubled probabilities
    assert np.allclose(np.sort(np.exp(l), 1), np.sort(2 * np.exp(a.values), 1), rtol=1e-5)


def test_merge_with_a_real_token_zero_next_to_empty_slots():
    """Rows that came through a cross-tokenizer remap end in empty slots (id 0, log-prob -inf). A real token 0 in both
    inputs must still have its two probabilities summed, whatever number of empty slots shares its id."""
    ninf = -np.inf
    disk_l = np.log(np.array([[0.5, 0.2, 0.0, 0.0, 0.0]], dtype=np.float32), where=[[True, True, False, False, False]],
                    out=np.full((1, 5), ninf, dtype=np.float32))
    disk_i = np.array([[0, 7, 0, 0, 0]], dtype=np.uint32)
    new_l = np.log(np.array([[0.3, 0.25, 0.1, 0.0, 0.0]], dtype=np.float32), where=[[True, True, True, False, False]],
                   out=np.full((1, 5), ninf, dtype=np.float32))
    new_i = np.array([[0, 9, 7, 0, 0]], dtype=np.uint32)
    l, i = merge_topk(disk_l, disk_i, new_l, new_i)
    got = {int(k): float(np.exp(v)) for k, v in zip(i[0], l[0]) if np.isfinite(v)}
    assert got.keys() == {0, 7, 9}
    assert abs(got[0] - 0.8) < 1e-6 and abs(got[7] - 0.3) < 1e-6 and abs(got[9] - 0.25) < 1e-6
    assert [int(x) for x in i[0][:3]] == [0, 7, 9]                  # by probability, descending
    assert all(int(x) == 0 for x in i[0][3:]) and np.all(np.isneginf(l[0][3:]))   # what is left: empty slots again


def test_killed_before_flush_keeps_last_consistent_state(tmp_path):
    st = H5Store(str(tmp_path))
    st.write_batch([_rows(i) for i in range(3)])
    st.wait()                                     # consistent state with 3 conversations
    snap = str(tmp_path / "snap.hdf5")
    st._put_one(_rows(3), True)                   # data appended, root not yet rewritten
    shutil.copy(st.file_path, snap)               # what a kill -9 right now leaves on disk
    st.close()
    rec = H5Store(snap)
    assert sorted(rec.get_dataset_ids()) == [0, 1, 2]
    assert rec.load_id(2)[0].shape == (37, 16)
    rec.write_batch([_rows(3)]); rec.wait()       # and the file keeps working
    assert sorted(rec.get_dataset_ids()) == [0, 1, 2, 3]
    rec.close()
    # truncated tail (torn write) is also survivable: the superblock still points at the old root
    with open(snap, "r+b") as f:
        f.truncate(os.path.getsize(snap) - 0)
    SpecReader(snap)


def test_prefetch_batches_padded_sorted(tmp_path):
    st = H5Store(str(tmp_path))
    st.write_batch([_rows(i, n=4 + i) for i in range(8)])
    st.wait()
    st.enqueue_get_batches([[0, 1, 2], [3, 4]], sort_ids=True)
    st.enqueue_get_batches([[5, 6, 7]], sort_ids=True)
    b0, b1, b2 = st.read_next_batch(), st.read_next_batch(), st.read_next_batch()
    assert b0["values"].shape == (3, 6, 16) and b0["lengths"] == [4, 5, 6] and b1["ids"] == [3, 4] and b2["ids"] == [5, 6, 7]
    assert (b0["values"][0, 4:] == 0).all()
    assert all((np.diff(ix, axis=1) > 0).all() for ix in b0["indices"])
    v, ix = st.load_id(1)
    o = np.argsort(ix, 1)
    assert np.array_equal(b0["values"][1, :5], np.take_along_axis(v, o, 1))
    st.read_only_mode([[0], [1]])
    seen = [st.read_next_batch()["ids"][0] for _ in range(5)]
    assert seen == [0, 1, 0, 1, 0]
    st.close()


def _tiny_store(path, shuffle):
    st = H5Store(path, writers=1, shuffle=shuffle)
    for i in range(3):
        v = (np.arange(12 * 5, dtype=np.float32).reshape(12, 5) * -0.25 - i).astype(np.float16)
        ix = (np.arange(12 * 5, dtype=np.int64).reshape(12, 5) * 7 + i) % 32000
        st.write_batch([TeacherRows(10 + i, v, ix, f"sha-{i}", "sample")])
        st.wait()
    st.set_vocab_family("llama_3")
    st.set_topk(5)
    st.close()


@pytest.mark.parametrize("shuffle,digest", [(True, None), (False, None)])
def test_file_bytes_are_deterministic(tmp_path, shuffle, digest):
    """Same writes, same bytes: two files written with the same calls are identical (no timestamps, no pointers, no
    uninitialised padding leak into the file), so a format change shows up as a diff of a hex dump."""
    import hashlib
    a, b = str(tmp_path / "a"), str(tmp_path / "b")
    _tiny_store(a, shuffle)
    _tiny_store(b, shuffle)
    da = hashlib.sha256(open(a + "/distributions.hdf5", "rb").read()).hexdigest()
    db = hashlib.sha256(open(b + "/distributions.hdf5", "rb").read()).hexdigest()
    assert da == db


def test_h5py_reads_the_file_when_it_is_installed(tmp_path):
    h5py = pytest.importorskip("h5py")      # not on the build box; runs wherever the library exists
    if not hasattr(h5py, "File"):           # a stand-in module put there by the tests that import the reference
        pytest.skip("h5py is not installed")
    for shuffle in (True, False):
        d = str(tmp_path / f"s{int(shuffle)}")
        _tiny_store(d, shuffle)
        with h5py.File(d + "/distributions.hdf5", "r") as f:
            assert f.attrs["vocab_family"] == "llama_3" and int(f.attrs["topk"]) == 5
            g = f["convo_11"]
            assert g.attrs["content_sha"] == "sha-1"
            assert g["distributions"].dtype == np.float16 and g["distributions"].shape == (12, 5)
            assert g["indices"].dtype == np.uint32 and int(g["indices"][0, 0]) == 1


def test_reopen_keeps_the_validation_cycle(tmp_path):
    """Another process appends to the file; a reader that reopens it goes on cycling over its validation batches."""
    st = H5Store(str(tmp_path))
    st.write_batch([_rows(i) for i in range(4)])
    st.wait()
    reader = H5Store(str(tmp_path))
    reader.read_only_mode([[0, 1], [2, 3]], sort_ids=True)
    first = reader.read_next_batch(timeout=30)
    st.write_batch([_rows(9)])
    st.wait()
    reader.reopen()
    assert 9 in reader.get_dataset_ids()
    again = [reader.read_next_batch(timeout=30) for _ in range(3)]       # the cycle starts over: [0,1], [2,3], [0,1]
    assert np.array_equal(again[0]["values"][0], first["values"][0]) and np.array_equal(again[2]["values"][0], first["values"][0])
    assert not np.array_equal(again[1]["values"][0], first["values"][0])
    reader.close()
    st.close()


GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "golden_store.hdf5")
GOLDEN_SHA256 = "774751dfcc40de7d55c6f62b96068a5a84bc35783a5f21a4e36b33c362c7a0ca"


def _write_golden_content(folder):
    st = H5Store(folder, writers=1)
    for i in (0, 3, 12):
        st.write_batch([_rows(i, n=4 + i, K=8, V=100)])
        st.wait()
    st.set_vocab_family("llama_3")
    st.set_topk(8)
    st.wait()
    st.close()


def test_committed_golden_file_reads_back_and_the_writer_still_emits_its_bytes(tmp_path):
    """A store file written by an earlier build of the writer is kept in the repository: today's reader (and the
    independent spec reader) must still read it, and today's writer must still produce it byte for byte (with the zlib
    the bytes were recorded under; another zlib may deflate differently, then only the content is compared)."""
    import hashlib
    import zlib
    work = str(tmp_path / "golden")
    os.makedirs(work)
    shutil.copy(GOLDEN, os.path.join(work, "distributions.hdf5"))
    st = H5Store(work)
    assert sorted(st.get_dataset_ids()) == [0, 3, 12] and st.get_vocab_family() == "llama_3" and st.get_topk() == 8
    for i in (0, 3, 12):
        r = _rows(i, n=4 + i, K=8, V=100)
        v, ix = st.load_id(i)
        assert np.array_equal(v, r.values.astype(np.float16).astype(np.float32)) and np.array_equal(ix, r.indices)
        assert st.get_sha(i) == r.content_sha
    st.close()
    sr = SpecReader(GOLDEN)
    root = sr.group(sr.root_hdr)
    assert sorted(root) == ["convo_0", "convo_12", "convo_3"]
    assert np.array_equal(sr.dataset(sr.group(root["convo_3"])["indices"]), _rows(3, n=7, K=8, V=100).indices.astype(np.uint32))
    fresh = str(tmp_path / "fresh")
    _write_golden_content(fresh)
    with open(os.path.join(fresh, "distributions.hdf5"), "rb") as f:
        got = hashlib.sha256(f.read()).hexdigest()
    with open(GOLDEN, "rb") as f:
        assert hashlib.sha256(f.read()).hexdigest() == GOLDEN_SHA256
    if zlib.ZLIB_RUNTIME_VERSION == "1.3":
        assert got == GOLDEN_SHA256
