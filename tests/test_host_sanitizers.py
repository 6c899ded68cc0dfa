"""The native host library (HDF5 store, byte-trie builder) under AddressSanitizer + UBSan and under ThreadSanitizer.

``build --sanitize`` compiles the same C++ sources with ``-fsanitize=address,undefined`` and with
``-fsanitize=thread``; a child interpreter
preloads the sanitizer runtime, loads that library instead of the regular one (``B200_HOST_LIB``) and drives the store
through writes from several threads, merges, renames, deletes, a repack, a reopen and a prefetch, and the trie builder
through a large vocabulary. Any heap overflow, use after free or undefined operation ends the child with the
sanitizer's report. No GPU is involved."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

CHILD = r'''
import os, sys, random
import numpy as np
sys.path.insert(0, sys.argv[1])
from llm_distillery_b200.align.aligner import ByteTrie, flat_trie
from llm_distillery_b200.data.convo import TeacherRows
from llm_distillery_b200.data.h5store import H5Store
from llm_distillery_b200.ops import _lib
assert "san.so" in os.environ["B200_HOST_LIB"] and _lib.host() is not None

def rows(cid, n, K=16, V=500):
    rng = np.random.default_rng(cid)
    lp = np.log(rng.dirichlet(np.ones(V), size=n)).astype(np.float32)
    idx = np.argsort(-lp, axis=1)[:, :K]
    return TeacherRows(cid, np.take_along_axis(lp, idx, 1), idx.astype(np.int64), ("%04d" % cid) * 16, "s-%d" % cid)

d = sys.argv[2]
for shuffle in (True, False):
    st = H5Store(os.path.join(d, "a%d" % shuffle), shuffle=shuffle, writers=4)
    st.write_batch([rows(i, 3 + (i * 7) % 40) for i in range(60)])
    st.write_batch([rows(i, 3 + (i * 7) % 40) for i in range(10)])        # second teacher: merge path
    st.set_vocab_family("llama_3"); st.set_topk(16)
    st.wait()
    assert len(st.get_dataset_ids()) == 60
    st.sync([4, 5], {0: 1, 1: 0, 2: 99})
    st.update_shas({3: "f" * 64})
    st.repack()
    ids = sorted(st.get_dataset_ids())
    assert 99 in ids and 4 not in ids
    st.enqueue_get_batches([ids[:4], ids[4:7]], sort_ids=True)
    b = st.read_next_batch(); b = st.read_next_batch()
    st.close()
    st2 = H5Store(os.path.join(d, "a%d" % shuffle))
    v, ix = st2.load_id(99)
    assert v.shape[1] == 16 and st2.get_topk() == 16
    st2.purge_dataset(ask_confirmation=False)
    st2.close()

rng = random.Random(0)
vocab = [bytes([b]) for b in range(256)] + [bytes(rng.randrange(97, 105) for _ in range(rng.randint(1, 10))) for _ in range(30000)]
ft = flat_trie(vocab + vocab[300:400] + [b""], None)
trie = ByteTrie()
for i, b in enumerate(vocab):
    trie.insert(b, i)
want = trie.flatten()
assert all(np.array_equal(ft[k], want[k]) for k in want)
assert flat_trie([], None)["node_value"].tolist() == [-1]
print("CHILD_OK")
'''


def _runtime(name: str) -> str | None:
    try:
        p = subprocess.run(["gcc", f"-print-file-name={name}"], capture_output=True, text=True, timeout=30).stdout.strip()
    except (OSError, subprocess.TimeoutExpired):
        return None
    return p if os.path.isabs(p) and os.path.exists(p) else None


@pytest.mark.parametrize("kind", ["asan", "tsan"])
def test_store_and_trie_builder_are_clean_under_sanitizers(tmp_path, kind):
    """asan: AddressSanitizer + UBSan; tsan: ThreadSanitizer (the store's writer pool and prefetch thread)."""
    runtime = _runtime("libasan.so" if kind == "asan" else "libtsan.so")
    if runtime is None:
        pytest.skip(f"no {kind} runtime on this machine")
    from llm_distillery_b200 import build as native_build
    out = native_build.build(sanitize=True)
    lib = out.get(f"host_{kind}")
    assert lib and os.path.exists(lib)
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ, LD_PRELOAD=runtime, B200_HOST_LIB=lib, B200_NO_PROGRESS="1",
               ASAN_OPTIONS="detect_leaks=0:alloc_dealloc_mismatch=0:detect_odr_violation=0:halt_on_error=1:abort_on_error=0",
               UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1",
               TSAN_OPTIONS="halt_on_error=0:report_signal_unsafe=0:exitcode=66")
    r = subprocess.run([sys.executable, str(script), ROOT, str(tmp_path)], capture_output=True, text=True, timeout=900,
                       env=env)
    report = r.stderr[-4000:]
    for marker in ("AddressSanitizer", "runtime error:", "ThreadSanitizer"):
        assert marker not in r.stderr, report
    assert r.returncode == 0 and "CHILD_OK" in r.stdout, (r.stdout[-1000:], report)
