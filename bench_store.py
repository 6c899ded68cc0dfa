#!/usr/bin/env python
"""Host-side data-plane benchmark (no GPU): writing collected top-K rows into the HDF5 store and reading training
batches back, against a restatement of what the reference does per conversation with the libraries it uses
(classes/data_manager.py:287-312: float16 + uint32 datasets, gzip level 6, one conversation at a time on one process;
h5py is not installed here, so the restatement is numpy + zlib + one file write per dataset).

    python bench_store.py [--convos 400] [--rows 1024] [--topk 200] [--writers 4]

One JSON line: raw MB/s and conversations/s for the store (multi-threaded deflate in C++, append-only file) and for the
single-threaded restatement, plus the read-back rate of batches.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import sys
import tempfile
import time
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from llm_distillery_b200.data.convo import TeacherRows  # noqa: E402
from llm_distillery_b200.data.h5store import H5Store  # noqa: E402


def make_rows(n: int, rows: int, k: int, seed: int = 0):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        logits = rng.standard_normal((rows, k)).astype(np.float32) * 3.0
        lp = np.sort(logits - np.log(np.exp(logits).sum(-1, keepdims=True)), axis=-1)[:, ::-1]
        ids = rng.integers(0, 32000, (rows, k)).astype(np.int64)
        out.append(TeacherRows(i, np.ascontiguousarray(lp.astype(np.float16)), ids, f"sha{i}", "s"))
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--convos", type=int, default=400)
    ap.add_argument("--rows", type=int, default=1024)
    ap.add_argument("--topk", type=int, default=200)
    ap.add_argument("--writers", type=int, default=4)
    a = ap.parse_args()
    data = make_rows(a.convos, a.rows, a.topk)
    raw = sum(r.values.nbytes + r.indices.shape[0] * r.indices.shape[1] * 4 for r in data)   # fp16 + uint32 on disk
    tmp = tempfile.mkdtemp(prefix="b200_store_")
    try:
        st = H5Store(os.path.join(tmp, "a"), writers=a.writers)
        t0 = time.perf_counter()
        for i in range(0, len(data), 8):
            st.write_batch(data[i:i + 8])
        st.wait()
        st.flush()
        t_store = time.perf_counter() - t0
        size_store = st.file_bytes()
        ids = st.get_dataset_ids()
        t0 = time.perf_counter()
        for i in range(0, len(ids), 8):
            st.make_batch(ids[i:i + 8])
        t_read = time.perf_counter() - t0
        st.close()
        # the reference's sequence per conversation, single process
        t0 = time.perf_counter()
        size_ref = 0
        with open(os.path.join(tmp, "ref.bin"), "wb") as f:
            for r in data:
                v = zlib.compress(np.ascontiguousarray(r.values.astype(np.float16)).tobytes(), 6)
                ix = zlib.compress(np.ascontiguousarray(r.indices.astype(np.uint32)).tobytes(), 6)
                f.write(v)
                f.write(ix)
                size_ref += len(v) + len(ix)
        t_ref = time.perf_counter() - t0
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    print(json.dumps({
        "case": "top-K rows -> HDF5", "convos": a.convos, "rows": a.rows, "topk": a.topk, "raw_mb": round(raw / 1e6, 1),
        "store": {"seconds": round(t_store, 3), "raw_mb_per_s": round(raw / 1e6 / t_store, 1),
                  "convos_per_s": round(a.convos / t_store, 1), "file_mb": round(size_store / 1e6, 1),
                  "ratio": round(raw / size_store, 2), "writer_threads": a.writers},
        "reference_restatement": {"seconds": round(t_ref, 3), "raw_mb_per_s": round(raw / 1e6 / t_ref, 1),
                                  "convos_per_s": round(a.convos / t_ref, 1), "file_mb": round(size_ref / 1e6, 1),
                                  "ratio": round(raw / size_ref, 2)},
        "speedup": round(t_ref / t_store, 2),
        "read_back": {"seconds": round(t_read, 3), "raw_mb_per_s": round(raw / 1e6 / t_read, 1)},
        "cpus": os.cpu_count()}))


if __name__ == "__main__":
    main()
