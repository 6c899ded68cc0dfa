"""HDF5 teacher-distribution store (Python face of csrc/h5/h5store.cc).

Covers the task set of the reference's ``H5DataManager`` (classes/data_manager.py:88-125: get/put/update batches,
clear, rename, ids, SHAs, vocab family, top-K, generic attrs, has_data) with one in-process object instead of a
spawned server process: the C++ store is thread-safe, deflate/inflate run with the GIL released, writes go through
a small thread pool (``write_batch`` returns at once; ``wait()`` is the reference's ``done_everything``), and
reads are prefetched by a background thread into a bounded queue (``enqueue_get_batches`` / ``read_only_mode`` /
``read_next_batch``). Batches are padded along the token axis like the reference (data_manager.py:332-353) and are
optionally delivered in pinned host memory with each row's ids sorted ascending (what the fused loss head wants).

Multi-teacher semantics: writing a conversation that already exists MERGES - probabilities of equal token ids are
summed over the union of both top-K sets, the best K are kept, the log is stored (data_manager.py:198-261;
normalisation happens at training time). The reference's merge path crashes (wrong argument count at :190); this
one is the intended behaviour.
"""
from __future__ import annotations

import ctypes
import queue
import threading
from concurrent.futures import ThreadPoolExecutor
from ctypes import c_char_p, c_int, c_longlong, c_void_p, POINTER

import numpy as np

from ..ops import _lib
from .convo import TeacherRows

_CONFIRM_WORDS = {"y", "yes", "ye", "1", "true", "t"}


def _bind():
    lib = _lib.host()
    if getattr(lib, "_h5_bound", False):
        return lib
    lib.h5s_open.restype = c_void_p
    lib.h5s_open.argtypes = [c_char_p, c_int, c_char_p, c_int]
    lib.h5s_error.restype = c_char_p
    lib.h5s_error.argtypes = [c_void_p]
    for name, args, res in [
        ("h5s_flush", [c_void_p], c_int), ("h5s_close", [c_void_p], c_int),
        ("h5s_put", [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_longlong, c_char_p, c_char_p, c_int], c_int),
        ("h5s_has", [c_void_p, c_longlong], c_int), ("h5s_count", [c_void_p], c_longlong),
        ("h5s_list_ids", [c_void_p, c_void_p, c_longlong], c_longlong),
        ("h5s_shape", [c_void_p, c_longlong, POINTER(c_longlong), POINTER(c_longlong), POINTER(c_int)], c_int),
        ("h5s_get", [c_void_p, c_longlong, c_void_p, c_void_p], c_int),
        ("h5s_get_attr_str", [c_void_p, c_longlong, c_char_p, c_void_p, c_longlong], c_longlong),
        ("h5s_set_root_attr_str", [c_void_p, c_char_p, c_char_p], c_int),
        ("h5s_get_root_attr_int", [c_void_p, c_char_p, POINTER(c_longlong)], c_int),
        ("h5s_set_root_attr_int", [c_void_p, c_char_p, c_longlong, c_int], c_int),
        ("h5s_delete", [c_void_p, c_longlong], c_int),
        ("h5s_rename_many", [c_void_p, c_void_p, c_void_p, c_longlong], c_int),
        ("h5s_update_sha", [c_void_p, c_longlong, c_char_p], c_int),
        ("h5s_file_bytes", [c_void_p], c_longlong), ("h5s_repack", [c_void_p, c_char_p], c_int),
    ]:
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, res
    lib._h5_bound = True
    return lib


def merge_topk(disk_logp: np.ndarray, disk_idx: np.ndarray, new_logp: np.ndarray, new_idx: np.ndarray):
    """Union of two top-K sets per token: sum the probabilities of equal ids, keep the best K, return logs.
    Rows beyond the shorter input are taken from the longer one unchanged. Vectorised over rows."""
    K = disk_logp.shape[1]
    n = min(len(disk_logp), len(new_logp))
    ids = np.concatenate([disk_idx[:n].astype(np.int64), new_idx[:n].astype(np.int64)], axis=1)
    p = np.exp(np.concatenate([disk_logp[:n].astype(np.float32), new_logp[:n].astype(np.float32)], axis=1))
    # empty slots (log-prob -inf, id 0: what a cross-tokenizer remap leaves when fewer than K ids have an image) carry
    # no mass but would sit next to a real token 0 and break the "duplicates come in pairs" rule below: give each of
    # them an id of its own above every vocabulary; they sort last by probability and leave as id 0 again
    empty = ~(p > 0)
    ids = np.where(empty, (1 << 40) + np.arange(ids.shape[1], dtype=np.int64)[None, :], ids)
    order = np.argsort(ids, axis=1, kind="stable")
    ids = np.take_along_axis(ids, order, 1)
    p = np.take_along_axis(p, order, 1)
    dup = ids[:, 1:] == ids[:, :-1]          # each source has unique ids per row: duplicates come in pairs
    p[:, :-1] += np.where(dup, p[:, 1:], 0.0)
    p[:, 1:] = np.where(dup, -1.0, p[:, 1:])  # second copy drops out of the ranking
    top = np.argsort(-p, axis=1, kind="stable")[:, :K]
    out_p = np.take_along_axis(p, top, 1)
    out_i = np.take_along_axis(ids, top, 1)
    out_i = np.where(out_i >= (1 << 40), 0, out_i)
    with np.errstate(divide="ignore"):
        out_l = np.log(np.maximum(out_p, 0.0))
    rest_l, rest_i = (disk_logp[n:], disk_idx[n:]) if len(disk_logp) > n else (new_logp[n:], new_idx[n:])
    if len(rest_l):
        out_l = np.concatenate([out_l, rest_l.astype(np.float32)])
        out_i = np.concatenate([out_i, rest_i.astype(np.int64)])
    return out_l, out_i


def merge_topk_on(device: str, disk_logp: np.ndarray, disk_idx: np.ndarray, new_logp: np.ndarray, new_idx: np.ndarray):
    """``merge_topk`` on the GPU the store was opened for (kernel ``topk_merge``: csrc/loss/topk_logprob.cu), or the
    NumPy statement above when the store runs without a GPU or the rows do not fit the kernel (K above 1024, the two
    teachers kept different K). Called from the store's writer threads: the merge of conversation i runs while the
    model computes the next batch."""
    K = disk_logp.shape[1]
    n = min(len(disk_logp), len(new_logp))
    dev = str(device or "cpu")
    if not dev.startswith("cuda") or K > 1024 or new_logp.shape[1] != K or n == 0:
        return merge_topk(disk_logp, disk_idx, new_logp, new_idx)
    import torch
    if not torch.cuda.is_available():
        return merge_topk(disk_logp, disk_idx, new_logp, new_idx)
    from ..ops import topk as topk_ops
    d = torch.device(dev)
    with torch.cuda.device(d):
        up = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a[:n]).astype(dt, copy=False)).to(d)   # noqa: E731
        lp, ix = topk_ops.topk_merge(up(disk_logp, np.float32), up(disk_idx, np.int32), up(new_logp, np.float32),
                                     up(new_idx, np.int32))
        out_l, out_i = lp.cpu().numpy(), ix.cpu().numpy().astype(np.int64)
    rest_l, rest_i = (disk_logp[n:], disk_idx[n:]) if len(disk_logp) > n else (new_logp[n:], new_idx[n:])
    if len(rest_l):
        out_l = np.concatenate([out_l, rest_l.astype(np.float32)])
        out_i = np.concatenate([out_i, rest_i.astype(np.int64)])
    return out_l, out_i


def merge_full(disk_logp: np.ndarray, new_logp: np.ndarray) -> np.ndarray:
    n = max(len(disk_logp), len(new_logp))
    acc = np.zeros((n, disk_logp.shape[1]), dtype=np.float32)
    acc[: len(disk_logp)] += np.exp(disk_logp.astype(np.float32))
    acc[: len(new_logp)] += np.exp(new_logp.astype(np.float32))
    with np.errstate(divide="ignore"):
        return np.log(acc)


class H5Store:
    def __init__(self, dataset_path: str, device: str = "cpu", max_queue_size: int = 7, manager_name: str = "",
                 file_name: str = "distributions.hdf5", writers: int | None = None, interactive: bool = False,
                 compression_level: int = 6, shuffle: bool = True):
        """``shuffle``: put the HDF5 byte-shuffle filter in front of deflate for newly written datasets (read back
        transparently by this store and by h5py). The reference writes plain gzip-6 (classes/data_manager.py:300-309);
        ``shuffle=False`` reproduces that byte for byte in the filter pipeline."""
        import os
        if writers is None:      # deflate is the cost of a write (~9 MB/s per core at level 6): use the cores there are
            writers = min(32, max(4, (os.cpu_count() or 8) // 2))
        self.lib = _bind()
        self.file_path = dataset_path if dataset_path.endswith((".hdf5", ".h5")) else os.path.join(dataset_path, file_name)
        os.makedirs(os.path.dirname(os.path.abspath(self.file_path)), exist_ok=True)
        err = ctypes.create_string_buffer(512)
        self.h = self.lib.h5s_open(self.file_path.encode(), 1, err, 512)
        if not self.h:
            raise IOError(f"cannot open {self.file_path}: {err.value.decode()}")
        self.device = device
        self.manager_name = manager_name + " " if manager_name else manager_name
        self.interactive = interactive
        self.level = int(compression_level) | (0x100 if shuffle else 0)
        self.max_queue_size = max_queue_size
        self._pool = ThreadPoolExecutor(max_workers=writers, thread_name_prefix="h5w")
        self._pending: list = []
        self._pending_lock = threading.Lock()
        self._write_locks: dict[int, threading.Lock] = {}
        self.result_queue: queue.Queue = queue.Queue(max_queue_size)
        self._prefetch_thread: threading.Thread | None = None
        self._stop = threading.Event()
        self._todo: list = []
        self._cycle = None
        self._todo_cv = threading.Condition()
        self.closed = False

    # ------------------------------------------------------------------ helpers
    def _err(self) -> str:
        return self.lib.h5s_error(self.h).decode()

    def _confirm(self, message: str, confirm) -> bool:
        if confirm is not None:
            return bool(confirm(message))
        if not self.interactive:
            return True
        return input(message).lower() in _CONFIRM_WORDS

    # ------------------------------------------------------------------ writing
    def _put_one(self, rows: TeacherRows, merge: bool) -> None:
        cid = int(rows.convo_id)
        with self._pending_lock:
            lock = self._write_locks.setdefault(cid, threading.Lock())
        with lock:
            values, indices = rows.values, rows.indices
            sha, sample = rows.content_sha, rows.sample
            if merge and self.lib.h5s_has(self.h, cid):
                d_l, d_i = self.load_id(cid)
                if indices is not None and d_i is not None:
                    values, indices = merge_topk_on(self.device, d_l, d_i, np.asarray(values, dtype=np.float32),
                                                    np.asarray(indices))
                else:
                    values = merge_full(d_l, np.asarray(values, dtype=np.float32))
                sha = sha or (self.get_sha(cid) or "")
                sample = sample or (self._attr(cid, "sample") or "")
            if len(values) == 0:
                return
            v16 = np.ascontiguousarray(values, dtype=np.float16)
            i32 = None if indices is None else np.ascontiguousarray(indices, dtype=np.uint32)
            rc = self.lib.h5s_put(self.h, cid, v16.ctypes.data_as(c_void_p), None if i32 is None else i32.ctypes.data_as(c_void_p),
                                  v16.shape[0], v16.shape[1], str(sha or "").encode(), str(sample or "").encode("utf-8", "replace"),
                                  self.level)
            if rc != 0:
                raise IOError(f"HDF5 write of convo_{cid} failed: {self._err()}")

    def write_batch(self, batch: list[TeacherRows]) -> None:
        """Asynchronous; merges into conversations that already exist."""
        with self._pending_lock:
            self._pending.extend(self._pool.submit(self._put_one, r, True) for r in batch)

    def update_batch(self, batch: list[TeacherRows]) -> None:
        """Asynchronous; replaces instead of merging."""
        with self._pending_lock:
            self._pending.extend(self._pool.submit(self._put_one, r, False) for r in batch)

    def wait(self) -> None:
        """Block until every queued write has reached the file, then make the file consistent on disk."""
        while True:
            with self._pending_lock:
                futs, self._pending = self._pending, []
            if not futs:
                break
            for f in futs:
                f.result()
        self.flush()

    def flush(self) -> None:
        if self.lib.h5s_flush(self.h) != 0:
            raise IOError(f"HDF5 flush failed: {self._err()}")

    # ------------------------------------------------------------------ reading
    def load_id(self, convo_id: int) -> tuple[np.ndarray, np.ndarray | None]:
        """(float32 log-probs [Lc, K], int64 ids [Lc, K] or None) like the reference's ``_load_id`` (:315-329)."""
        v16, i32 = self.load_id_raw(convo_id)
        return v16.astype(np.float32), None if i32 is None else i32.astype(np.int64)

    def load_id_raw(self, convo_id: int) -> tuple[np.ndarray, np.ndarray | None]:
        r, c, hi = c_longlong(), c_longlong(), c_int()
        if self.lib.h5s_shape(self.h, int(convo_id), ctypes.byref(r), ctypes.byref(c), ctypes.byref(hi)) != 0:
            raise ValueError(self._err() or f"Convo ID {convo_id} not found in dataset.")
        v = np.empty((r.value, c.value), dtype=np.float16)
        ix = np.empty((r.value, c.value), dtype=np.uint32) if hi.value else None
        if self.lib.h5s_get(self.h, int(convo_id), v.ctypes.data_as(c_void_p), None if ix is None else ix.ctypes.data_as(c_void_p)) != 0:
            raise IOError(f"HDF5 read of convo_{convo_id} failed: {self._err()}")
        return v, ix

    def make_batch(self, batch_ids: list[int], sort_ids: bool = False, pinned: bool = False) -> dict:
        """Zero-padded batch: ``values`` float32 [B, Lmax, K], ``indices`` list of int64 [Lc, K] (or None),
        ``lengths`` true row counts. With ``sort_ids`` every row's (ids, values) are reordered by ascending id."""
        loaded = [self.load_id(i) for i in batch_ids]
        lengths = [len(v) for v, _ in loaded]
        lmax, K = max(lengths), loaded[0][0].shape[1]
        if pinned:
            import torch
            vals_t = torch.zeros((len(loaded), lmax, K), dtype=torch.float32).pin_memory()
            vals = vals_t.numpy()
        else:
            vals = np.zeros((len(loaded), lmax, K), dtype=np.float32)
        idx_out = []
        for b, (v, ix) in enumerate(loaded):
            if sort_ids and ix is not None:
                order = np.argsort(ix, axis=1, kind="stable")
                ix = np.take_along_axis(ix, order, 1)
                v = np.take_along_axis(v, order, 1)
            vals[b, : len(v)] = v
            idx_out.append(ix)
        return {"ids": list(batch_ids), "values": vals, "indices": idx_out, "lengths": lengths}

    def get_batch(self, batch_ids: list[int], **kw) -> dict:
        return self.make_batch(batch_ids, **kw)

    # ---- prefetch: one background worker drains a to-do list of batches into the bounded result queue
    def _worker(self, stop: threading.Event) -> None:
        cyc = 0
        while not stop.is_set():
            with self._todo_cv:
                while not self._todo and self._cycle is None and not stop.is_set():
                    self._todo_cv.wait(timeout=0.05)
                if stop.is_set():
                    return
                if self._todo:
                    ids, kw = self._todo.pop(0)
                else:
                    batches, kw = self._cycle
                    ids = batches[cyc % len(batches)]
                    cyc += 1
            try:
                item = self.make_batch(ids, **kw)
            except Exception as e:  # noqa: BLE001 - surfaced to the consumer by read_next_batch
                item = e
            while not stop.is_set():
                try:
                    self.result_queue.put(item, timeout=0.05)
                    break
                except queue.Full:
                    continue

    def _ensure_worker(self) -> None:
        t = self._prefetch_thread
        if t is None or not t.is_alive():
            self._stop = threading.Event()
            self._prefetch_thread = threading.Thread(target=self._worker, args=(self._stop,), name="h5-prefetch",
                                                     daemon=True)
            self._prefetch_thread.start()

    def enqueue_get_batches(self, batches: list[list[int]], **kw) -> None:
        """Queue one pass over ``batches`` (appended behind what is already queued); fetch each with
        ``read_next_batch``. Reads, inflation and padding happen in the background."""
        with self._todo_cv:
            self._todo.extend((list(ids), kw) for ids in batches)
            self._todo_cv.notify_all()
        self._ensure_worker()

    def read_only_mode(self, batches: list[list[int]], **kw) -> None:
        """Cycle over ``batches`` forever (validation)."""
        with self._todo_cv:
            self._cycle = ([list(b) for b in batches], kw)
            self._todo_cv.notify_all()
        self._ensure_worker()

    def read_next_batch(self, timeout: float | None = 300.0) -> dict:
        item = self.result_queue.get(timeout=timeout)
        if isinstance(item, Exception):
            raise item
        return item

    def stop_prefetch(self) -> None:
        self._stop.set()
        with self._todo_cv:
            self._todo.clear()
            self._cycle = None
            self._todo_cv.notify_all()
        t = self._prefetch_thread
        while t is not None and t.is_alive():
            try:
                self.result_queue.get_nowait()
            except queue.Empty:
                pass
            t.join(timeout=0.05)
        while True:
            try:
                self.result_queue.get_nowait()
            except queue.Empty:
                break
        self._prefetch_thread = None

    # ------------------------------------------------------------------ metadata
    def get_dataset_ids(self) -> list[int]:
        n = self.lib.h5s_count(self.h)
        buf = (c_longlong * max(1, n))()
        n = self.lib.h5s_list_ids(self.h, buf, n)
        return [int(buf[i]) for i in range(n)]

    def _attr(self, convo_id: int, name: str) -> str | None:
        n = self.lib.h5s_get_attr_str(self.h, int(convo_id), name.encode(), None, 0)
        if n < 0:
            return None
        buf = ctypes.create_string_buffer(n + 1)
        self.lib.h5s_get_attr_str(self.h, int(convo_id), name.encode(), buf, n + 1)
        return buf.raw[:n].decode("utf-8", "replace")

    def get_sha(self, convo_id: int) -> str | None:
        return self._attr(convo_id, "content_sha")

    def get_available_shas(self) -> dict[int, str]:
        self.wait()
        return {i: (self.get_sha(i) or "") for i in self.get_dataset_ids()}

    def update_shas(self, shas: dict) -> None:
        self.wait()
        for cid, sha in shas.items():
            if self.lib.h5s_has(self.h, int(cid)):
                self.lib.h5s_update_sha(self.h, int(cid), str(sha).encode())
        self.flush()

    def get_dataset_attr(self, attr: str):
        s = self._attr(-1, attr)
        if s is not None:
            return s
        v = c_longlong()
        if self.lib.h5s_get_root_attr_int(self.h, attr.encode(), ctypes.byref(v)) == 0:
            return int(v.value)
        return None

    def set_dataset_attr(self, attr: str, value) -> None:
        if isinstance(value, (int, np.integer)) and not isinstance(value, bool):
            self.lib.h5s_set_root_attr_int(self.h, attr.encode(), int(value), 0)
        else:
            self.lib.h5s_set_root_attr_str(self.h, attr.encode(), str(value).encode())
        self.flush()

    def get_vocab_family(self) -> str | None:
        self.wait()
        return self._attr(-1, "vocab_family")

    def set_vocab_family(self, vocab_family: str) -> None:
        self.wait()
        self.set_dataset_attr("vocab_family", str(vocab_family))

    def get_topk(self) -> int | None:
        self.wait()
        v = c_longlong()
        return int(v.value) if self.lib.h5s_get_root_attr_int(self.h, b"topk", ctypes.byref(v)) == 0 else None

    def set_topk(self, topk: int) -> None:
        self.wait()
        self.set_dataset_attr("topk", int(topk))

    def has_data(self) -> bool:
        self.wait()
        return self.lib.h5s_count(self.h) > 0

    # ------------------------------------------------------------------ maintenance
    def purge_dataset(self, ask_confirmation: bool = True, confirm=None) -> None:
        """Deletes every conversation and the file-level ``vocab_family`` / ``topk`` attributes (:356-368)."""
        if ask_confirmation:
            if not self._confirm("The script is going to delete all distributions from the h5 dataset.\n"
                                 "Are you sure you want to proceed? (y/n):", confirm):
                raise ValueError("User cancelled operation.")
        self.wait()
        self.stop_prefetch()
        for cid in self.get_dataset_ids():
            self.lib.h5s_delete(self.h, cid)
        self.lib.h5s_set_root_attr_str(self.h, b"vocab_family", None)
        self.lib.h5s_set_root_attr_int(self.h, b"topk", 0, 1)
        self.flush()
        self.compact_if_wasteful()

    def delete_ids(self, ids: list[int], confirm=None) -> None:
        if not ids:
            return
        if not self._confirm(f"The script called for deletion of {len(ids)} samples from the {self.manager_name}h5 "
                             f"dataset.\nAre you sure you want to proceed? (y/n):", confirm):
            raise ValueError("User cancelled operation.")
        self.wait()
        for cid in ids:
            self.lib.h5s_delete(self.h, int(cid))
        self.flush()

    def rename_ids(self, ids_to_rename: dict[int, int], confirm=None) -> None:
        if not ids_to_rename:
            return
        if not self._confirm(f"The script called for renaming of {len(ids_to_rename)} samples in the {self.manager_name}"
                             f"h5 dataset.\nAre you sure you want to proceed? (y/n):", confirm):
            raise ValueError("User cancelled operation.")
        self.wait()
        n = len(ids_to_rename)
        old = (c_longlong * n)(*[int(k) for k in ids_to_rename])
        new = (c_longlong * n)(*[int(v) for v in ids_to_rename.values()])
        if self.lib.h5s_rename_many(self.h, old, new, n) != 0:
            raise IOError(f"rename failed: {self._err()}")
        self.flush()

    def sync(self, ids_to_delete, ids_to_rename, confirm=None) -> None:
        self.delete_ids(list(ids_to_delete), confirm=confirm)
        self.rename_ids(dict(ids_to_rename), confirm=confirm)

    def file_bytes(self) -> int:
        return int(self.lib.h5s_file_bytes(self.h))

    def repack(self) -> None:
        """Rewrite the file without the dead space left by deletions / replacements."""
        import os
        self.wait()
        tmp = self.file_path + ".repack"
        if os.path.exists(tmp):
            os.remove(tmp)
        if self.lib.h5s_repack(self.h, tmp.encode()) != 0:
            raise IOError(f"repack failed: {self._err()}")
        self.lib.h5s_close(self.h)
        os.replace(tmp, self.file_path)
        err = ctypes.create_string_buffer(512)
        self.h = self.lib.h5s_open(self.file_path.encode(), 1, err, 512)
        if not self.h:
            raise IOError(f"cannot reopen {self.file_path}: {err.value.decode()}")

    def compact_if_wasteful(self, min_bytes: int = 64 << 20) -> None:
        if self.lib.h5s_count(self.h) == 0 and self.file_bytes() > min_bytes:
            self.repack()

    def reopen(self) -> None:
        """Drop this handle's view of the file and read it again (another process has written to it)."""
        cycle = self._cycle              # a validation cycle set up earlier goes on after the reopen, from its first batch
        self.stop_prefetch()
        self.wait()
        self.lib.h5s_close(self.h)
        err = ctypes.create_string_buffer(512)
        self.h = self.lib.h5s_open(self.file_path.encode(), 1, err, 512)
        if not self.h:
            raise IOError(f"cannot reopen {self.file_path}: {err.value.decode()}")
        if cycle is not None:
            self.read_only_mode(cycle[0], **cycle[1])

    def close(self) -> None:
        if self.closed:
            return
        self.closed = True
        self.stop_prefetch()
        try:
            self.wait()
        finally:
            self._pool.shutdown(wait=True)
            self.lib.h5s_close(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


H5DataManager = H5Store  # the reference's name for this role
