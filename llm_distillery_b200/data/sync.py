"""Keeping the HDF5 cache in step with the text dataset by per-conversation content SHA
(reference: collect_and_finetune.py:211-315).

Equal SHAs are matched as a multiset: surplus copies on disk are removed, missing ones are collected, and
matched pairs whose ids differ are renamed - so a reordered or de-duplicated dataset is renamed on disk instead
of being recollected. A vocabulary-family mismatch (or a file without one) recollects everything.
Unlike the reference, pairing is deterministic: ids are matched in ascending order, and ids that already agree
are kept in place before anything is renamed.
"""
from __future__ import annotations


def match_shas(disk_sha: dict, current_sha: dict):
    """disk_sha / current_sha: {id -> sha}. Returns (ids_to_collect, ids_to_rename{old->new}, ids_to_remove)."""
    disk, cur = {}, {}
    for i, s in disk_sha.items():
        disk.setdefault(s, set()).add(int(i))
    for i, s in current_sha.items():
        cur.setdefault(s, set()).add(int(i))
    collect, remove, rename = [], [], {}
    for sha in set(disk) | set(cur):
        d, c = disk.get(sha, set()), cur.get(sha, set())
        keep = d & c                      # already in place
        d_rest, c_rest = sorted(d - keep), sorted(c - keep)
        n = min(len(d_rest), len(c_rest))
        for old, new in zip(d_rest[:n], c_rest[:n]):
            rename[old] = new
        remove.extend(d_rest[n:])
        collect.extend(c_rest[n:])
    return sorted(collect), rename, sorted(remove)


def calculate_sync(student_dataset, store, student_vocab_family: str):
    """What to collect / rename / remove so that ``store`` matches ``student_dataset``."""
    current = {c.origin_convo_id: c.content_sha for c in student_dataset}
    disk = store.get_available_shas()
    family = store.get_vocab_family()
    if family is None:
        return sorted(current), {}, sorted(int(i) for i in disk)
    if family != student_vocab_family:
        print("Vocab family mismatch between the current models and the dataset on disk!\n"
              "All data will be recollected using the new vocab family.")
        return sorted(current), {}, sorted(int(i) for i in disk)
    return match_shas(disk, current)


def sync_datasets(validation_store, store, rebase: bool, student, use_teachers: bool, confirm=None):
    """Applies the sync to both stores; returns (ids_collect, ids_collect_val)."""
    if rebase:
        store.update_shas({c.origin_convo_id: c.content_sha for c in student.dataset})
        validation_store.update_shas({c.origin_convo_id: c.content_sha for c in student.validation_dataset})
        store.set_vocab_family(student.vocab_family)
        validation_store.set_vocab_family(student.vocab_family)
        return [], []
    if not use_teachers:
        return [], []
    c, rn, rm = calculate_sync(student.dataset, store, student.vocab_family)
    cv, rnv, rmv = calculate_sync(student.validation_dataset, validation_store, student.vocab_family)
    store.sync(rm, rn, confirm=confirm)
    validation_store.sync(rmv, rnv, confirm=confirm)
    return c, cv
