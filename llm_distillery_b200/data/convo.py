"""Per-conversation carriers (reference: classes/data_classes.py).

``ConvoTokenized`` is one tokenised sample padded to ``context_len`` with its content ranges; its ``content_sha``
is the key that keeps the HDF5 cache in sync with the text dataset. ``TeacherRows`` carries one conversation's
collected distribution (content rows only) from the collector to the HDF5 store - by reference, inside one
process; there is no shared-memory hop.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field

import numpy as np


def content_sha(tokens: np.ndarray, content_ranges: list[tuple[int, int]]) -> str:
    """SHA-256 over the decimal strings of tokens[start+1:end] of every range, concatenated without separators
    (data_classes.py:59-62). Byte-compatible with datasets written by the reference."""
    h = hashlib.sha256()
    for start, end in content_ranges:
        h.update("".join(map(str, tokens[start + 1:end].tolist())).encode())
    return h.hexdigest()


class ConvoTokenized:
    __slots__ = ("tokenized", "content_ranges", "padding", "cropped_end", "length", "len_content", "content_sha",
                 "origin_convo_id", "sample")

    def __init__(self, tokenized: np.ndarray, content_ranges, padding: int, cropped_end: bool, convo_id: int,
                 sample: str = ""):
        self.tokenized = tokenized
        self.content_ranges = [(int(s), int(e)) for s, e in content_ranges]
        self.padding = int(padding)
        self.cropped_end = bool(cropped_end)
        self.length = len(tokenized) - self.padding
        self.len_content = sum(e - s for s, e in self.content_ranges)
        self.content_sha = content_sha(tokenized, self.content_ranges)
        self.origin_convo_id = int(convo_id)
        self.sample = sample

    def content_indices(self) -> np.ndarray:
        """Positions whose next-token distribution is collected / trained on, in order."""
        if not self.content_ranges:
            return np.zeros(0, dtype=np.int64)
        return np.concatenate([np.arange(s, e, dtype=np.int64) for s, e in self.content_ranges])

    def ce_indices(self, context_len: int) -> tuple[np.ndarray, np.ndarray]:
        """Token positions of the labels for the content rows, and the content-row indices to leave out of the
        cross-entropy term (last row of every range when there are several). Reference:
        classes/student/model.py:93-116."""
        ce, avoid = [], []
        row = 0
        many = len(self.content_ranges) > 1
        for s, e in self.content_ranges:
            if s + 1 > context_len:
                continue
            ce.append(np.arange(s + 1, e + 1, dtype=np.int64))
            last = row + (e - s) - 1
            if many:
                avoid.append(last)
            row = last + 1
        ce_idx = np.concatenate(ce) if ce else np.zeros(0, dtype=np.int64)
        if len(ce_idx) and ce_idx[-1] >= self.length:
            ce_idx = ce_idx[:-1]
            if avoid:
                avoid.pop()
        return ce_idx, np.asarray(avoid, dtype=np.int64)


@dataclass
class TeacherRows:
    """Collected distribution of one conversation: ``values`` [Lc, K] (or [Lc, Vc] when top-K is off) natural-log
    probabilities, ``indices`` [Lc, K] token ids (None for full distributions)."""
    convo_id: int
    values: np.ndarray
    indices: np.ndarray | None
    content_sha: str = ""
    sample: str = ""
    meta: dict = field(default_factory=dict)


# Rows of a teacher that is not the last one of the run are stored under a marked SHA: the conversation only counts as
# collected (its SHA equals the dataset's) once the last teacher has merged its rows. A run killed between two teachers
# leaves marked conversations, which the next run's sync sees as changed and collects again from the first teacher on.
PARTIAL_SHA_PREFIX = "partial:"

