"""Console progress bars with status postfixes.

The reference's console UI is nested tqdm bars - Teachers / Convos while collecting (classes/teacher/model.py:81-99),
Epochs / Chunks / Training while distilling - whose postfix says what the worker is busy with ("Loading model...",
"Saving state...", classes/student/model.py:81-85, 119, 226, 260, 271, 283). ``progress`` makes a bar, ``status`` sets
and clears such a postfix around a block, and the latest status of the process is kept for the heartbeat records and
the tests (bars are disabled when stderr is not a terminal).
"""
from __future__ import annotations

import os
import sys
from contextlib import contextmanager

from tqdm import tqdm

_LAST_STATUS = [""]
_HISTORY: list[str] = []


def progress(iterable=None, **kw):
    kw.setdefault("smoothing", 0.06)
    kw.setdefault("disable", bool(os.environ.get("B200_NO_PROGRESS")) or not sys.stderr.isatty())
    return tqdm(iterable, **kw)


def last_status() -> str:
    return _LAST_STATUS[0]


def status_history() -> list[str]:
    """Every status text set so far in this process, oldest first (bounded)."""
    return list(_HISTORY)


def set_status(bar, text: str) -> None:
    _LAST_STATUS[0] = text
    if text:
        _HISTORY.append(text)
        del _HISTORY[:-200]
    if bar is not None:
        bar.set_postfix_str(text)


@contextmanager
def status(bar, text: str):
    """``with status(bar, "Saving state..."):`` - the postfix is shown for the duration of the block."""
    set_status(bar, text)
    try:
        yield
    finally:
        set_status(bar, "")
