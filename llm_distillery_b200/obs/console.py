"""Console progress bars (the reference's "console UI" is nested tqdm bars with status postfixes)."""
from __future__ import annotations

import os
import sys

from tqdm import tqdm


def progress(iterable=None, **kw):
    kw.setdefault("smoothing", 0.06)
    kw.setdefault("disable", bool(os.environ.get("B200_NO_PROGRESS")) or not sys.stderr.isatty())
    return tqdm(iterable, **kw)
