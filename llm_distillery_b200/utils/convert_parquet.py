"""Parquet shards -> one JSONL file (reference: utils/convert_parquet.py): shards matching a glob are concatenated,
values that JSON cannot carry are converted (bytes and uint8 arrays -> base64, numpy scalars/arrays -> Python,
timestamps -> ISO strings, nested containers recursively), and a one-line-per-field preview is returned.

    python -m llm_distillery_b200.utils.convert_parquet 'train-*.parquet'
"""
from __future__ import annotations

import base64
import glob
import json
import os
import sys


def jsonable(x):
    import numpy as np
    import pandas as pd
    if isinstance(x, (bytes, bytearray)):
        return base64.b64encode(bytes(x)).decode("utf-8")
    if isinstance(x, np.generic):
        return x.item()
    if isinstance(x, np.ndarray):
        if x.dtype == object:
            return [jsonable(v) for v in x]
        if x.dtype == np.uint8:
            return base64.b64encode(x.tobytes()).decode("utf-8")
        return x.tolist()
    if isinstance(x, pd.Timestamp):
        return x.isoformat()
    if isinstance(x, (dict, pd.Series)):
        return {k: jsonable(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [jsonable(v) for v in x]
    return x


def convert_parquet_to_jsonl(parquet_pattern: str, jsonl_path: str | None = None) -> tuple[str, str]:
    import pandas as pd
    files = sorted(glob.glob(parquet_pattern))
    if not files:
        raise FileNotFoundError(f"No files found for pattern: {parquet_pattern}")
    df = pd.concat([pd.read_parquet(f) for f in files], ignore_index=True)
    jsonl_path = jsonl_path or os.path.splitext(files[-1])[0].replace("-00000-of", "") + ".jsonl"
    first = None
    with open(jsonl_path, "w", encoding="utf-8") as f:
        for rec in df.to_dict(orient="records"):
            row = {k: jsonable(v) for k, v in rec.items()}
            first = first or row
            f.write(json.dumps(row, ensure_ascii=False) + "\n")
    crop = lambda v: v[:50] if isinstance(v, str) and len(v) > 50 else v  # noqa: E731
    preview = "\n ".join(f"{k}: {crop(v)}" for k, v in (first or {}).items())
    return jsonl_path, preview


if __name__ == "__main__":
    path, fmt = convert_parquet_to_jsonl(sys.argv[1])
    print(f"Conversion complete: {path}\nDataset format:\n {fmt}")
