"""JSONL dataset reading. Schema per line (reference: utils/dataset_converter.py:39-44, dataset_utils.py:92-153):
``{"init": str, "conversations": [{"from": "human"|"gpt", "value": str}, ...], "source": str, "tags": [str]}``.
A sample's id is its 0-based line index among the lines that parse."""
from __future__ import annotations

import json
from typing import Iterator


def read_jsonl_lazy(file_path: str) -> Iterator[dict]:
    with open(file_path, "r", encoding="utf-8") as f:
        for line_number, line in enumerate(f, 1):
            if not line.strip():
                continue
            try:
                yield json.loads(line)
            except json.JSONDecodeError as e:
                print(f"Skipping malformed JSON on line {line_number}: {e.msg}. Line content: {line.strip()[:200]}")


def read_jsonl(file_path: str) -> list[dict]:
    return list(read_jsonl_lazy(file_path))


def write_jsonl(file_path: str, rows) -> None:
    with open(file_path, "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
