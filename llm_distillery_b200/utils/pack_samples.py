"""Pack short completion samples into context-length documents (reference: utils/pack_samples.py).

Rule: take the shortest remaining sample, then keep appending the LONGEST remaining sample that still fits
``context_len`` (counting the ``eos + bos`` separator) until the document reaches ``min_desired_len`` or nothing
fits; samples longer than the context stay alone. Output is sorted by packed length, longest first, with an
``encoded_len`` field. The search for "longest that fits" is a bisection over a sorted length list.

    python -m llm_distillery_b200.utils.pack_samples INPUT.jsonl --model MODEL_DIR --context-len 8192 --min-len 7500
"""
from __future__ import annotations

import argparse
import bisect
import json
import os
from collections import defaultdict
from concurrent.futures import ThreadPoolExecutor


def plan_packing(lengths: list[int], context_len: int, min_desired_len: int, sep_len: int) -> list[list[int]]:
    """Groups of sample lengths; every input length appears in exactly one group."""
    pool = sorted(lengths)
    groups = []
    while pool:
        cur = pool.pop(0)
        group = [cur]
        total = cur
        if cur <= context_len:
            while total < min_desired_len and pool:
                room = context_len - total - sep_len
                j = bisect.bisect_right(pool, room) - 1
                if j < 0:
                    break
                nxt = pool.pop(j)
                group.append(nxt)
                total += sep_len + nxt
        groups.append(group)
    return groups


def prepack(input_path: str, output_path: str, tokenizer, context_len: int, min_desired_len: int, bos: str = "<s>",
            eos: str = "</s>", workers: int = 8) -> int:
    from ..data.tokenize import good_encode
    sep_len = len(good_encode(bos, tokenizer)) + len(good_encode(eos, tokenizer))
    with open(input_path, "r", encoding="utf-8") as f:
        data = [json.loads(line) for line in f if line.strip()]

    def text_of(s):
        c = s["conversations"][0]
        return c["value"] if isinstance(c, dict) else c

    with ThreadPoolExecutor(max_workers=workers) as ex:
        lens = list(ex.map(lambda s: len(good_encode(text_of(s), tokenizer)), data))
    by_len = defaultdict(list)
    for s, n in zip(data, lens):
        s["encoded_len"] = n
        by_len[n].append(s)
    out = []
    for group in plan_packing(lens, context_len, min_desired_len, sep_len):
        base = by_len[group[0]].pop()
        for n in group[1:]:
            other = by_len[n].pop()
            joined = text_of(base) + eos + bos + text_of(other)
            if isinstance(base["conversations"][0], dict):
                base["conversations"][0]["value"] = joined
            else:
                base["conversations"][0] = joined
            base["encoded_len"] += sep_len + n
        out.append(base)
    out.sort(key=lambda s: s["encoded_len"], reverse=True)
    with open(output_path, "w", encoding="utf-8") as f:
        for s in out:
            f.write(json.dumps(s, ensure_ascii=False) + "\n")
    return len(out)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("input")
    ap.add_argument("--model", required=True, help="folder with the tokenizer")
    ap.add_argument("--output")
    ap.add_argument("--context-len", type=int, default=8192)
    ap.add_argument("--min-len", type=int, default=7500)
    ap.add_argument("--bos", default="<s>")
    ap.add_argument("--eos", default="</s>")
    a = ap.parse_args()
    from ..data.tokenize import load_tokenizer
    outp = a.output or os.path.join(os.path.dirname(a.input), "Prepacked_" + os.path.basename(a.input))
    print(prepack(a.input, outp, load_tokenizer(a.model), a.context_len, a.min_len, a.bos, a.eos), "documents ->", outp)
