"""Tokenisation front-end: JSONL samples -> ``ConvoTokenized`` with content ranges.

Behavioural contract (reference: utils/dataset_utils.py:44-264): token layout
``[BOS?] [SYS_START sys SYS_END]? ([ROLE_START text ROLE_END])*`` zero-padded to ``context_len``; text is encoded
as ``encode("\\n" + text)[2:]`` to dodge sentencepiece's leading-space artefact; a content range (s, e) names the
positions whose *next-token* distribution is collected, so it starts one position before the first content token
and - for user / assistant turns - covers one token of the end marker. Without BOS all ranges shift by -1 and one
slot is kept free at the end (unless no model in the run adds BOS) so that over-long samples keep the same number
of content tokens whichever model tokenises them.

The builder below is a small state machine over an output buffer instead of the reference's inline index
arithmetic; tests compare it against the reference function on generated samples.
"""
from __future__ import annotations

import os
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass

import numpy as np

from .convo import ConvoTokenized
from .jsonl import read_jsonl
from .vocab import get_family_bos_id

PF_KEYS = ("SYS_START", "USER_START", "ASSISTANT_START", "SYS_END", "USER_END", "ASSISTANT_END")


def good_encode(text: str, tokenizer, encode_special: bool = False) -> np.ndarray:
    """``encode("\\n" + text)`` minus its first two ids. Works with any HF-style tokenizer (``encode(str,
    add_special_tokens=False) -> list[int]``)."""
    ids = tokenizer.encode("\n" + text, add_special_tokens=False)[2:]
    return np.asarray(ids, dtype=np.int64)


def encode_prompt_format(prompt_format: dict, tokenizer) -> dict[str, np.ndarray]:
    return {k: good_encode(v, tokenizer, encode_special=True) for k, v in prompt_format.items()}


@dataclass
class TokenizeSpec:
    """Everything that decides how one model sees the dataset."""
    context_len: int
    save_sys_range: bool = True
    save_user_range: bool = True
    save_assistant_range: bool = True
    model_completion: bool = False
    model_student: bool = False
    model_add_bos: bool = True
    ignore_model_type: bool = True
    all_not_add_bos: bool = False
    bos_token_id: int | None = None


class _Builder:
    """Output buffer with a write cursor that may run past the end (writes are clipped, the cursor is not)."""

    def __init__(self, spec: TokenizeSpec):
        self.ctx = spec.context_len
        self.buf = np.zeros(self.ctx, dtype=np.int64)
        self.ranges: list[tuple[int, int]] = []
        if spec.model_add_bos and spec.bos_token_id is not None:
            self.buf[0] = spec.bos_token_id
            self.n = 1          # tokens written
            self.shift = 0      # range positions are token positions + shift - 1 ... see range_start()
            self.end_crop = 0
        else:
            self.n = 0
            self.shift = -1
            self.end_crop = 0 if spec.all_not_add_bos else 1
        # position (in range coordinates) of the last token written so far
        self.last = self.shift

    def put(self, toks: np.ndarray, limit: int | None = None) -> None:
        limit = self.ctx if limit is None else limit
        room = max(0, limit - self.n)
        k = min(len(toks), room)
        if k > 0 and self.n < self.ctx:
            self.buf[self.n:self.n + k] = toks[:k]


def tokenize_sample(convo_id: int, item: dict, tokenizer, pf: dict[str, np.ndarray], spec: TokenizeSpec):
    """Returns (convo_id, tokens[context_len], content_ranges, num_tokens, empty)."""
    b = _Builder(spec)
    ctx = spec.context_len
    tags = item.get("tags", []) or []
    completion = "completion" in tags
    as_student = spec.model_student or spec.ignore_model_type
    convs = item.get("conversations", []) or []

    if completion:
        if not (spec.model_completion or as_student):
            return convo_id, b.buf, b.ranges, b.n, True
        first = convs[0] if convs else {}
        text = first.get("value", "") if isinstance(first, dict) else ""
        if not text:
            return convo_id, b.buf, b.ranges, b.n, True
        toks = good_encode(text.strip(), tokenizer)[: max(0, ctx - b.n - b.end_crop)]
        b.buf[b.n:b.n + len(toks)] = toks
        b.ranges.append((b.n, b.n + len(toks)))
        return convo_id, b.buf, b.ranges, b.n + len(toks), False
    if spec.model_completion and not as_student:
        return convo_id, b.buf, b.ranges, b.n, True
    if not convs:
        return convo_id, b.buf, b.ranges, b.n, True

    sys_text = item.get("init", "")
    if sys_text:
        body = good_encode(sys_text.strip(), tokenizer)
        block = np.concatenate([pf["SYS_START"], body, pf["SYS_END"]]).astype(np.int64)
        b.put(block)
        b.n += len(block)
        if spec.save_sys_range:
            b.ranges.append((len(pf["SYS_START"]) + b.last, b.n - len(pf["SYS_END"])))
        b.last = b.n - 1

    for turn in convs:
        speaker = turn.get("from", "")
        text = turn.get("value", "")
        if not speaker or not text:
            return convo_id, b.buf, b.ranges, b.n, True
        assistant = speaker == "gpt"
        start_t = pf["ASSISTANT_START"] if assistant else pf["USER_START"]
        end_t = pf["ASSISTANT_END"] if assistant else pf["USER_END"]
        body = good_encode(text.strip(), tokenizer)
        block = np.concatenate([start_t, body, end_t]).astype(np.int64)
        if (spec.save_assistant_range and assistant) or (spec.save_user_range and not assistant):
            cs = b.last + len(start_t)
            b.ranges.append((cs, cs + len(body) + 1))
        b.last += len(block)
        if b.n + len(block) > ctx:
            b.put(block, limit=ctx - b.end_crop)
            b.n = ctx - b.end_crop
            break
        b.put(block)
        b.n += len(block)

    if not b.ranges:
        return convo_id, b.buf, b.ranges, b.n, True
    empty = b.ranges[0][0] > ctx
    return convo_id, b.buf, b.ranges, b.n, empty


def load_tokenizer(model_path: str):
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(model_path, legacy=False)


def tokenize_items(items: dict[int, dict], tokenizer, prompt_format: dict, spec: TokenizeSpec,
                   workers: int | None = None) -> tuple[list[ConvoTokenized], set[int]]:
    """Tokenise {id: sample}. Threads are enough: HF fast tokenizers release the GIL inside ``encode``."""
    pf = encode_prompt_format(prompt_format, tokenizer)
    ctx = spec.context_len
    workers = workers or min(32, os.cpu_count() or 4)

    def one(kv):
        return tokenize_sample(kv[0], kv[1], tokenizer, pf, spec)

    if len(items) > 256 and workers > 1:
        with ThreadPoolExecutor(max_workers=workers) as ex:
            results = list(ex.map(one, items.items(), chunksize=64))
    else:
        results = [one(kv) for kv in items.items()]

    dataset, ids = [], set()
    for convo_id, toks, ranges, n, empty in results:
        if empty:
            continue
        fixed, cropped_end = [], False
        for s, e in ranges:
            if s > ctx:
                break
            if e > ctx:
                e, cropped_end = ctx, True
            fixed.append((s, e))
        dataset.append(ConvoTokenized(toks, fixed, ctx - n, cropped_end, convo_id, str(items[convo_id])))
        ids.add(convo_id)
    if not dataset:
        raise ValueError("No conversations were tokenized.\nIf you are using a completion model, make sure the "
                         "completion tag is present in the conversations of your dataset.")
    dataset.sort(key=lambda c: c.origin_convo_id)
    return dataset, ids


def tokenize_dataset(dataset_path: str, context_len: int, save_sys_range: bool, save_user_range: bool,
                     save_assistant_range: bool, model, ignore_model_type: bool, all_not_add_bos: bool,
                     tokenizer=None) -> tuple[list[ConvoTokenized], set[int]]:
    """Same signature role as the reference's ``tokenize_dataset`` (dataset_utils.py:199-264); ``model`` needs
    ``model_path, prompt_format, vocab_family, completion, student, add_bos``."""
    tokenizer = tokenizer or load_tokenizer(model.model_path)
    spec = TokenizeSpec(
        context_len=context_len, save_sys_range=save_sys_range, save_user_range=save_user_range,
        save_assistant_range=save_assistant_range, model_completion=model.completion, model_student=model.student,
        model_add_bos=model.add_bos, ignore_model_type=ignore_model_type, all_not_add_bos=all_not_add_bos,
        bos_token_id=get_family_bos_id(model.vocab_family, tokenizer))
    items = dict(enumerate(read_jsonl(dataset_path)))
    return tokenize_items(items, tokenizer, model.prompt_format, spec)
