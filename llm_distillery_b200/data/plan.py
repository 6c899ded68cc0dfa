"""Cache-size estimate and chunk plan (reference: collect_and_finetune.py:19-52).

On-disk size per content token: top-K stores an fp16 value and a 32-bit index per entry (6 bytes, assumed to
compress 1.7x under gzip-6); full distributions store 2 bytes per vocabulary entry (1.55x). The dataset is walked
in training order; a new chunk starts when the running estimate reaches ``max_cache_size_gb``.
"""
from __future__ import annotations

KB_PER_FP16 = 2.0 / 1024.0
TOPK_RATIO = 1.7
FULL_RATIO = 1.55


def kb_per_content_token(enable_topk: bool, save_topk: int, crop_to_size: int) -> float:
    if enable_topk:
        return (KB_PER_FP16 * 3) / TOPK_RATIO * save_topk
    return KB_PER_FP16 / FULL_RATIO * crop_to_size


def calculate_loop_ids(dataset, max_cache_size_gb: float, enable_topk: bool, save_topk: int, crop_to_size: int):
    """Returns (loop_ids, full_collect): lists of conversation ids per chunk, and whether one chunk holds all."""
    per_tok = kb_per_content_token(enable_topk, save_topk, crop_to_size)
    limit_kb = max_cache_size_gb * 1e6
    loop_ids: list[list[int]] = []
    chunk: list[int] = []
    running = 0.0
    for convo in dataset:
        running += per_tok * convo.len_content
        if running >= limit_kb:
            loop_ids.append(chunk)
            chunk = []
            running = 0.0
        chunk.append(convo.origin_convo_id)
    full_collect = not loop_ids
    if chunk:
        loop_ids.append(chunk)
    return loop_ids, full_collect


def estimate_dataset_gb(dataset, enable_topk: bool, save_topk: int, crop_to_size: int) -> float:
    per_tok = kb_per_content_token(enable_topk, save_topk, crop_to_size)
    return sum(per_tok * c.len_content for c in dataset) / 1e6
