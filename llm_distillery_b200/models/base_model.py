"""Model metadata shared by the teacher and student roles (reference: classes/base_model.py).

A model folder carries two sidecar files next to the HF weights: ``prompt_format.json`` (the six prompt-format
strings) and ``pipeline_config.json`` ({batch_size, add_bos, seq_chunk_len, completion}). The reference asks for
missing ones on stdin; here they are filled with the same defaults and written back, and the prompts are shown
only with ``interactive=True``.
"""
from __future__ import annotations

import codecs
import json
import os

from ..config import DEFAULT_PROMPT_FORMAT, TRUE_WORDS
from ..data.vocab import get_vocab_family, vocab_identity
from ..ckpt.hf import is_model_safetensors

DEFAULT_PIPELINE_CONFIG = {"batch_size": 1, "add_bos": True, "seq_chunk_len": 256, "completion": False}


def load_prompt_format(model_path: str):
    p = os.path.join(model_path, "prompt_format.json")
    if not os.path.exists(p):
        return None
    with open(p, "r", encoding="utf-8") as f:
        return json.load(f)


def save_prompt_format(prompt_format: dict, save_folder: str) -> None:
    with open(os.path.join(save_folder, "prompt_format.json"), "w", encoding="utf-8") as f:
        json.dump(prompt_format, f, ensure_ascii=False, indent=4)


def load_config(model_path: str):
    p = os.path.join(model_path, "pipeline_config.json")
    if not os.path.exists(p):
        return None
    with open(p, "r", encoding="utf-8") as f:
        return json.load(f)


def save_config(config: dict, model_path: str) -> None:
    with open(os.path.join(model_path, "pipeline_config.json"), "w", encoding="utf-8") as f:
        json.dump(config, f, ensure_ascii=False, indent=4)


def _ask(defaults: dict, title: str, parse) -> dict:
    out = dict(defaults)
    keys = list(out)
    print(f"{title}, use '<' to go back a step.")
    i = 0
    while i < len(keys):
        k = keys[i]
        shown = out[k].encode("unicode_escape").decode() if isinstance(out[k], str) else out[k]
        raw = input(f"{k} (default: {shown}): ")
        if raw == "<":
            i = max(0, i - 1)
        elif raw == "":
            i += 1
        else:
            try:
                out[k] = parse(defaults[k], raw)
                i += 1
            except ValueError:
                print(f"Enter a valid value for {k}.")
    return out


def input_prompt_format() -> dict:
    return _ask(DEFAULT_PROMPT_FORMAT, "Enter the prompt format", lambda d, raw: codecs.decode(raw, "unicode_escape"))


def input_config() -> dict:
    def parse(default, raw):
        if isinstance(default, bool):
            return raw.lower() in TRUE_WORDS
        if isinstance(default, int):
            return int(raw)
        return raw
    return _ask(DEFAULT_PIPELINE_CONFIG, "Enter the model config", parse)


class BaseModel:
    def __init__(self, model_path: str, student: bool = False, interactive: bool = False):
        self.student = student
        self.model_path = model_path
        self.model_name = ""
        self.device = "cuda:0"
        self.prompt_format: dict = {}
        self.completion = False
        self.batch_size = 0
        self.add_bos = False
        self.context_len = 0
        self.seq_chunk_len = 0
        self.dataset = []
        self.dataset_len = 0
        self.dataset_sorted = False
        self.validation_dataset = []
        self.validation_dataset_batched = []
        self.validation_dataset_len = 0
        self.validation_dataset_sorted = False
        self.vocab_family = ""
        self.vocab_id = ""
        self.temperature = 1.0
        self.crop_to_size = 0
        self.enable_topK = False
        self.topK = 0
        self.interactive = interactive
        self._prepare()

    def _prepare(self) -> None:
        self.model_name = os.path.basename(os.path.normpath(self.model_path))
        if os.path.exists(f"{self.model_path}_safetensors"):
            self.model_path = f"{self.model_path}_safetensors"
        if not is_model_safetensors(self.model_path):
            from ..utils.convert_to_safetensor import convert_model
            self.model_path = convert_model(self.model_path)
        pf = load_prompt_format(self.model_path)
        if pf is None:
            pf = input_prompt_format() if self.interactive else dict(DEFAULT_PROMPT_FORMAT)
            save_prompt_format(pf, self.model_path)
        cfg = load_config(self.model_path)
        if cfg is None:
            cfg = input_config() if self.interactive else dict(DEFAULT_PIPELINE_CONFIG)
            save_config(cfg, self.model_path)
        self.prompt_format = pf
        self.batch_size = cfg.get("batch_size", 1)
        self.add_bos = cfg.get("add_bos", True)
        self.completion = cfg.get("completion", False)
        self.seq_chunk_len = cfg.get("seq_chunk_len", 256)
        self.vocab_family = get_vocab_family(model_path=self.model_path)
        self.vocab_id = vocab_identity(model_path=self.model_path)

    # ---- debugging dumps of the tokenised datasets (reference: base_model.py:184-218)
    def _dump(self, convos, folder: str, stem: str) -> None:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(self.model_path)
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, f"{stem}.jsonl"), "w", encoding="utf-8") as f, \
                open(os.path.join(folder, f"content_{stem}.jsonl"), "w", encoding="utf-8") as fc:
            for c in convos:
                d = {"tokenized": c.tokenized.tolist(), "decoded": [tok.decode(c.tokenized)],
                     "content_ranges": c.content_ranges,
                     "content_indices": [list(range(s, e)) for s, e in c.content_ranges],
                     "content_decoded": [tok.decode(c.tokenized[s:e]) for s, e in c.content_ranges],
                     "padding": c.padding, "cropped_end": c.cropped_end, "origin_convo_id": c.origin_convo_id}
                f.write(json.dumps(d, ensure_ascii=False) + "\n")
                d.pop("tokenized")
                fc.write(json.dumps(d, ensure_ascii=False) + "\n")

    def write_dataset_to_file(self, folder: str) -> None:
        self._dump(self.dataset, folder, "tokenized_dataset")

    def write_validation_dataset_to_file(self, folder: str) -> None:
        self._dump(self.validation_dataset, folder, "tokenized_validation_dataset")
