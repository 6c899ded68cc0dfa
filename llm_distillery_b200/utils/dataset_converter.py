"""Rewrite public dataset schemas into the pipeline's JSONL schema
``{"init": str, "conversations": [{"from": "human"|"gpt", "value": str}], "source": str, "tags": [str]}``.

Covers the nine source formats of the reference's converter (utils/dataset_converter.py:30-199) as a registry of
small field mappers; random choices (separator between instruction and input, dropping system prompts) take a
seeded generator so a conversion is reproducible.

    python -m llm_distillery_b200.utils.dataset_converter INPUT.jsonl --format sharegpt [--sort] [--seed 0]
"""
from __future__ import annotations

import argparse
import json
import os
import random
from typing import Callable

Sample = dict
_FORMATS: dict[str, Callable] = {}


def _register(name):
    def deco(fn):
        _FORMATS[name] = fn
        return fn
    return deco


def _pair(user: str, assistant: str, source: str, init: str = "", tags=None) -> Sample:
    return {"init": init, "conversations": [{"from": "human", "value": user}, {"from": "gpt", "value": assistant}],
            "source": source, "tags": list(tags or [])}


@_register("alpaca_gpt4")
def alpaca_gpt4(s, source, rng):
    sep = "\n" if rng.random() < 0.5 else " "
    user = s["instruction"] if not s.get("input") else f"{s['instruction']}{sep}{s['input']}"
    return _pair(user, s["output"], source)


@_register("codefeedback")
def codefeedback(s, source, rng):
    return _pair(s["query"], s["answer"], source)


@_register("multitask")
def multitask(s, source, rng):
    return _pair(s["prompt"], s["chosen"], source, init=s.get("system", ""))


@_register("dolly")
def dolly(s, source, rng):
    instruction, context, response = s["instruction"].strip(), s["context"].strip(), s["response"].strip()
    sep = rng.choice(["\n", " ", "  ", "  ", "\n\n", "\n\n\n", " | "])
    return _pair(instruction if not context else f"{context}{sep}{instruction}", response, source)


@_register("gpt_roleplay")
def gpt_roleplay(s, source, rng):
    out = []
    for chat in s.get("dialogues", []) or []:
        turns = [{"from": "gpt", "value": s["greeting"]}] if s.get("greeting") else []
        turns += [{"from": "gpt" if t["role"] == "char" else "human", "value": t["content"]} for t in chat["chat"]]
        out.append({"init": s.get("context") or "", "conversations": turns, "source": source, "tags": []})
    return out or None


@_register("random_samples")
def random_samples(s, source, rng):
    return {"init": "", "conversations": [{"from": "human", "value": s["text"]}], "source": source, "tags": ["completion"]}


@_register("sharegpt")
def sharegpt(s, source, rng, drop_system_probability: float = 0.75):
    system, turns = "", []
    for t in s["conversations"]:
        if t["from"] == "system":
            system = t["value"]
        else:
            turns.append({"from": t["from"], "value": t["value"]})
    if rng.random() < drop_system_probability:
        system = ""
    return {"init": system, "conversations": turns, "source": source, "tags": []}


@_register("magpie_reasoning")
def magpie_reasoning(s, source, rng):
    return _pair(s["instruction"], s["response"], source)


@_register("custom")
def custom(s, source, rng):
    """The pipeline's older format: conversations is a list of strings alternating human / gpt ("reversed" flips)."""
    tags = s.get("tags", [])
    flip = "reversed" in tags or s.get("reversed", False)
    turns = [{"from": "gpt" if ((i + 1) % 2 if flip else i % 2) else "human", "value": text}
             for i, text in enumerate(s["conversations"])]
    return {"init": s.get("init", ""), "conversations": turns, "source": s.get("source", source), "tags": tags}


def available_formats() -> list[str]:
    return sorted(_FORMATS)


def convert_samples(samples, fmt: str, source: str, seed: int = 0, sort: bool = False) -> list[Sample]:
    if fmt not in _FORMATS:
        raise ValueError(f"unknown format {fmt}; available: {available_formats()}")
    rng = random.Random(seed)
    out = []
    for s in samples:
        r = _FORMATS[fmt](s, source, rng)
        if r is None:
            continue
        out.extend(r if isinstance(r, list) else [r])
    if sort:
        out.sort(key=lambda x: sum(len(t["value"]) for t in x["conversations"]))
    return out


def rewrite_dataset(input_path: str, output_path: str | None, fmt: str, dataset_name: str | None = None,
                    sort: bool = True, seed: int = 0) -> str:
    name = dataset_name or os.path.basename(input_path).split(".")[0]
    output_path = output_path or os.path.join(os.path.dirname(input_path), f"Converted_{name}.jsonl")
    with open(input_path, "r", encoding="utf-8") as f:
        samples = [json.loads(line) for line in f if line.strip()]
    with open(output_path, "w", encoding="utf-8") as f:
        for s in convert_samples(samples, fmt, name, seed, sort):
            f.write(json.dumps(s, ensure_ascii=False) + "\n")
    return output_path


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("input")
    ap.add_argument("--format", required=True, choices=available_formats())
    ap.add_argument("--output")
    ap.add_argument("--name")
    ap.add_argument("--sort", action="store_true")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    print(rewrite_dataset(a.input, a.output, a.format, a.name, a.sort, a.seed))
