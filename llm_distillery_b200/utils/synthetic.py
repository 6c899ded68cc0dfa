"""Synthetic fixtures that need no network: a sentencepiece-style byte-fallback BPE tokenizer trained on generated
text, random-init model folders in HF layout (with the pipeline sidecar files), and JSONL datasets in the
pipeline schema. Tests, the CPU plumbing run and the benchmarks build everything they need from here."""
from __future__ import annotations

import json
import os
import random
import string

import torch

WORDS = ("the quick brown fox jumps over lazy dog while seven wizards quietly judge boxing matches and pack my box "
         "with five dozen liquor jugs then sphinx of black quartz hears vow model token teacher student logit").split()


def random_text(rng: random.Random, n_words: int) -> str:
    out = []
    for _ in range(n_words):
        r = rng.random()
        if r < 0.8:
            out.append(rng.choice(WORDS))
        elif r < 0.9:
            out.append(str(rng.randint(0, 9999)))
        else:
            out.append("".join(rng.choice(string.ascii_letters) for _ in range(rng.randint(2, 8))))
    return " ".join(out)


def make_tokenizer(folder: str, vocab_size: int = 512, seed: int = 0, extra_merges_text: str = ""):
    """Llama-style tokenizer: "▁" word-boundary marker, BPE merges, <0xNN> byte fallback, <unk>/<s>/</s> = 0/1/2."""
    from tokenizers import Tokenizer, decoders, models, normalizers, trainers
    from transformers import PreTrainedTokenizerFast
    rng = random.Random(seed)
    tok = Tokenizer(models.BPE(unk_token="<unk>", byte_fallback=True, fuse_unk=True))
    tok.normalizer = normalizers.Sequence([normalizers.Prepend("▁"), normalizers.Replace(" ", "▁")])
    tok.decoder = decoders.Sequence([decoders.Replace("▁", " "), decoders.ByteFallback(), decoders.Fuse(),
                                     decoders.Strip(" ", 1, 0)])
    specials = ["<unk>", "<s>", "</s>"] + [f"<0x{i:02X}>" for i in range(256)]
    trainer = trainers.BpeTrainer(vocab_size=vocab_size, special_tokens=specials, show_progress=False)
    corpus = [random_text(rng, 40) for _ in range(400)]
    if extra_merges_text:
        corpus.append(extra_merges_text)
    tok.train_from_iterator(corpus, trainer)
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, bos_token="<s>", eos_token="</s>", unk_token="<unk>")
    os.makedirs(folder, exist_ok=True)
    fast.save_pretrained(folder)
    return fast


def make_model_dir(folder: str, cfg, tokenizer_src: str, seed: int = 0, dtype=torch.float32, batch_size: int = 2,
                   add_bos: bool = True, completion: bool = False, prompt_format: dict | None = None) -> str:
    """Random-init model in HF layout + tokenizer files + prompt_format.json / pipeline_config.json."""
    from ..ckpt.hf import save_hf_model
    from ..config import DEFAULT_PROMPT_FORMAT
    from ..models.llama import build_model
    model = build_model(cfg, dtype=dtype, device="cpu", seed=seed)
    save_hf_model(model, folder, tokenizer_src=tokenizer_src)
    with open(os.path.join(folder, "prompt_format.json"), "w", encoding="utf-8") as f:
        json.dump(prompt_format or DEFAULT_PROMPT_FORMAT, f)
    with open(os.path.join(folder, "pipeline_config.json"), "w", encoding="utf-8") as f:
        json.dump({"batch_size": batch_size, "add_bos": add_bos, "seq_chunk_len": 256, "completion": completion}, f)
    return folder


def make_dataset(path: str, n: int, seed: int = 0, completion_fraction: float = 0.25, max_turns: int = 3,
                 words=(5, 40)) -> list[dict]:
    rng = random.Random(seed)
    rows = []
    for i in range(n):
        if rng.random() < completion_fraction:
            rows.append({"init": "", "conversations": [{"from": "human", "value": random_text(rng, rng.randint(*words))}],
                         "source": "synthetic", "tags": ["completion"]})
            continue
        conv = []
        for t in range(rng.randint(1, max_turns)):
            conv.append({"from": "human", "value": random_text(rng, rng.randint(*words))})
            conv.append({"from": "gpt", "value": random_text(rng, rng.randint(*words))})
        rows.append({"init": random_text(rng, 6) if rng.random() < 0.5 else "", "conversations": conv,
                     "source": "synthetic", "tags": []})
    with open(path, "w", encoding="utf-8") as f:
        for r in rows:
            f.write(json.dumps(r, ensure_ascii=False) + "\n")
    return rows
