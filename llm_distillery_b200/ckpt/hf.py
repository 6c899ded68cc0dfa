"""HuggingFace-layout checkpoints (config.json + safetensors [+ shard index] + tokenizer files) and trainer state.

Model folders written here load with ``transformers.AutoModelForCausalLM.from_pretrained`` and folders written by
HF load here: fused projections are split into q/k/v and gate/up tensors on save and concatenated on load.
Trainer state lives in ``<cache>/student/states`` with the reference's file names (model_state.pt,
optimizer_state.pt, scheduler_state.pt; classes/student/model.py:270-297) plus ``trainer_state.json`` (sample
counters, next validation/save/accumulation thresholds, data-order seed), so a run resumes across processes - the
reference only resumes inside one process.
"""
from __future__ import annotations

import json
import os
import shutil

import torch

from ..models.llama import LlamaConfig, LlamaModel

TOKENIZER_FILES = ("tokenizer.json", "tokenizer.model", "tokenizer_config.json", "special_tokens_map.json",
                   "added_tokens.json", "vocab.json", "merges.txt", "generation_config.json", "prompt_format.json",
                   "pipeline_config.json")


def is_model_safetensors(model_path: str) -> bool:
    return os.path.isdir(model_path) and any(f.endswith(".safetensors") for f in os.listdir(model_path))


def save_hf_model(model: LlamaModel, folder: str, tokenizer_src: str | None = None,
                  max_shard_bytes: int = 5 * 1024 ** 3, dtype: torch.dtype | None = None) -> None:
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    cfg = model.cfg.to_hf_dict()
    sd = {k: v.detach().to("cpu", dtype or v.dtype).contiguous() for k, v in model.to_hf_state_dict().items()}
    cfg["torch_dtype"] = str(next(iter(sd.values())).dtype).replace("torch.", "")
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=2)
    shards, cur, cur_bytes = [], {}, 0
    for k, v in sd.items():
        n = v.numel() * v.element_size()
        if cur and cur_bytes + n > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[k] = v
        cur_bytes += n
    shards.append(cur)
    if len(shards) == 1:
        save_file(shards[0], os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})
    else:
        index = {"metadata": {"total_size": sum(v.numel() * v.element_size() for v in sd.values())}, "weight_map": {}}
        for i, sh in enumerate(shards, 1):
            name = f"model-{i:05d}-of-{len(shards):05d}.safetensors"
            save_file(sh, os.path.join(folder, name), metadata={"format": "pt"})
            for k in sh:
                index["weight_map"][k] = name
        with open(os.path.join(folder, "model.safetensors.index.json"), "w", encoding="utf-8") as f:
            json.dump(index, f, indent=2)
    if tokenizer_src and os.path.isdir(tokenizer_src):
        for name in TOKENIZER_FILES:
            src = os.path.join(tokenizer_src, name)
            if os.path.exists(src):
                shutil.copy(src, os.path.join(folder, name))


def load_hf_state_dict(path: str) -> dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {path}")
    sd = {}
    for f in files:
        sd.update(load_file(os.path.join(path, f)))
    return sd


def load_hf_model(path: str, dtype: torch.dtype = torch.bfloat16, device="cpu") -> LlamaModel:
    cfg = LlamaConfig.from_pretrained(path)
    model = LlamaModel(cfg, dtype=dtype, device=device)
    model.load_hf_state_dict(load_hf_state_dict(path), strict=False)
    return model


# ------------------------------------------------------------------------------------------------- trainer state
def save_trainer_state(states_dir: str, model: LlamaModel, optimizer, schedule, counters: dict) -> None:
    os.makedirs(states_dir, exist_ok=True)
    torch.save({k: v.detach().cpu() for k, v in model.to_hf_state_dict().items()}, os.path.join(states_dir, "model_state.pt"))
    osd = optimizer.state_dict()
    osd = {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else
               ({kk: vv.detach().cpu() for kk, vv in v.items()} if isinstance(v, dict) else v)) for k, v in osd.items()}
    rank = osd["shard"][0]
    name = "optimizer_state.pt" if osd["shard"][1] == 1 else f"optimizer_state.rank{rank}.pt"
    torch.save(osd, os.path.join(states_dir, name))
    torch.save(schedule.state_dict() if schedule is not None else {}, os.path.join(states_dir, "scheduler_state.pt"))
    with open(os.path.join(states_dir, "trainer_state.json"), "w", encoding="utf-8") as f:
        json.dump(counters, f, indent=2)


def load_trainer_state(states_dir: str, model: LlamaModel, optimizer, schedule) -> dict:
    model.load_hf_state_dict(torch.load(os.path.join(states_dir, "model_state.pt"), map_location="cpu"), strict=False)
    shard = optimizer.state_dict()["shard"]
    name = "optimizer_state.pt" if shard[1] == 1 else f"optimizer_state.rank{shard[0]}.pt"
    p = os.path.join(states_dir, name)
    if os.path.exists(p):
        osd = torch.load(p, map_location=optimizer.flat.device)
        if tuple(osd["shard"]) == tuple(shard) and osd["total"] == optimizer.flat.total:
            optimizer.load_state_dict(osd)
        else:   # different world size: optimizer moments restart, weights (above) carry over
            optimizer.flat.master.copy_(optimizer.flat.model_shard().float())
    else:
        optimizer.flat.master.copy_(optimizer.flat.model_shard().float())
    sp = os.path.join(states_dir, "scheduler_state.pt")
    if schedule is not None and os.path.exists(sp):
        sd = torch.load(sp)
        if sd:
            schedule.load_state_dict(sd)
    cp = os.path.join(states_dir, "trainer_state.json")
    if os.path.exists(cp):
        with open(cp, "r", encoding="utf-8") as f:
            return json.load(f)
    return {}


def has_trainer_state(states_dir: str) -> bool:
    return os.path.exists(os.path.join(states_dir, "model_state.pt")) and \
        os.path.exists(os.path.join(states_dir, "trainer_state.json"))
