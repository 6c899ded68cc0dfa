"""PyTorch ``.bin`` checkpoints -> fp16 safetensors in a sibling ``<folder>_safetensors`` directory (reference:
utils/convert_to_safetensor.py). Tied / aliased tensors are written once, the reloaded file is compared
bit-for-bit with what was written, the shard index is rewritten, auxiliary files are copied.

Unlike the reference the source folder is kept unless ``delete_source=True`` (the reference deletes it, :99-102).
"""
from __future__ import annotations

import json
import os
import shutil
from collections import defaultdict

import torch


def shared_pointers(tensors: dict) -> list[list[str]]:
    groups = defaultdict(list)
    for k, v in tensors.items():
        groups[v.data_ptr()].append(k)
    return [names for names in groups.values() if len(names) > 1]


def check_file_size(sf_filename: str, pt_filename: str) -> None:
    sf, pt = os.stat(sf_filename).st_size, os.stat(pt_filename).st_size
    # the copy is fp16: allow up to 2x shrink, reject growth of more than 1 %
    if (sf - pt) / pt > 0.01:
        raise RuntimeError(f"The file size difference is more than 1%:\n - {sf_filename}: {sf}\n - {pt_filename}: {pt}")


def convert_file(pt_filename: str, sf_filename: str) -> None:
    from safetensors.torch import load_file, save_file
    loaded = torch.load(pt_filename, map_location="cpu", weights_only=True)
    if "state_dict" in loaded:
        loaded = loaded["state_dict"]
    for group in shared_pointers(loaded):
        for name in group[1:]:
            loaded.pop(name)
    loaded = {k: v.contiguous().half() for k, v in loaded.items()}
    os.makedirs(os.path.dirname(sf_filename), exist_ok=True)
    save_file(loaded, sf_filename, metadata={"format": "pt"})
    check_file_size(sf_filename, pt_filename)
    reloaded = load_file(sf_filename)
    for k, v in loaded.items():
        if not torch.equal(v, reloaded[k]):
            raise RuntimeError(f"The output tensors do not match for key {k}")


def rename(pt_filename: str) -> str:
    name = pt_filename.replace(".bin", ".safetensors").replace("pytorch_model", "model")
    return name


def convert_multi(folder: str, out: str) -> None:
    with open(os.path.join(folder, "pytorch_model.bin.index.json"), "r", encoding="utf-8") as f:
        index = json.load(f)
    for fn in sorted(set(index["weight_map"].values())):
        convert_file(os.path.join(folder, fn), os.path.join(out, rename(fn)))
    index["weight_map"] = {k: rename(v) for k, v in index["weight_map"].items()}
    with open(os.path.join(out, "model.safetensors.index.json"), "w", encoding="utf-8") as f:
        json.dump(index, f, indent=4)


def convert_model(folder: str, delete_source: bool = False) -> str:
    out = f"{folder.rstrip('/')}_safetensors"
    os.makedirs(out, exist_ok=True)
    files = os.listdir(folder)
    if "pytorch_model.bin.index.json" in files:
        convert_multi(folder, out)
    elif "pytorch_model.bin" in files:
        convert_file(os.path.join(folder, "pytorch_model.bin"), os.path.join(out, "model.safetensors"))
    else:
        raise FileNotFoundError(f"no pytorch_model.bin or shard index in {folder}")
    for fn in files:
        if fn.endswith(".bin") or fn == "pytorch_model.bin.index.json":
            continue
        src = os.path.join(folder, fn)
        if os.path.isfile(src):
            shutil.copy(src, os.path.join(out, fn))
    if delete_source:
        shutil.rmtree(folder)
    return out


if __name__ == "__main__":
    import sys
    print(convert_model(sys.argv[1]))
