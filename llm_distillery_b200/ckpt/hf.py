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
                  max_shard_bytes: int = 5 * 1024 ** 3, dtype: torch.dtype | None = None,
                  writer: tuple[int, int] = (0, 1)) -> None:
    """HuggingFace folder layout: ``config.json``, ``model.safetensors`` or numbered shards + index, tokenizer files.

    ``writer = (rank, world)``: several ranks that all hold the whole weights share the work - every rank cuts the
    same shard list, rank r writes shards r, r + world, ...; rank 0 also writes the config, the index and the
    tokenizer files. Only tensors this rank writes are copied to the host."""
    from safetensors.torch import save_file
    rank, world = writer
    os.makedirs(folder, exist_ok=True)
    cfg = model.cfg.to_hf_dict()
    named = list(model.to_hf_state_dict().items())
    out_dtype = dtype or named[0][1].dtype
    cfg["torch_dtype"] = str(out_dtype).replace("torch.", "")
    size = lambda v: v.numel() * torch.empty((), dtype=dtype or v.dtype).element_size()  # noqa: E731
    shards, cur, cur_bytes = [], [], 0
    for k, v in named:
        n = size(v)
        if cur and cur_bytes + n > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = [], 0
        cur.append(k)
        cur_bytes += n
    shards.append(cur)
    by_name = dict(named)
    to_host = lambda k: by_name[k].detach().to("cpu", dtype or by_name[k].dtype).contiguous()  # noqa: E731
    if len(shards) == 1:
        names = ["model.safetensors"]
    else:
        names = [f"model-{i:05d}-of-{len(shards):05d}.safetensors" for i in range(1, len(shards) + 1)]
    for i, (name, keys) in enumerate(zip(names, shards)):
        if i % world == rank:
            save_file({k: to_host(k) for k in keys}, os.path.join(folder, name), metadata={"format": "pt"})
    if rank != 0:
        return
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=2)
    if len(shards) > 1:
        index = {"metadata": {"total_size": sum(size(v) for _, v in named)}, "weight_map": {}}
        for name, keys in zip(names, shards):
            for k in keys:
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
    if any(k.endswith((".qweight", ".q_weight")) for k in sd):
        # a quantised export (GPTQ, AWQ): expanded to bf16 here, once (ckpt/gptq.py says why and which layouts are read)
        from . import gptq
        sd = gptq.dequantize_state_dict(sd, gptq.quantization_config(path) or {})
    return sd


def load_hf_model(path: str, dtype: torch.dtype = torch.bfloat16, device="cpu") -> LlamaModel:
    cfg = LlamaConfig.from_pretrained(path)
    model = LlamaModel(cfg, dtype=dtype, device=device)
    model.load_hf_state_dict(load_hf_state_dict(path), strict=False)
    return model


# ------------------------------------------------------------------------------------------------- trainer state
def save_trainer_state(states_dir: str, model: LlamaModel, optimizer, schedule, counters: dict) -> None:
    """``model`` None: this rank writes no ``model_state.pt`` (another rank does, or the weights cannot be had)."""
    os.makedirs(states_dir, exist_ok=True)
    if model is not None:
        torch.save({k: v.detach().cpu() for k, v in model.to_hf_state_dict().items()},
                   os.path.join(states_dir, "model_state.pt"))
    osd = optimizer.state_dict()
    osd = {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else
               ({kk: vv.detach().cpu() for kk, vv in v.items()} if isinstance(v, dict) else v)) for k, v in osd.items()}
    rank = osd["shard"][0]
    name = "optimizer_state.pt" if osd["shard"][1] == 1 else f"optimizer_state.rank{rank}.pt"
    torch.save(osd, os.path.join(states_dir, name))
    torch.save(schedule.state_dict() if schedule is not None else {}, os.path.join(states_dir, "scheduler_state.pt"))
    with open(os.path.join(states_dir, "trainer_state.json"), "w", encoding="utf-8") as f:
        json.dump(counters, f, indent=2)


def _saved_optimizer_shards(states_dir: str) -> list[dict] | None:
    """All optimizer shard files of the state folder in rank order (CPU tensors), or None if the set is incomplete."""
    single = os.path.join(states_dir, "optimizer_state.pt")
    if os.path.exists(single):
        return [torch.load(single, map_location="cpu")]
    first = os.path.join(states_dir, "optimizer_state.rank0.pt")
    if not os.path.exists(first):
        return None
    world = int(torch.load(first, map_location="cpu")["shard"][1])
    out = []
    for r in range(world):
        p = os.path.join(states_dir, f"optimizer_state.rank{r}.pt")
        if not os.path.exists(p):
            return None
        out.append(torch.load(p, map_location="cpu"))
    return out


def reshard_optimizer_state(shards: list[dict], optimizer) -> bool:
    """Load a state saved under another world size: the flat parameter space is the same up to tail padding, so the
    saved slices are concatenated in rank order and this rank's slice is cut out. Only element-wise fp32 state
    (master weights and moments as long as a slice) can be cut this way; block-quantised 8-bit state cannot - the
    function then returns False and the caller restarts the moments."""
    flat = optimizer.flat
    old_size = int(shards[0]["total"]) // len(shards)
    if shards[0]["name"] != optimizer.name:
        return False
    saved_layout, layout = shards[0].get("layout", "contiguous"), getattr(flat, "layout", "contiguous")
    if saved_layout != layout:
        return False        # per-unit pieces (full sharding) and slices of one flat space do not convert
    if layout == "per_unit":
        return _reshard_per_unit(shards, optimizer)
    keys = list(shards[0]["state"].keys())
    for sd in shards:
        if sd["master"].numel() != old_size or any(
                (not torch.is_tensor(sd["state"][k])) or sd["state"][k].numel() != old_size or
                sd["state"][k].dtype != torch.float32 for k in keys):
            return False
    if any(k not in optimizer.state or optimizer.state[k].numel() != flat.shard_size for k in keys):
        return False

    def cut(parts: list[torch.Tensor]) -> torch.Tensor:
        full = torch.cat([t.reshape(-1).float() for t in parts])
        if full.numel() < flat.total:       # the new layout pads further: zeros there (no parameter lives in padding)
            full = torch.cat([full, torch.zeros(flat.total - full.numel())])
        return full[flat.shard_lo: flat.shard_lo + flat.shard_size]

    flat.master.copy_(cut([sd["master"] for sd in shards]))
    for k in keys:
        optimizer.state[k].copy_(cut([sd["state"][k] for sd in shards]))
    optimizer.step_count = int(shards[0]["step_count"])
    flat.model_shard().copy_(flat.master.to(flat.dtype))
    return True


def _reshard_per_unit(shards: list[dict], optimizer) -> bool:
    """Full sharding: every rank holds piece r of every unit. A unit's saved pieces, in rank order, are the unit up to
    its (world-dependent) tail padding; the new rank's piece is cut out of that, unit by unit."""
    flat = optimizer.flat
    old_units, new_units = shards[0].get("units"), flat.unit_table()
    if not old_units or len(old_units) != len(new_units):
        return False
    if any(o[0] != n[0] or int(o[1]) != int(n[1]) for o, n in zip(old_units, new_units)):
        return False        # other units or other sizes: not the same model / freeze pattern
    keys = list(shards[0]["state"].keys())
    old_size = sum(int(u[2]) for u in old_units)
    for sd in shards:
        if sd["master"].numel() != old_size or any(
                (not torch.is_tensor(sd["state"][k])) or sd["state"][k].numel() != old_size or
                sd["state"][k].dtype != torch.float32 for k in keys):
            return False
    if any(k not in optimizer.state or optimizer.state[k].numel() != flat.shard_size for k in keys):
        return False

    def cut(parts: list[torch.Tensor]) -> torch.Tensor:
        out, old_lo = [], 0
        for (_, payload, old_piece), (_, _, new_piece) in zip(old_units, new_units):
            full = torch.cat([t.reshape(-1)[old_lo:old_lo + old_piece].float().cpu() for t in parts])[:payload]
            need = new_piece * flat.world
            if full.numel() < need:
                full = torch.cat([full, torch.zeros(need - full.numel())])
            out.append(full[flat.rank * new_piece:(flat.rank + 1) * new_piece])
            old_lo += old_piece
        return torch.cat(out)

    flat.master.copy_(cut([sd["master"] for sd in shards]))
    for k in keys:
        optimizer.state[k].copy_(cut([sd["state"][k] for sd in shards]))
    optimizer.step_count = int(shards[0]["step_count"])
    flat.model_shard().copy_(flat.master.to(flat.dtype))
    return True


def load_model_state(states_dir: str, model: LlamaModel) -> None:
    model.load_hf_state_dict(torch.load(os.path.join(states_dir, "model_state.pt"), map_location="cpu"), strict=False)


def load_trainer_state(states_dir: str, model: LlamaModel | None, optimizer, schedule) -> dict:
    """``model`` None: the weights have been loaded already (``load_model_state``)."""
    if model is not None:
        load_model_state(states_dir, model)
    shard = optimizer.state_dict()["shard"]
    name = "optimizer_state.pt" if shard[1] == 1 else f"optimizer_state.rank{shard[0]}.pt"
    p = os.path.join(states_dir, name)
    done = False
    if os.path.exists(p):
        osd = torch.load(p, map_location=optimizer.flat.device)
        if (tuple(osd["shard"]) == tuple(shard) and osd["total"] == optimizer.flat.total
                and osd.get("layout", "contiguous") == getattr(optimizer.flat, "layout", "contiguous")):
            optimizer.load_state_dict(osd)
            done = True
    if not done:    # saved under another world size: cut this rank's slice out of the saved ones
        shards = _saved_optimizer_shards(states_dir)
        done = bool(shards) and reshard_optimizer_state(shards, optimizer)
    if not done:    # nothing usable: optimizer moments restart, weights (above) carry over
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


# ------------------------------------------------------------------------------------------------- tensor-parallel load
def load_tp_weights(path: str, rank: int, tp: int, vocab: int | None = None, dtype: torch.dtype = torch.bfloat16,
                    device="cpu") -> tuple[LlamaConfig, dict]:
    """Read ONE tensor-parallel rank's slices straight out of a HF safetensors checkpoint (no rank ever holds the
    whole model): q/k/v and gate/up rows, o_proj / down_proj columns, an equal slice of the (cropped) LM head,
    replicated embedding and norms. Returns (config, weights) in the layout of ``parallel.tp.shard_llama_weights``."""
    from safetensors import safe_open
    from . import gptq
    if (gptq.quantization_config(path) or {}).get("quant_method") in ("gptq", "awq", "exl2"):
        raise ValueError(f"{path} is a quantised checkpoint: the tensor-parallel loader reads slices of plain 16-bit "
                         "tensors. Collect with tp_size = 1 (the dequantised model fits one GPU) or export the "
                         "checkpoint to bf16 first.")
    cfg = LlamaConfig.from_pretrained(path)
    if cfg.model_type == "granite":
        raise NotImplementedError("tensor-parallel collection does not apply Granite's multipliers: use tp_size = 1")
    if cfg.o_bias or cfg.mlp_bias:
        raise NotImplementedError("tensor-parallel collection does not carry o_proj / MLP biases: use tp_size = 1")
    if cfg.sandwich or cfg.rope_interleaved:
        raise NotImplementedError(f"tensor-parallel collection is built for Llama-style pre-norm layers; a "
                                  f"{cfg.model_type} teacher runs with tp_size = 1 (ranks become data-parallel replicas)")
    if cfg.num_local_experts:
        raise NotImplementedError("tensor-parallel collection is built for dense decoders; a mixture-of-experts teacher "
                                  "runs with tp_size = 1 (ranks become data-parallel replicas)")
    H, Hkv, d, f = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.intermediate_size
    if H % tp or Hkv % tp or f % tp:
        raise ValueError(f"tp={tp} must divide heads ({H}), kv heads ({Hkv}) and the FFN width ({f})")
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx, encoding="utf-8") as fh:
            where = json.load(fh)["weight_map"]
    else:
        files = sorted(x for x in os.listdir(path) if x.endswith(".safetensors"))
        where = {}
        for fn in files:
            with safe_open(os.path.join(path, fn), "pt") as sf:
                for k in sf.keys():
                    where[k] = fn
    handles: dict = {}
    # a multimodal wrapper keeps its language model under a prefix: the plain names point at the prefixed tensors
    stored = {k: k for k in where}
    wrapped = [k for k in where if "language_model" in k and k.endswith("embed_tokens.weight")]
    if wrapped:
        prefix = wrapped[0][: -len("embed_tokens.weight")]
        stored.update({"model." + k[len(prefix):]: k for k in where if k.startswith(prefix)})
        stored.update({"lm_head.weight": k for k in where if k.endswith("lm_head.weight")})

    def sl(name: str, rows=None, cols=None) -> torch.Tensor:
        if name not in stored:
            raise KeyError(f"tensor {name} is not in the checkpoint at {path}")
        name = stored[name]
        fn = where[name]
        if fn not in handles:
            handles[fn] = safe_open(os.path.join(path, fn), "pt")
        s = handles[fn].get_slice(name)
        if rows is not None:
            t = s[rows[0]:rows[1]]
        elif cols is not None:
            t = s[:, cols[0]:cols[1]]
        else:
            t = s[:]
        return t.to(device=device, dtype=dtype)

    Hl, Hkvl, fl = H // tp, Hkv // tp, f // tp
    w = {"embed_tokens": sl("model.embed_tokens.weight"), "norm": sl("model.norm.weight")}
    for i in range(cfg.num_hidden_layers):
        hp, p = f"model.layers.{i}.", f"layers.{i}."
        if cfg.model_type == "phi3":        # fused tensors in the checkpoint: this rank's q / k / v and gate / up rows
            qn, kn = H * d, Hkv * d
            fused = hp + "self_attn.qkv_proj.weight"
            w[p + "qkv_proj"] = torch.cat([sl(fused, rows=(rank * Hl * d, (rank + 1) * Hl * d)),
                                           sl(fused, rows=(qn + rank * Hkvl * d, qn + (rank + 1) * Hkvl * d)),
                                           sl(fused, rows=(qn + kn + rank * Hkvl * d, qn + kn + (rank + 1) * Hkvl * d))], 0)
            w[p + "o_proj"] = sl(hp + "self_attn.o_proj.weight", cols=(rank * Hl * d, (rank + 1) * Hl * d)).contiguous()
            gu = hp + "mlp.gate_up_proj.weight"
            w[p + "gate_up_proj"] = torch.cat([sl(gu, rows=(rank * fl, (rank + 1) * fl)),
                                               sl(gu, rows=(f + rank * fl, f + (rank + 1) * fl))], 0)
            w[p + "down_proj"] = sl(hp + "mlp.down_proj.weight", cols=(rank * fl, (rank + 1) * fl)).contiguous()
            w[p + "input_layernorm"] = sl(hp + "input_layernorm.weight")
            w[p + "post_attention_layernorm"] = sl(hp + "post_attention_layernorm.weight")
            continue
        w[p + "qkv_proj"] = torch.cat([sl(hp + "self_attn.q_proj.weight", rows=(rank * Hl * d, (rank + 1) * Hl * d)),
                                       sl(hp + "self_attn.k_proj.weight", rows=(rank * Hkvl * d, (rank + 1) * Hkvl * d)),
                                       sl(hp + "self_attn.v_proj.weight", rows=(rank * Hkvl * d, (rank + 1) * Hkvl * d))], 0)
        if cfg.attention_bias:
            w[p + "qkv_bias"] = torch.cat([sl(hp + "self_attn.q_proj.bias", rows=(rank * Hl * d, (rank + 1) * Hl * d)),
                                           sl(hp + "self_attn.k_proj.bias", rows=(rank * Hkvl * d, (rank + 1) * Hkvl * d)),
                                           sl(hp + "self_attn.v_proj.bias", rows=(rank * Hkvl * d, (rank + 1) * Hkvl * d))])
        if cfg.qk_norm:          # one weight vector for all heads: replicated
            w[p + "q_norm"] = sl(hp + "self_attn.q_norm.weight")
            w[p + "k_norm"] = sl(hp + "self_attn.k_norm.weight")
        w[p + "o_proj"] = sl(hp + "self_attn.o_proj.weight", cols=(rank * Hl * d, (rank + 1) * Hl * d)).contiguous()
        w[p + "gate_up_proj"] = torch.cat([sl(hp + "mlp.gate_proj.weight", rows=(rank * fl, (rank + 1) * fl)),
                                           sl(hp + "mlp.up_proj.weight", rows=(rank * fl, (rank + 1) * fl))], 0)
        w[p + "down_proj"] = sl(hp + "mlp.down_proj.weight", cols=(rank * fl, (rank + 1) * fl)).contiguous()
        w[p + "input_layernorm"] = sl(hp + "input_layernorm.weight")
        w[p + "post_attention_layernorm"] = sl(hp + "post_attention_layernorm.weight")
    head_name = "lm_head.weight" if "lm_head.weight" in stored else "model.embed_tokens.weight"
    V = min(vocab or cfg.vocab_size, cfg.vocab_size)
    Vl = -(-(-(-V // tp)) // 8) * 8
    lo, hi = min(rank * Vl, V), min((rank + 1) * Vl, V)
    piece = torch.zeros((Vl, cfg.hidden_size), dtype=dtype, device=device)
    if hi > lo:
        piece[: hi - lo] = sl(head_name, rows=(lo, hi))
    w["lm_head"] = piece
    w["_vocab"] = (V, Vl, lo, hi - lo)
    return cfg, w
