"""Per-GPU memory estimate of student training under each sharding strategy, for sizing a run to 180 GB of HBM.

The reference sizes its student by hand (``num_gpu0_layers``, ``max_memory``, ``reserve_vram``:
classes/student/model.py:154-201); here the three strategies have closed-form footprints:

  ddp    bf16 weights (2 B) and fp32 gradient (4 B) per parameter on every rank; fp32 master + two moments (12 B) on
         every rank with the NCCL communicator, split over the ranks with the peer-to-peer one
  fsdp   as ddp, master + moments always split over the ranks (ZeRO-1)
  zero3  everything split: (2 + 4 + 4 + 8) B per parameter / world, plus two decoder layers and the embedding / head
         units whole (bf16 weights + fp32 gradients: 6 B per parameter of those units)

Activations are what ``models.llama.DecoderLayerFn`` saves for backward: per token and layer 4 hidden + 2 q + 2 kv + 3 ffn
bf16 values (layer input, two normalised copies, qkv, attention output, mid residual, gate|up, activation) - only the
layer input under gradient checkpointing, plus one layer's worth while it is recomputed - and the loss head's working
set (hidden rows, the bf16 dlogits tile buffer, top-K targets).

``python -m llm_distillery_b200.parallel.memory --model llama-3-8b --world 8 --seq-len 4096 --micro-batch 2`` prints
the table; ``recommend`` picks the cheapest strategy that fits.
"""
from __future__ import annotations

import argparse
import json
from dataclasses import dataclass

GB = float(2 ** 30)
HBM_GB = 180.0           # B200
HEADROOM_GB = 12.0       # allocator slack, CUDA context, NCCL / symmetric-memory bookkeeping, rope tables


@dataclass
class Footprint:
    strategy: str
    weights_gb: float          # model-dtype weights resident on a rank
    gradients_gb: float        # fp32 gradient buffers
    optimizer_gb: float        # fp32 master + state
    buffers_gb: float          # gather / gradient buffers of full sharding
    activations_gb: float
    head_gb: float

    @property
    def total_gb(self) -> float:
        return (self.weights_gb + self.gradients_gb + self.optimizer_gb + self.buffers_gb + self.activations_gb
                + self.head_gb)

    def fits(self, hbm_gb: float = HBM_GB) -> bool:
        return self.total_gb + HEADROOM_GB <= hbm_gb

    def as_dict(self) -> dict:
        d = {k: round(getattr(self, k), 2) for k in ("weights_gb", "gradients_gb", "optimizer_gb", "buffers_gb",
                                                     "activations_gb", "head_gb")}
        return {"strategy": self.strategy, **d, "total_gb": round(self.total_gb, 2), "fits_180gb": self.fits()}


def _layer_params(cfg) -> int:
    h, f = cfg.hidden_size, cfg.intermediate_size
    n = h * (cfg.q_size + 2 * cfg.kv_size) + cfg.q_size * h + 3 * h * f + 2 * h
    if getattr(cfg, "attention_bias", False):
        n += cfg.q_size + 2 * cfg.kv_size
    return n


def state_bytes_per_param(optimizer: str) -> float:
    """fp32 master copy + optimizer state."""
    o = optimizer.lower()
    if "8bit" in o and "adam" in o:
        return 4 + 2 + 8 / 256.0
    if "adam" in o or o.startswith("rmsprop"):
        return 4 + 8
    return 4 + 4                      # sgd (momentum), adagrad


def activation_bytes(cfg, tokens: int, grad_checkpointing: bool = False) -> float:
    h, q, kv, f = cfg.hidden_size, cfg.q_size, cfg.kv_size, cfg.intermediate_size
    per_layer = (4 * h + 2 * q + 2 * kv + 3 * f) * 2 + 8 + 4 * cfg.num_attention_heads      # + rstd x2, lse
    if grad_checkpointing:
        return tokens * (cfg.num_hidden_layers * h * 2 + per_layer)
    # the backward of one layer additionally holds its gradient temporaries (dgu, dact, dqkv, datt, two dh)
    return tokens * (cfg.num_hidden_layers * per_layer + (3 * f + 2 * q + 2 * kv + 3 * h) * 2)


def head_bytes(cfg, rows: int, topk: int) -> float:
    """Loss-head working set: gathered hidden rows and their gradient, bf16 dlogits for the two backward GEMMs, per-row
    statistics and the teacher targets (ids int32 + log-probs fp32 + gathered logits fp32)."""
    V, h = cfg.vocab_size, cfg.hidden_size
    return rows * (2 * h * 2 + V * 2 + topk * 12 + 64)


def estimate(cfg, world: int, strategy: str, tokens: int, *, topk: int = 200, optimizer: str = "adamw",
             grad_checkpointing: bool = False, comm: str = "p2p", content_rows: int | None = None) -> Footprint:
    """``tokens``: micro-batch x sequence length on one rank; ``content_rows``: rows that reach the loss head (default: all)."""
    world = max(1, int(world))
    P = cfg.num_params()
    sb = state_bytes_per_param(optimizer)
    act = activation_bytes(cfg, tokens, grad_checkpointing) / GB
    head = head_bytes(cfg, tokens if content_rows is None else content_rows, topk) / GB
    if strategy == "zero3" and world > 1:
        lp = _layer_params(cfg)
        emb = cfg.vocab_size * cfg.hidden_size
        whole = 2 * lp + emb + (cfg.hidden_size if cfg.tie_word_embeddings else emb + cfg.hidden_size)
        return Footprint("zero3", 2 * P / world / GB, 4 * P / world / GB, sb * P / world / GB, 6 * whole / GB, act, head)
    sharded_state = world > 1 and (strategy in ("fsdp", "zero3") or comm == "p2p")
    return Footprint(strategy if world > 1 else "single", 2 * P / GB, 4 * P / GB,
                     sb * P / (world if sharded_state else 1) / GB, 0.0, act, head)


def recommend(cfg, world: int, tokens: int, **kw) -> tuple[str, dict[str, Footprint]]:
    """The first of ddp, zero3, zero3 + gradient checkpointing that fits 180 GB (ddp keeps whole weights next to the
    kernels and needs no gathers); "none" if even the last does not."""
    table = {"ddp": estimate(cfg, world, "ddp", tokens, **kw)}
    if world > 1:
        table["zero3"] = estimate(cfg, world, "zero3", tokens, **kw)
        table["zero3+checkpointing"] = estimate(cfg, world, "zero3", tokens, **{**kw, "grad_checkpointing": True})
    else:
        table["ddp+checkpointing"] = estimate(cfg, world, "ddp", tokens, **{**kw, "grad_checkpointing": True})
    for name, fp in table.items():
        if fp.fits():
            return name, table
    return "none", table


def teacher_footprint_gb(cfg, tp: int, tokens: int, topk: int = 200, vocab: int | None = None) -> float:
    """bf16 teacher collecting ``tokens`` positions per forward at tensor-parallel width ``tp``: the rank's slices of the
    layers and of the (cropped) LM head, the replicated embedding and norms, the token-major working set of one layer
    (gathered / staged activations are double-buffered), the fp32 logits of the rank's vocabulary slice and the top-K
    candidates."""
    tp = max(1, int(tp))
    h, f, q, kv = cfg.hidden_size, cfg.intermediate_size, cfg.q_size, cfg.kv_size
    V = min(vocab or cfg.vocab_size, cfg.vocab_size)
    layer = _layer_params(cfg) - 2 * h
    weights = 2 * (cfg.num_hidden_layers * (layer / tp + 2 * h) + cfg.vocab_size * h + V * h / tp + h)
    work = tokens * ((8 * h + 2 * (q + 2 * kv) / tp + 4 * f / tp) * 2 + (V / tp) * 4 + tp * topk * 12)
    return (weights + work) / GB


def recommend_tp(cfgs, world: int, tokens: int, topk: int = 200, vocab: int | None = None) -> int:
    """Smallest tensor-parallel width (a divisor of ``world`` that also divides every teacher's heads, KV heads and FFN
    width) at which every teacher fits 180 GB per GPU. Smaller is better when it fits: the ranks that are not needed
    for width become data-parallel replicas, which collect without any communication. Returns ``world``'s largest
    valid width if nothing fits."""
    valid = [t for t in range(1, max(1, world) + 1) if world % t == 0 and all(
        c.num_attention_heads % t == 0 and c.num_key_value_heads % t == 0 and c.intermediate_size % t == 0 for c in cfgs)]
    for t in valid:
        if all(teacher_footprint_gb(c, t, tokens, topk, vocab) + HEADROOM_GB <= HBM_GB for c in cfgs):
            return t
    return valid[-1] if valid else 1


def main(argv=None) -> int:
    from ..models.llama import LlamaConfig, preset
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--model", required=True, help="preset name or a HuggingFace model folder")
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--topk", type=int, default=200)
    ap.add_argument("--optimizer", default="adamw")
    a = ap.parse_args(argv)
    import os
    cfg = LlamaConfig.from_pretrained(a.model) if os.path.isdir(a.model) else preset(a.model)
    pick, table = recommend(cfg, a.world, a.seq_len * a.micro_batch, topk=a.topk, optimizer=a.optimizer)
    for name, fp in table.items():
        print(json.dumps({"plan": name, **fp.as_dict()}))
    print(json.dumps({"recommended": pick, "params_b": round(cfg.num_params() / 1e9, 3), "world": a.world,
                      "tokens_per_rank": a.seq_len * a.micro_batch}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
