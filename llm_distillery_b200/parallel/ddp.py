"""Data-parallel gradient exchange for the flat parameter space.

``AllReduceComm`` is the library baseline (NCCL on GPUs, gloo on CPU ranks): all-reduce the flat fp32 gradient, every
rank runs the same full optimizer step (``ddp``) - or, with ``shard_strategy="fsdp"``, reduce-scatter the
gradient, update only the local 1/world shard of the fp32 master weights / optimizer state, and all-gather the
updated weights (ZeRO-style sharding of optimizer state; the model-dtype weights stay replicated).

``FullShardComm`` (``parallel/fsdp.py``, ``shard_strategy="zero3"``) also shards the weights and gradients: each unit
of the model is all-gathered just before it runs and its gradient reduce-scattered right after its backward.

``P2PComm`` (``parallel/p2p.py``) is the NVLink path: gradient and weight buffers live in symmetric memory and ONE
kernel per step reads every peer's gradient shard over NVLink, applies AdamW to the local shard and stores the new
weights into every peer's weight buffer.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class AllReduceComm:
    def __init__(self, device, shard_strategy: str = "ddp"):
        self.device = torch.device(device)
        self.rank = dist.get_rank()
        self.world = dist.get_world_size()
        self.shards_optimizer = shard_strategy == "fsdp"
        self.flat = None
        self.opt = None

    def allocate_flat_buffers(self, model):
        return None

    def attach(self, flat, opt) -> None:
        self.flat, self.opt = flat, opt

    def barrier(self) -> None:
        dist.barrier()

    def reduce_and_step(self, lr: float, grad_scale: float) -> None:
        f = self.flat
        if not self.shards_optimizer:
            dist.all_reduce(f.grad, op=dist.ReduceOp.SUM)
            self.opt.step(lr, grad_scale=grad_scale / self.world)
            return
        shard = torch.empty(f.shard_size, dtype=torch.float32, device=f.grad.device)
        if dist.get_backend() == "gloo":      # gloo has no reduce_scatter_tensor
            dist.all_reduce(f.grad, op=dist.ReduceOp.SUM)
            shard.copy_(f.grad_shard())
        else:
            dist.reduce_scatter_tensor(shard, f.grad, op=dist.ReduceOp.SUM)
        self.opt.step(lr, grad_scale=grad_scale / self.world, grad=shard)
        if dist.get_backend() == "gloo":
            parts = [torch.empty_like(f.model_shard()) for _ in range(self.world)]
            dist.all_gather(parts, f.model_shard().contiguous())
            f.model.copy_(torch.cat(parts))
        else:
            dist.all_gather_into_tensor(f.model, f.model_shard().clone())


NcclComm = AllReduceComm


def make_comm(kind: str, device, shard_strategy: str = "ddp"):
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return None
    if shard_strategy == "zero3":
        from .fsdp import FullShardComm, P2PFullShardComm
        if kind == "p2p" and torch.device(device).type == "cuda":
            return P2PFullShardComm(device)
        return FullShardComm(device)
    if kind in ("nccl", "gloo") or torch.device(device).type != "cuda":
        return AllReduceComm(device, shard_strategy)
    from .p2p import P2PComm
    return P2PComm(device, shard_strategy)
