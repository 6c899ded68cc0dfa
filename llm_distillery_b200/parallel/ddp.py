"""Data-parallel gradient exchange for the flat parameter space.

``NcclComm`` (the baseline path): NCCL all-reduce of the flat fp32 gradient, then every rank runs the same
optimizer step. ``P2PComm`` (``parallel/p2p.py``, the product path): gradients and weights live in symmetric
memory; one kernel per step reduce-scatters the gradient over NVLink with peer loads, applies AdamW to the local
shard and stores the updated bf16 weights into every peer's weight buffer.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class NcclComm:
    shards_optimizer = False

    def __init__(self, device):
        self.device = device
        self.rank = dist.get_rank()
        self.world = dist.get_world_size()
        self.flat = None
        self.opt = None

    def allocate_flat_buffers(self, model):
        return None

    def attach(self, flat, opt):
        self.flat, self.opt = flat, opt

    def reduce_and_step(self, lr: float, grad_scale: float) -> None:
        dist.all_reduce(self.flat.grad, op=dist.ReduceOp.SUM)
        self.opt.step(lr, grad_scale=grad_scale / self.world)


def make_comm(kind: str, device):
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return None
    if kind == "nccl":
        return NcclComm(device)
    from .p2p import P2PComm
    return P2PComm(device)
