"""Optimizers over ONE flat parameter space.

Trainable parameters are re-pointed into a single contiguous buffer in the model dtype; alongside it live an fp32
master copy, an fp32 gradient buffer (parameters' ``grad_slot`` views: wgrad GEMM epilogues accumulate straight
into it) and the optimizer state. A step is one kernel launch over the (local shard of the) flat space
(csrc/optim/optim.cu), which also makes the sharded / fused-with-reduce-scatter variants in ``parallel`` a matter
of handing the kernel a sub-range.

The reference's twelve optimizer names (utils/finetuning_utils.py:127-155, bitsandbytes classes) map to:
  adam                      Adam with L2 weight decay, fp32 state
  adamw, adamw32bit         AdamW, fp32 state
  adamw8bit                 AdamW, block-wise 8-bit state (256-value blocks, dynamic absmax per block)
  paged_adamw*              same as the unpaged variants: with 180 GB of HBM per GPU optimizer state is never paged
  sgd                       momentum SGD (momentum 0.01 as in the reference), optional Nesterov
  rmsprop, rmsprop8bit/32   centred RMSprop (alpha 0.9, eps 1e-10), fp32 state
  adagrad                   Adagrad, fp32 state
Hyper-parameters the reference fixes are the defaults here: betas (0.9, 0.99), weight_decay 2e-8, Adam eps 1e-8.
"""
from __future__ import annotations

import math

import torch

from ..models.llama import GradSlot
from ..ops import _lib

ALIGN = 64  # elements; keeps every parameter 128-byte aligned inside the flat buffers (TMA needs 16)

_ADAM = {"adam": (False, False), "adamw": (True, False), "adamw32bit": (True, False), "adamw8bit": (True, True),
         "paged_adamw": (True, False), "paged_adamw32bit": (True, False), "paged_adamw8bit": (True, True)}
_SIMPLE = {"sgd": 0, "rmsprop": 1, "rmsprop8bit": 1, "rmsprop32bit": 1, "adagrad": 2}


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class FlatParams:
    """Flattens the trainable parameters of a module. ``shard`` = (rank, world) makes the fp32 master / state
    cover only this rank's contiguous 1/world slice (padded so slices are equal and 256-aligned)."""

    def __init__(self, params: list[torch.nn.Parameter], shard: tuple[int, int] = (0, 1), buffers: dict | None = None):
        seen, uniq = set(), []
        for p in params:
            if p.requires_grad and id(p) not in seen:
                seen.add(id(p))
                uniq.append(p)
        if not uniq:
            raise ValueError("no trainable parameters")
        self.params = uniq
        self.dtype = uniq[0].dtype
        self.device = uniq[0].device
        self.offsets = []
        off = 0
        for p in uniq:
            self.offsets.append(off)
            off += _round_up(p.numel(), ALIGN)
        rank, world = shard
        self.rank, self.world = rank, world
        self.total = _round_up(off, 256 * world)
        self.shard_size = self.total // world
        self.shard_lo = rank * self.shard_size
        buffers = buffers or {}
        # model-dtype weights and fp32 gradients span the whole space on every rank
        self.model = buffers.get("model")
        if self.model is None:
            self.model = torch.zeros(self.total, dtype=self.dtype, device=self.device)
        self.grad = buffers.get("grad")
        if self.grad is None:
            self.grad = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        self.slots: list[GradSlot] = []
        with torch.no_grad():
            for p, o in zip(uniq, self.offsets):
                n = p.numel()
                self.model[o:o + n].copy_(p.data.reshape(-1))
                p.data = self.model[o:o + n].view(p.shape)
                slot = GradSlot(self.grad[o:o + n].view(p.shape))
                p.grad_slot = slot
                self.slots.append(slot)
        self.master = self.model[self.shard_lo:self.shard_lo + self.shard_size].float().clone()
        self._offset_by_id = {id(p): o for p, o in zip(uniq, self.offsets)}

    def offset_of(self, p) -> int | None:
        """Offset of a parameter in the flat space (None: not a trainable parameter of this engine)."""
        return self._offset_by_id.get(id(p))

    def zero_untouched_in(self, lo: int, hi: int) -> None:
        """``untouched_to_zero`` restricted to the parameters that start in [lo, hi)."""
        for s, o in zip(self.slots, self.offsets):
            if lo <= o < hi and s.fresh:
                s.buf.zero_()
                s.fresh = False

    def absorb_autograd_grads(self) -> None:
        """Fold gradients that autograd left in ``p.grad`` (ops without a fused wgrad epilogue, e.g. the PyTorch
        restatement of the loss head on CPU) into the flat fp32 gradient."""
        for p, s in zip(self.params, self.slots):
            if p.grad is not None:
                if s.fresh:
                    s.buf.copy_(p.grad)
                    s.fresh = False
                else:
                    s.buf.add_(p.grad)
                p.grad = None

    def mark_fresh(self) -> None:
        for s in self.slots:
            s.fresh = True

    def untouched_to_zero(self) -> None:
        """Parameters that received no gradient since the last step must read as zero gradient."""
        for s in self.slots:
            if s.fresh:
                s.buf.zero_()

    def grad_shard(self) -> torch.Tensor:
        return self.grad[self.shard_lo:self.shard_lo + self.shard_size]

    def model_shard(self) -> torch.Tensor:
        return self.model[self.shard_lo:self.shard_lo + self.shard_size]


class FlatOptimizer:
    def __init__(self, flat: FlatParams, name: str = "adamw", lr: float = 1e-6, betas=(0.9, 0.99), eps: float = 1e-8,
                 weight_decay: float = 2e-8, momentum: float = 0.01, nesterov: bool = False):
        name = name.lower()
        if name not in _ADAM and name not in _SIMPLE:
            raise ValueError(f"Invalid optimizer name: {name}\nAvailable optimizers: {sorted(list(_ADAM) + list(_SIMPLE))}")
        self.flat, self.name = flat, name
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.momentum, self.nesterov = momentum, nesterov
        self.step_count = 0
        n, dev = flat.shard_size, flat.device
        self.state: dict[str, torch.Tensor] = {}
        if name in _ADAM:
            self.decoupled, self.eightbit = _ADAM[name]
            if self.eightbit:
                nb = (n + 255) // 256
                self.state = {"mq": torch.zeros(n, dtype=torch.int8, device=dev),
                              "vq": torch.zeros(n, dtype=torch.uint8, device=dev),
                              "mabs": torch.zeros(nb, dtype=torch.float32, device=dev),
                              "vabs": torch.zeros(nb, dtype=torch.float32, device=dev)}
            else:
                self.state = {"m": torch.zeros(n, dtype=torch.float32, device=dev),
                              "v": torch.zeros(n, dtype=torch.float32, device=dev)}
        else:
            self.kind = _SIMPLE[name]
            self.state = {"s0": torch.zeros(n, dtype=torch.float32, device=dev)}
            if self.kind == 1:
                self.state["s1"] = torch.zeros(n, dtype=torch.float32, device=dev)
                self.eps = 1e-10
            if self.kind == 2:
                self.eps = 1e-10

    # ---- one update of the local shard; grad (fp32, shard-sized) defaults to the flat gradient shard
    def step(self, lr: float | None = None, grad_scale: float = 1.0, grad: torch.Tensor | None = None) -> None:
        f = self.flat
        lr = self.lr if lr is None else lr
        grad = f.grad_shard() if grad is None else grad
        model = f.model_shard()
        self.step_count += 1
        if f.device.type == "cuda":
            self._step_cuda(lr, grad_scale, grad, model)
        else:
            self._step_torch(lr, grad_scale, grad, model)

    def _step_cuda(self, lr, gs, grad, model):
        lib, f, st = _lib.kernels(), self.flat, self.state
        n = f.shard_size
        mptr = _lib.ptr(model) if model.dtype == torch.bfloat16 else None
        if self.name in _ADAM:
            b1, b2 = self.betas
            if self.eightbit:
                rc = lib.b200_adam8_step(_lib.ptr(f.master), mptr, _lib.ptr(grad), _lib.ptr(st["mq"]), _lib.ptr(st["vq"]),
                                         _lib.ptr(st["mabs"]), _lib.ptr(st["vabs"]), n, lr, b1, b2, self.eps,
                                         self.weight_decay, self.step_count, gs, int(self.decoupled), _lib.stream())
            else:
                rc = lib.b200_adam_step(_lib.ptr(f.master), mptr, _lib.ptr(grad), _lib.ptr(st["m"]), _lib.ptr(st["v"]), n,
                                        lr, b1, b2, self.eps, self.weight_decay, self.step_count, gs,
                                        int(self.decoupled), _lib.stream())
            _lib.check(rc, "adam step")
        else:
            rc = lib.b200_simple_opt_step(_lib.ptr(f.master), mptr, _lib.ptr(grad), _lib.ptr(st["s0"]),
                                          _lib.ptr(st.get("s1")), n, self.kind, lr, self.weight_decay, self.momentum, 0.9,
                                          self.eps, int(self.nesterov), int(self.step_count == 1), gs, _lib.stream())
            _lib.check(rc, "optimizer step")
        if mptr is None:
            model.copy_(f.master.to(model.dtype))

    @torch.no_grad()
    def _step_torch(self, lr, gs, grad, model):
        f, st = self.flat, self.state
        p = f.master
        g = grad.float() * gs
        if self.name in _ADAM:
            b1, b2 = self.betas
            if self.eightbit:   # CPU restatement keeps fp32 state under the 8-bit names' behaviour envelope
                st.setdefault("m", torch.zeros_like(p))
                st.setdefault("v", torch.zeros_like(p))
            if self.decoupled:
                p.mul_(1 - lr * self.weight_decay)
            else:
                g = g + self.weight_decay * p
            st["m"].mul_(b1).add_(g, alpha=1 - b1)
            st["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
            bc1 = 1 - b1 ** self.step_count
            bc2 = 1 - b2 ** self.step_count
            p.addcdiv_(st["m"], (st["v"] / bc2).sqrt() + self.eps, value=-lr / bc1)
        else:
            g = g + self.weight_decay * p
            if self.kind == 0:
                buf = g.clone() if self.step_count == 1 else st["s0"] * self.momentum + g
                st["s0"].copy_(buf)
                upd = g if self.momentum == 0 else (g + self.momentum * buf if self.nesterov else buf)
                p.add_(upd, alpha=-lr)
            elif self.kind == 1:
                st["s0"].mul_(0.9).addcmul_(g, g, value=0.1)
                st["s1"].mul_(0.9).add_(g, alpha=0.1)
                p.addcdiv_(g, (st["s0"] - st["s1"] ** 2).clamp_min(0).sqrt() + self.eps, value=-lr)
            else:
                st["s0"].addcmul_(g, g)
                p.addcdiv_(g, st["s0"].sqrt() + self.eps, value=-lr)
        model.copy_(p.to(model.dtype))

    def zero_grad(self) -> None:
        self.flat.mark_fresh()

    def state_dict(self) -> dict:
        return {"name": self.name, "step_count": self.step_count, "lr": self.lr, "master": self.flat.master,
                "state": dict(self.state), "shard": (self.flat.rank, self.flat.world), "total": self.flat.total,
                "layout": getattr(self.flat, "layout", "contiguous"),
                "units": self.flat.unit_table() if hasattr(self.flat, "unit_table") else None}

    def load_state_dict(self, sd: dict) -> None:
        if sd["name"] != self.name:
            raise ValueError(f"optimizer state is for {sd['name']}, not {self.name}")
        self.step_count = int(sd["step_count"])
        self.flat.master.copy_(sd["master"])
        for k, v in sd["state"].items():
            if k in self.state:
                self.state[k].copy_(v)
            else:
                self.state[k] = v.to(self.flat.device)
        self.flat.model_shard().copy_(self.flat.master.to(self.flat.dtype))


def set_optimizer(params, lr: float, betas=(0.9, 0.99), optimizer_name: str = "adamw", weight_decay: float = 2e-8,
                  momentum: float = 0.01, nesterov: bool = False, shard=(0, 1), buffers=None) -> FlatOptimizer:
    """Reference-shaped factory (utils/finetuning_utils.py:127)."""
    flat = FlatParams(list(params), shard=shard, buffers=buffers)
    return FlatOptimizer(flat, optimizer_name, lr=lr, betas=betas, weight_decay=weight_decay, momentum=momentum,
                         nesterov=nesterov)
