"""Training engine: micro-batch forward/backward through the fused loss head, gradient accumulation into the flat
fp32 gradient space, one fused optimizer launch per step, optional data-parallel / sharded gradient exchange.

``DistillEngine.train_step(host_batches)`` is the public per-step call: it takes micro-batches that live in pinned
host memory, copies them to the device asynchronously, runs forward + backward for each, then the (communicating)
optimizer step, and returns the summed loss as a device scalar (``.item()`` is the caller's device-to-host read).

Batch layout (``HostBatch`` / ``DeviceBatch``):
  input_ids [B, L] int64          padded token ids
  rows      [M] int64 or None     flattened (b*L + pos) positions of the content rows; None = every position
  ids       [M, K] int32          teacher top-K token ids, ascending per row
  logp      [M, K] fp16/fp32      teacher log-probs at T = 1 aligned with ids
  seg       [M] int64             conversation index of each row (0 .. n_seg-1)
  labels    [M] int64, avoid [M] bool   only for the reference loss
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..loss.head import distill_head_loss
from ..ops import basic
from .optim import FlatOptimizer, FlatParams
from .schedule import LRSchedule
from ..obs.trace import PhaseTimer


@dataclass
class HostBatch:
    input_ids: torch.Tensor
    ids: torch.Tensor
    logp: torch.Tensor
    seg: torch.Tensor
    n_seg: int
    rows: torch.Tensor | None = None
    labels: torch.Tensor | None = None
    avoid: torch.Tensor | None = None
    n_tokens: int = 0

    def pin(self) -> "HostBatch":
        for k in ("input_ids", "ids", "logp", "seg", "rows", "labels", "avoid"):
            t = getattr(self, k)
            if t is not None and not t.is_pinned() and torch.cuda.is_available():
                setattr(self, k, t.pin_memory())
        return self

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.input_ids, self.ids, self.logp, self.seg, self.rows,
                                                          self.labels, self.avoid) if t is not None)

    def to_device(self, device) -> "HostBatch":
        mv = lambda t: None if t is None else t.to(device, non_blocking=True)  # noqa: E731
        return HostBatch(mv(self.input_ids), mv(self.ids), mv(self.logp), mv(self.seg), self.n_seg, mv(self.rows),
                         mv(self.labels), mv(self.avoid), self.n_tokens)


class DistillEngine:
    def __init__(self, model, *, loss: str = "reference", temperature: float = 1.0, alpha: float = 2.0,
                 crop_to_size: int | None = None, optimizer: str = "adamw", lr: float = 1e-6, betas=(0.9, 0.99),
                 weight_decay: float = 2e-8, grad_accum: int = 1, schedule: LRSchedule | None = None, comm=None,
                 jsd_renorm: bool = False, vocab_parallel: bool = False, max_rows_per_rank: int = 0):
        self.model = model
        self.loss_kind = loss
        self.temperature = float(temperature)
        self.alpha = float(alpha)
        self.vocab = min(crop_to_size or model.cfg.vocab_size, model.cfg.vocab_size)
        self.grad_accum = int(grad_accum)
        self.schedule = schedule
        self.comm = comm
        self.jsd_renorm = jsd_renorm
        self.device = model.embed_tokens.device
        if comm is not None and getattr(comm, "full_shard", False):
            # weights, gradients and optimizer state all sharded: the communicator owns the layout (parallel/fsdp.py)
            self.flat = comm.build_flat(model)
        else:
            shard = (comm.rank, comm.world) if comm is not None and comm.shards_optimizer else (0, 1)
            buffers = comm.allocate_flat_buffers(model) if comm is not None else None
            self.flat = FlatParams([p for p in model.parameters() if p.requires_grad], shard=shard, buffers=buffers)
        self.opt = FlatOptimizer(self.flat, optimizer, lr=lr, betas=betas, weight_decay=weight_decay)
        if comm is not None:
            comm.attach(self.flat, self.opt)
        self.micro_in_step = 0
        self.vp_loss = None
        if vocab_parallel:
            import torch.distributed as dist
            if not (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
                raise ValueError("vocab_parallel_loss needs more than one rank")
            if getattr(comm, "full_shard", False):
                raise ValueError("vocab_parallel_loss runs with replicated or optimizer-sharded weights (ddp / fsdp), not zero3")
            from .vp_loss import VocabParallelLoss
            self.vp_loss = VocabParallelLoss(model, self.vocab, loss, self.temperature, max_rows_per_rank or 16384,
                                             jsd_renorm=jsd_renorm)
        self.timer = PhaseTimer(device=self.device)     # B200_TRACE=1 / B200_NVTX=1: device-timed phases, NVTX ranges

    # ---- forward of one micro-batch: (sum over conversations of per-conversation loss, logs)
    def loss_on_batch(self, mb: HostBatch):
        hs = self.model.hidden_states(mb.input_ids)
        Hc = hs if mb.rows is None else basic.GatherRowsFn.apply(hs, mb.rows)
        logp = mb.logp if mb.logp.dtype == torch.float32 else mb.logp.float()
        if self.vp_loss is not None:
            return self.vp_loss(Hc, self.model.lm_head, mb.ids, logp, mb.seg, mb.n_seg)
        return distill_head_loss(Hc, self.model.lm_head, mb.ids, logp, kind=self.loss_kind,
                                 temperature=self.temperature, vocab=self.vocab, alpha=self.alpha, labels=mb.labels,
                                 avoid=mb.avoid, seg=mb.seg, n_seg=mb.n_seg, jsd_renorm=self.jsd_renorm)

    def micro_step(self, mb: HostBatch, last: bool | None = None):
        """Forward + backward of one micro-batch. ``last``: the caller knows whether the optimizer step follows this
        micro-batch (None: not known; then it is taken to be the ``grad_accum``-th micro-batch of the step)."""
        with self.timer.phase("forward+loss"):
            loss, logs = self.loss_on_batch(mb)
        # last micro-batch of the step under a communicator that can do it: the gradient of each layer is reduced
        # (and its shard of the weights updated) as soon as that layer's backward is through, behind the backward
        # of the earlier layers
        is_last = (self.micro_in_step + 1 == self.grad_accum) if last is None else bool(last)
        overlap = self.comm is not None and getattr(self.comm, "supports_overlap", False) and is_last
        if last and self.comm is not None and hasattr(self.comm, "last_micro_batch"):
            self.comm.last_micro_batch(self.lr, 1.0 / self.grad_accum)
        if overlap:
            from ..models import llama as _llama
            self.comm.begin_overlap(self.lr, 1.0 / self.grad_accum)
            _llama.LAYER_BACKWARD_DONE[0] = self._layer_done
        try:
            with self.timer.phase("backward"):
                loss.backward()
                self.flat.absorb_autograd_grads()
        finally:
            if overlap:
                _llama.LAYER_BACKWARD_DONE[0] = None
        self.micro_in_step += 1
        return loss.detach(), logs

    def _layer_done(self, first_param) -> None:
        off = self.flat.offset_of(first_param)
        if off is not None:
            self.comm.range_ready(off)

    def idle_micro_step(self, last: bool | None = None) -> None:
        """This rank has no micro-batch where other ranks have one: under full sharding it still takes part in their
        collectives; otherwise nothing to do."""
        if self.comm is not None and hasattr(self.comm, "idle_micro_step"):
            if last and hasattr(self.comm, "last_micro_batch"):
                self.comm.last_micro_batch(self.lr, 1.0 / self.grad_accum)
            self.comm.idle_micro_step()

    def full_parameters(self, writeback: bool = False):
        """Context in which every parameter holds its whole current value (checkpoint save / load). All ranks enter
        together under full sharding; a no-op otherwise."""
        if self.comm is not None and hasattr(self.comm, "gathered"):
            return self.comm.gathered(writeback=writeback)
        import contextlib
        return contextlib.nullcontext()

    @property
    def lr(self) -> float:
        return self.schedule.lr if self.schedule is not None else self.opt.lr

    def optimizer_step(self, n_micro: int | None = None) -> None:
        """Applies the accumulated gradient. The reference divides each micro-batch loss by ``grad_accum`` before
        backward (classes/losses.py:77); here that factor rides in the optimizer kernel's gradient scale."""
        self.flat.untouched_to_zero()
        scale = 1.0 / self.grad_accum
        with self.timer.phase("reduce+optimizer"):
            if self.comm is not None:
                self.comm.reduce_and_step(self.lr, scale)
            else:
                self.opt.step(self.lr, grad_scale=scale)
        self.flat.mark_fresh()
        self.micro_in_step = 0
        if self.schedule is not None:
            self.schedule.step()

    def train_step(self, host_batches: list[HostBatch]) -> torch.Tensor:
        total = None
        for k, hb in enumerate(host_batches):
            mb = hb.to_device(self.device)
            loss, _ = self.micro_step(mb, last=(k + 1 == len(host_batches)))
            total = loss if total is None else total + loss
        self.optimizer_step()
        return total

    @torch.no_grad()
    def eval_batch(self, hb: HostBatch):
        mb = hb.to_device(self.device)
        return self.loss_on_batch(mb)


def synthetic_batch(vocab: int, B: int, L: int, K: int, seed: int, device="cpu", logit_std: float = 3.0,
                    reference_fields: bool = False) -> HostBatch:
    """Synthetic micro-batch of the benchmark shape: token ids uniform in [0, vocab); for every position K teacher
    ids drawn without replacement with log-probs from a softmax over N(0, logit_std) logits, stored fp16 at T = 1.
    Every position is a content row and each sequence is one conversation."""
    g = torch.Generator(device=device).manual_seed(seed)
    input_ids = torch.randint(0, vocab, (B, L), generator=g, device=device)
    M = B * L
    ids = torch.empty((M, K), dtype=torch.int32, device=device)
    step = 2048
    for r0 in range(0, M, step):  # K ids without replacement: top-K of iid uniforms, a row block at a time
        n = min(step, M - r0)
        ids[r0:r0 + n] = torch.rand((n, vocab), generator=g, device=device).topk(K, dim=-1).indices.to(torch.int32)
    ids = ids.sort(dim=-1).values
    logits = torch.randn((M, K), generator=g, device=device) * logit_std
    logp = torch.log_softmax(logits, dim=-1).to(torch.float16)
    seg = torch.arange(B, device=device).repeat_interleave(L)
    hb = HostBatch(input_ids.cpu(), ids.cpu(), logp.cpu(), seg.cpu(), B, None, None, None, n_tokens=M)
    if reference_fields:
        labels = torch.cat([input_ids[:, 1:], torch.full((B, 1), -1, device=device, dtype=input_ids.dtype)], 1).reshape(-1)
        hb.labels = labels.cpu()
        hb.avoid = torch.zeros(M, dtype=torch.bool)
    return hb
