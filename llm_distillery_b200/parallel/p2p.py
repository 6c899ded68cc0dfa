"""NVLink peer-to-peer communicator for the flat parameter space (kernels: csrc/comm/p2p.cu).

The flat fp32 gradient and the flat bf16 weights are allocated in symmetric memory, so every rank holds device
pointers to every other rank's copies. One optimizer step is then

    barrier (all backward passes done)  ->  rs_adamw_ag kernel  ->  barrier (all weight stores landed)

where the middle kernel, for this rank's 1/world shard, sums all ranks' gradients with peer loads, applies AdamW to
the local fp32 master weights / moments and writes the new bf16 weights into every rank's weight buffer with peer
stores. The peers' gradients cross NVLink as bf16 (each rank casts its fp32 gradient into a symmetric "wire" buffer
first; the owner of a shard adds its own fp32 gradient and the peers' bf16 copies in fp32), which halves the bytes;
``B200_WIRE=fp32`` keeps the fp32 exchange.

With ``B200_OVERLAP=1`` the same kernel runs per finished layer range on a side
stream behind the backward of the earlier layers, on a handful of CTAs (``B200_OVERLAP_CTAS``): the exchange needs a
few tens of GB/s to keep up with backward, so it does not need the SMs the backward GEMMs are using, and only the
last range (embedding and first layer) is left for after backward. Optimizer state is therefore sharded (ZeRO-1) for ``ddp`` and ``fsdp`` alike. Optimizers other than the
fp32-state Adam family run reduce-scatter kernel -> local optimizer kernel -> all-gather kernel.

Barriers are flag exchanges with growing epoch numbers; every device-side wait is bounded and reports through the
error word (``ops._lib.take_device_error``). ``check()`` turns a reported time-out into a Python exception.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p

import torch
import torch.distributed as dist

from ..engine.optim import ALIGN, _round_up
from ..ops import _lib
from ..ops._lib import _VP, _I, _LL, _F

_U = ctypes.c_uint
_lib.register("b200_p2p_barrier", [_VP, _I, _I, _U, _VP])
_lib.register("b200_p2p_rs_adamw_ag", [_VP, _VP, _I, _VP, _VP, _VP, _VP, _LL, _LL, _LL, _I, _I, _F, _F, _F, _F, _F, _I, _F,
                                        _I, _I, _VP])
_lib.register("b200_p2p_cast_wire", [_VP, _VP, _LL, _LL, _VP])
_lib.register("b200_p2p_clear_poison", [_VP])
_lib.register("b200_p2p_mark_step", [_VP, _VP])
_lib.register("b200_p2p_reduce_scatter_f32", [_VP, _VP, _LL, _LL, _I, _I, _F, _I, _VP])
_lib.register("b200_p2p_allgather", [_VP, _VP, _LL, _LL, _I, _I, _I, _VP])


def _ptr_array(ptrs) -> ctypes.Array:
    return (c_void_p * len(ptrs))(*[c_void_p(int(p)) for p in ptrs])


class SymmetricBuffer:
    """A tensor allocated in symmetric memory plus the device pointers of every rank's copy."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.c_ptrs = _ptr_array(self.ptrs)


class P2PComm:
    shards_optimizer = True

    def __init__(self, device, shard_strategy: str = "ddp"):
        self.device = torch.device(device)
        self.rank = dist.get_rank()
        self.world = dist.get_world_size()
        self.shard_strategy = shard_strategy
        self.flat = None
        self.opt = None
        self.epoch = 0
        self.sig = SymmetricBuffer(64, torch.int32, self.device)
        # gradient reduction behind backward: its own stream, flag words and epoch counter (barriers of the two
        # streams must not share flags: a flag holds the latest epoch, and the streams run in no fixed order)
        self.sig_side = SymmetricBuffer(64, torch.int32, self.device)
        self.side_epoch = 0
        self.side = torch.cuda.Stream(device=self.device)
        self._ov = None
        import os
        # B200_OVERLAP=1: the SUM of finished layer ranges over the ranks runs beside backward on a few CTAs, into a
        # local fp32 buffer of the shard's size; the kernel after backward then only updates and all-gathers. (An
        # earlier form ran the whole fused kernel there: the AdamW pass moves 30 bytes per parameter through HBM,
        # which a small grid cannot do in time - 149.5 ms per step against 122.6 on two GPUs.) Default: one fused
        # kernel after backward.
        self._overlap_enabled = os.environ.get("B200_OVERLAP", "0") == "1"
        self._buckets = max(1, int(os.environ.get("B200_OVERLAP_BUCKETS", "8")))   # ranges per step handed over early
        self._overlap_ctas = max(1, int(os.environ.get("B200_OVERLAP_CTAS", "32")))
        # the overlapped reduction reads the peers' fp32 gradients directly: its traffic is hidden, a cast pass is not
        self._wire16 = os.environ.get("B200_WIRE", "bf16") != "fp32" and not self._overlap_enabled
        self._reduced = None           # fp32 sum over the ranks of this rank's shard (overlapped reduction only)
        self.grad_buf = None
        self.model_buf = None
        self.wire_buf = None
        self._rdv = torch.zeros(1, dtype=torch.float32, device=self.device)
        # optimizer steps issued by the host / steps whose reduction kernels really ran (a kernel behind a barrier
        # that gave up does nothing): the difference is what an emergency save must not claim
        # set by a benchmark: two events per step bracket the exchange proper (from the moment every rank has arrived
        # to the closing barrier), so that it can be told apart from the wait for the slowest rank before it
        self.time_exchange = False
        self._xev = None
        self.steps_issued = 0
        self._steps_applied = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.failed_step = False
        torch.cuda.synchronize(self.device)
        dist.barrier()

    # ---- buffers for FlatParams (same layout rule as engine.optim.FlatParams)
    def allocate_flat_buffers(self, model) -> dict:
        seen, total = set(), 0
        dtype = None
        for p in model.parameters():
            if p.requires_grad and id(p) not in seen:
                seen.add(id(p))
                total += _round_up(p.numel(), ALIGN)
                dtype = dtype or p.dtype
        total = _round_up(total, 256 * self.world)
        self.grad_buf = SymmetricBuffer(total, torch.float32, self.device)
        self.model_buf = SymmetricBuffer(total, dtype, self.device)
        if self._wire16 and dtype == torch.bfloat16:
            self.wire_buf = SymmetricBuffer(total, torch.bfloat16, self.device)
        return {"grad": self.grad_buf.tensor, "model": self.model_buf.tensor}

    def attach(self, flat, opt) -> None:
        self.flat, self.opt = flat, opt
        if flat.grad.data_ptr() != self.grad_buf.tensor.data_ptr() or flat.model.data_ptr() != self.model_buf.tensor.data_ptr():
            raise RuntimeError("flat buffers are not the symmetric allocations")
        self.barrier()

    # ---- primitives
    def rendezvous(self) -> None:
        """A tiny NCCL all-reduce on the current stream: what is enqueued after it starts only once every rank's
        stream has got here. The flag barriers of this module wait for at most two seconds and then report a lost peer;
        ranks can be further apart than that for harmless reasons (rank 0 writing a checkpoint, one rank's batch coming
        late from disk), so the first flag barrier of a step is preceded by this - NCCL's own wait has no such bound -
        and the bounded waits only ever see the skew of a few kernels."""
        dist.all_reduce(self._rdv)

    def barrier(self) -> None:
        self.epoch += 1
        _lib.check(_lib.kernels().b200_p2p_barrier(self.sig.c_ptrs, self.rank, self.world, self.epoch, _lib.stream()),
                   "b200_p2p_barrier")

    def check(self, sync: bool = False) -> None:
        """Raises when a bounded device-side wait has run out. Without ``sync`` the error word is read where it lives,
        in pinned host memory, with no device synchronisation: a wait that ran out in the step just queued may then
        only be seen at the next call. That is safe, because the kernels behind a failed barrier change nothing (see
        csrc/comm/p2p.cu); callers that are about to SAVE state pass ``sync=True``."""
        err = _lib.take_device_error() if sync else _lib.peek_device_error()
        if err:
            torch.cuda.synchronize(self.device)
            _lib.take_device_error()
            _lib.check(_lib.kernels().b200_p2p_clear_poison(_lib.stream()), "b200_p2p_clear_poison")
            torch.cuda.synchronize(self.device)
            self.failed_step = True
            raise RuntimeError(f"peer-to-peer wait timed out on rank {self.rank} (device error code {err})")

    def _mark_step(self) -> None:
        self.steps_issued += 1
        _lib.check(_lib.kernels().b200_p2p_mark_step(_lib.ptr(self._steps_applied), _lib.stream()), "b200_p2p_mark_step")

    def unapplied_steps(self) -> int:
        """Optimizer steps the host issued whose kernels did NOT run because a peer was lost (synchronises)."""
        torch.cuda.synchronize(self.device)
        return self.steps_issued - int(self._steps_applied.item())

    def _grad_sources(self):
        """(pointer table of the gradients the peers are read from, this rank's fp32 gradient, wire flag)."""
        if self.wire_buf is not None:
            return self.wire_buf.c_ptrs, _lib.ptr(self.flat.grad), 1
        return self.grad_buf.c_ptrs, None, 0

    def _cast_wire(self, lo: int, hi: int) -> None:
        """bf16 copy of this rank's gradient on [lo, hi) for the peers; its own shard is skipped (nobody reads it)."""
        if self.wire_buf is None:
            return
        f = self.flat
        for a, b in ((lo, min(hi, f.shard_lo)), (max(lo, f.shard_lo + f.shard_size), hi)):
            if b > a:
                _lib.check(_lib.kernels().b200_p2p_cast_wire(_lib.ptr(f.grad), _lib.ptr(self.wire_buf.tensor), a, b - a,
                                                             _lib.stream()), "b200_p2p_cast_wire")

    def reduce_scatter(self, src: SymmetricBuffer, out: torch.Tensor, lo: int, scale: float = 1.0,
                       max_ctas: int = 0) -> None:
        """out[i] = scale * sum over ranks of src[lo + i]; callers bracket this with barriers."""
        _lib.check(_lib.kernels().b200_p2p_reduce_scatter_f32(src.c_ptrs, _lib.ptr(out), lo, out.numel(), self.rank,
                                                              self.world, float(scale), int(max_ctas), _lib.stream()),
                   "p2p reduce_scatter")

    def allgather(self, dst: SymmetricBuffer, local: torch.Tensor, lo_elems: int, skip_self: bool = False) -> None:
        es = local.element_size()
        _lib.check(_lib.kernels().b200_p2p_allgather(dst.c_ptrs, _lib.ptr(local), lo_elems * es, local.numel() * es,
                                                     self.rank, self.world, int(skip_self), _lib.stream()), "p2p allgather")

    def allreduce_(self, buf: SymmetricBuffer, scale: float = 1.0) -> torch.Tensor:
        """In-place sum of a symmetric fp32 buffer over all ranks (reduce-scatter + all-gather by peer access)."""
        n = buf.tensor.numel()
        per = _round_up(-(-n // self.world), 4)
        lo = min(self.rank * per, n)
        cnt = max(0, min(per, n - lo))
        self.barrier()
        tmp = torch.empty(max(cnt, 4), dtype=torch.float32, device=self.device)
        if cnt:
            self.reduce_scatter(buf, tmp[:cnt], lo, scale)
        self.barrier()          # everyone has finished reading before anyone overwrites
        if cnt:
            self.allgather(buf, tmp[:cnt], lo)
        self.barrier()
        return buf.tensor

    # ---- gradient reduction overlapped with backward (fp32-state Adam family only)
    def _fused(self) -> bool:
        return (self.opt.name in ("adam", "adamw", "adamw32bit", "paged_adamw", "paged_adamw32bit")
                and self.flat.dtype == torch.bfloat16)

    @property
    def supports_overlap(self) -> bool:
        return self._overlap_enabled and self.world > 1 and self.flat is not None and self._fused()

    def begin_overlap(self, lr: float, grad_scale: float) -> None:
        """Before the last backward of a step: from now on ``range_ready(lo)`` may hand over finished gradients."""
        if self._reduced is None:
            self._reduced = torch.empty(self.flat.shard_size, dtype=torch.float32, device=self.device)
        self._ov = {"hi": self.flat.total, "met": False}

    def range_ready(self, lo: int) -> None:
        """Flat offsets >= lo hold final gradients on THIS rank. Every rank calls this with the same offsets in the
        same order; the range [lo, previous lo) is reduced on the side stream once every rank has got there."""
        ov = self._ov
        if ov is None or lo >= ov["hi"]:
            return
        if ov["hi"] - lo < self.flat.total // (self._buckets + 1):
            return          # too little for a launch of its own: goes with the next layer(s)
        hi, ov["hi"] = ov["hi"], lo
        self._launch_range(lo, hi)

    def _launch_range(self, lo: int, hi: int, tail: bool = False) -> None:
        f, ov = self.flat, self._ov
        f.zero_untouched_in(lo, hi)
        a, b = max(lo, f.shard_lo), min(hi, f.shard_lo + f.shard_size)
        ev = torch.cuda.Event()
        ev.record()                                   # this rank's gradients of the range are complete here
        with torch.cuda.stream(self.side):
            self.side.wait_event(ev)
            if not ov["met"]:
                self.rendezvous()
                ov["met"] = True
            self.side_epoch += 1                      # every rank takes part, also with an empty intersection
            _lib.check(_lib.kernels().b200_p2p_barrier(self.sig_side.c_ptrs, self.rank, self.world, self.side_epoch,
                                                       _lib.stream()), "b200_p2p_barrier")
            if b > a:
                # ranges that run beside backward take a few CTAs; the last one has the GPU to itself
                self.reduce_scatter(self.grad_buf, self._reduced[a - f.shard_lo:b - f.shard_lo], a, 1.0,
                                    0 if tail else self._overlap_ctas)

    # ---- the optimizer step
    def reduce_and_step(self, lr: float, grad_scale: float) -> None:
        f, opt = self.flat, self.opt
        gs = grad_scale / self.world
        if self._ov is not None:
            # the tail of the flat space (first layers, embedding); then, with everything of the side stream done, the
            # update of the shard from the summed gradient and the all-gather of the new weights; the closing barrier
            # says that every rank's weight stores have landed - and that every rank has finished READING the
            # gradients - before the next forward and backward run
            self._launch_range(0, self._ov["hi"], tail=True)
            self._ov = None
            done = torch.cuda.Event()
            done.record(self.side)
            torch.cuda.current_stream().wait_event(done)
            opt.step_count += 1
            b1, b2 = opt.betas
            st = opt.state
            _lib.check(_lib.kernels().b200_p2p_rs_adamw_ag(
                None, _lib.ptr(self._reduced), 2, self.model_buf.c_ptrs, _lib.ptr(f.master), _lib.ptr(st["m"]),
                _lib.ptr(st["v"]), f.shard_lo, f.shard_size, 0, self.rank, self.world, lr, b1, b2, opt.eps,
                opt.weight_decay, opt.step_count, gs, int(opt.decoupled), 0, _lib.stream()), "b200_p2p_rs_adamw_ag")
            self._mark_step()
            self.barrier()
            return
        fused = self._fused()
        if fused:
            self._cast_wire(0, f.total)
        self.rendezvous()
        self.barrier()
        if self.time_exchange:
            self._xev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._xev[0].record()
        if fused:
            opt.step_count += 1
            b1, b2 = opt.betas
            st = opt.state
            gp, own, w16 = self._grad_sources()
            _lib.check(_lib.kernels().b200_p2p_rs_adamw_ag(
                gp, own, w16, self.model_buf.c_ptrs, _lib.ptr(f.master), _lib.ptr(st["m"]), _lib.ptr(st["v"]),
                f.shard_lo, f.shard_size, 0, self.rank, self.world, lr, b1, b2, opt.eps, opt.weight_decay,
                opt.step_count, gs, int(opt.decoupled), 0, _lib.stream()), "b200_p2p_rs_adamw_ag")
        else:
            shard = torch.empty(f.shard_size, dtype=torch.float32, device=self.device)
            self.reduce_scatter(self.grad_buf, shard, f.shard_lo, 1.0)
            opt.step(lr, grad_scale=gs, grad=shard)
            self.allgather(self.model_buf, f.model_shard(), f.shard_lo, skip_self=True)
        self._mark_step()
        self.barrier()
        if self.time_exchange and self._xev is not None:
            self._xev[1].record()

    def exchange_ms(self) -> float | None:
        """Device time of the latest step's exchange proper (reduce-scatter, update, all-gather, closing barrier) when
        ``time_exchange`` was set; the bf16 wire cast and the wait for the slowest rank come before it. Synchronises."""
        if self._xev is None:
            return None
        torch.cuda.synchronize(self.device)
        return float(self._xev[0].elapsed_time(self._xev[1]))
