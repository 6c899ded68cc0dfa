"""NVLink peer-to-peer communicator for the flat parameter space (kernels: csrc/comm/p2p.cu).

The flat fp32 gradient and the flat bf16 weights are allocated in symmetric memory, so every rank holds device
pointers to every other rank's copies. One optimizer step is then

    barrier (all backward passes done)  ->  rs_adamw_ag kernel  ->  barrier (all weight stores landed)

where the middle kernel, for this rank's 1/world shard, sums all ranks' gradients with peer loads, applies AdamW to
the local fp32 master weights / moments and writes the new bf16 weights into every rank's weight buffer with peer
stores. Optimizer state is therefore sharded (ZeRO-1) for ``ddp`` and ``fsdp`` alike. Optimizers other than the
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
_lib.register("b200_p2p_rs_adamw_ag", [_VP, _VP, _VP, _VP, _VP, _LL, _LL, _I, _I, _F, _F, _F, _F, _F, _I, _F, _I, _VP])
_lib.register("b200_p2p_reduce_scatter_f32", [_VP, _VP, _LL, _LL, _I, _I, _F, _VP])
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
        # off by default: on 2 and 8 B200s the step was 1-2 % SLOWER with the reduction running beside backward (the
        # side-stream kernel competes with the backward GEMMs for HBM and SM slots, and the reduction it hides is
        # only ~4 % of the step); B200_OVERLAP=1 turns it on
        self._overlap_enabled = os.environ.get("B200_OVERLAP", "0") == "1"
        self._buckets = max(1, int(os.environ.get("B200_OVERLAP_BUCKETS", "4")))   # ranges per step handed over early
        self.grad_buf = None
        self.model_buf = None
        self._rdv = torch.zeros(1, dtype=torch.float32, device=self.device)
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

    def check(self) -> None:
        err = _lib.take_device_error()
        if err:
            raise RuntimeError(f"peer-to-peer wait timed out on rank {self.rank} (device error code {err})")

    def reduce_scatter(self, src: SymmetricBuffer, out: torch.Tensor, lo: int, scale: float = 1.0) -> None:
        """out[i] = scale * sum over ranks of src[lo + i]; callers bracket this with barriers."""
        _lib.check(_lib.kernels().b200_p2p_reduce_scatter_f32(src.c_ptrs, _lib.ptr(out), lo, out.numel(), self.rank,
                                                              self.world, float(scale), _lib.stream()), "p2p reduce_scatter")

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
        self.opt.step_count += 1
        self._ov = {"lr": lr, "gs": grad_scale / self.world, "hi": self.flat.total, "met": False}

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

    def _launch_range(self, lo: int, hi: int) -> None:
        f, opt, ov = self.flat, self.opt, self._ov
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
                o = a - f.shard_lo
                b1, b2 = opt.betas
                st = opt.state
                _lib.check(_lib.kernels().b200_p2p_rs_adamw_ag(
                    self.grad_buf.c_ptrs, self.model_buf.c_ptrs, _lib.ptr(f.master[o:]), _lib.ptr(st["m"][o:]),
                    _lib.ptr(st["v"][o:]), a, b - a, self.rank, self.world, ov["lr"], b1, b2, opt.eps,
                    opt.weight_decay, opt.step_count, ov["gs"], int(opt.decoupled), _lib.stream()),
                    "b200_p2p_rs_adamw_ag")

    # ---- the optimizer step
    def reduce_and_step(self, lr: float, grad_scale: float) -> None:
        f, opt = self.flat, self.opt
        gs = grad_scale / self.world
        if self._ov is not None:
            # the tail of the flat space (first layers, embedding) and then: everything of the side stream is done,
            # and every rank's weight stores have landed, before the next forward reads the weights
            self._launch_range(0, self._ov["hi"])
            self._ov = None
            done = torch.cuda.Event()
            done.record(self.side)
            torch.cuda.current_stream().wait_event(done)
            self.barrier()
            return
        self.rendezvous()
        self.barrier()
        fused = self._fused()
        if fused:
            opt.step_count += 1
            b1, b2 = opt.betas
            st = opt.state
            _lib.check(_lib.kernels().b200_p2p_rs_adamw_ag(
                self.grad_buf.c_ptrs, self.model_buf.c_ptrs, _lib.ptr(f.master), _lib.ptr(st["m"]), _lib.ptr(st["v"]),
                f.shard_lo, f.shard_size, self.rank, self.world, lr, b1, b2, opt.eps, opt.weight_decay, opt.step_count,
                gs, int(opt.decoupled), _lib.stream()), "b200_p2p_rs_adamw_ag")
        else:
            shard = torch.empty(f.shard_size, dtype=torch.float32, device=self.device)
            self.reduce_scatter(self.grad_buf, shard, f.shard_lo, 1.0)
            opt.step(lr, grad_scale=gs, grad=shard)
            self.allgather(self.model_buf, f.model_shard(), f.shard_lo, skip_self=True)
        self.barrier()
