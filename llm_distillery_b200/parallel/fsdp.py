"""Full parameter sharding for student training (ZeRO-3 / FSDP "full shard").

The reference trains its student on one device with everything resident (classes/student/model.py:139-175); the
largest students it names fit there only with 8-bit optimizers. Here ``shard_strategy = "zero3"`` spreads weights,
gradients, fp32 master weights and optimizer state over the data-parallel ranks:

* The trainable parameters are grouped into UNITS in execution order: the embedding, every decoder layer, and the
  final norm (+ an untied LM head). A unit is padded to a multiple of ``256 * world`` elements and cut into ``world``
  equal pieces; rank r keeps piece r of every unit, in the model dtype, plus the fp32 master copy, the fp32 gradient
  and the optimizer state of exactly those elements ("shard space": the pieces one behind the other).
* Before a unit runs (forward, and again before its backward) its pieces are all-gathered into a unit-sized buffer
  that the parameters' ``.data`` point into. Decoder layers share TWO such buffers and alternate between them, so
  that layer i+1 (forward) / i-1 (backward) is gathered on a side stream while layer i computes; the embedding and
  the head have buffers of their own, which stay valid for the whole step.
* Weight-gradient kernels write fp32 into a unit-sized gradient buffer beside the weights (again two for the
  layers). When a layer's backward is through (``models.llama.LAYER_BACKWARD_DONE``) the buffer is
  reduce-scattered and this rank's piece is added to the gradient of the shard space; the embedding's and the
  head's gradients accumulate over the micro-batches and are reduced once, before the optimizer step.
* The optimizer step is the ordinary flat kernel over the shard space (``engine.optim.FlatOptimizer`` sees
  ``ShardedFlat`` through the interface of ``FlatParams``); no all-gather follows it - the next forward gathers.

Per-rank memory is (2 + 4 + 4 + state) bytes x parameters / world plus two layers and the embedding / head in full,
against (2 + 4) bytes x parameters replicated under ``ddp`` / ``fsdp`` (which shard only master weights and state).

``FullShardComm`` runs the collectives through ``torch.distributed`` (NCCL on GPUs, on a side stream; gloo between
CPU ranks). ``P2PFullShardComm`` replaces them by kernels over NVLink peer access: a handshake-free pull gather, and a
reduction that on the last micro-batch of a step is fused with the AdamW update of the rank's piece. Every rank must
issue the same sequence of collectives: a rank without a micro-batch in the last step of an epoch calls
``idle_micro_step`` instead of skipping.
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist

from ..engine.optim import ALIGN, _round_up
from ..models import llama as _llama
from ..models.llama import GradSlot


def model_units(model) -> list[tuple[str, list[torch.nn.Parameter]]]:
    """Trainable parameters of a LlamaModel grouped in execution order; frozen parameters stay whole on every rank."""
    tied = model.lm_head is model.embed_tokens
    raw = [("embed", [model.embed_tokens])]
    raw += [(f"layer{i}", list(layer.parameters())) for i, layer in enumerate(model.layers)]
    raw.append(("head", [model.norm] + ([] if tied else [model.lm_head])))
    out = []
    for name, ps in raw:
        ps = [p for p in ps if p.requires_grad]
        if ps:
            out.append((name, ps))
    return out


class _Unit:
    def __init__(self, index: int, name: str, params, world: int):
        self.index, self.name, self.params = index, name, params
        self.offsets, off = [], 0
        for p in params:
            self.offsets.append(off)
            off += _round_up(p.numel(), ALIGN)
        self.payload = off           # elements before the padding that depends on the world size
        self.numel = _round_up(off, 256 * world)
        self.piece = self.numel // world
        self.is_layer = name.startswith("layer")
        self.shard_lo = 0            # offset of this rank's piece in the shard space
        self.slot = -1               # which of the two rotating buffers (layers only)
        self.weights = None          # [numel] model dtype: where the gathered unit lives
        self.grads = None            # [numel] fp32
        self.slots: list[GradSlot] = []
        self.valid = False           # weights hold the current values (dedicated buffers only)
        self.reduced = False         # a reduce-scatter of this unit has already gone into the shard gradient this step
        self.stepped = False         # the optimizer update of this unit's piece has been done with its last reduction


class ShardedFlat:
    """The shard space of one rank, with the attribute / method surface of ``engine.optim.FlatParams``."""

    layout = "per_unit"

    def __init__(self, model, rank: int, world: int, alloc=None):
        """``alloc(numel, dtype, role)`` returns a zeroed buffer; roles "shard" (this rank's weight pieces) and "grads"
        (a unit-sized gradient buffer) are what peers read under the peer-to-peer communicator."""
        units = model_units(model)
        if not units:
            raise ValueError("no trainable parameters")
        self.rank, self.world = rank, world
        self.units = [_Unit(i, n, ps, world) for i, (n, ps) in enumerate(units)]
        first = self.units[0].params[0]
        self.dtype, self.device = first.dtype, first.device
        self.params = [p for u in self.units for p in u.params]
        off = 0
        for u in self.units:
            u.shard_lo = off
            off += u.piece
        self.shard_size = off
        self.shard_lo = rank * off             # nominal: the shard space is not a slice of one flat space
        self.total = off * world
        kw = dict(device=self.device)
        if alloc is None:
            alloc = lambda n, dt, role: torch.zeros(n, dtype=dt, **kw)      # noqa: E731
        self._model_shard = alloc(off, self.dtype, "shard")
        self._grad_shard = torch.zeros(off, dtype=torch.float32, **kw)
        # gather buffers: two shared by the layers, one each for the other units
        layers = [u for u in self.units if u.is_layer]
        big = max((u.numel for u in layers), default=0)
        self.rot_w = [torch.zeros(big, dtype=self.dtype, **kw) for _ in range(2 if layers else 0)]
        self.rot_g = [alloc(big, torch.float32, "grads") for _ in range(2 if layers else 0)]
        self.rot_owner: list[int | None] = [None, None]
        for k, u in enumerate(layers):
            u.slot = k & 1
            u.weights, u.grads = self.rot_w[u.slot][:u.numel], self.rot_g[u.slot][:u.numel]
        for u in self.units:
            if not u.is_layer:
                u.weights = torch.zeros(u.numel, dtype=self.dtype, **kw)
                u.grads = alloc(u.numel, torch.float32, "grads")
        self.unit_of: dict[int, _Unit] = {}
        self.slots: list[GradSlot] = []
        with torch.no_grad():
            for u in self.units:
                full = torch.zeros(u.numel, dtype=self.dtype, **kw)
                for p, o in zip(u.params, u.offsets):
                    full[o:o + p.numel()].copy_(p.data.reshape(-1))
                self.piece_of(u).copy_(full[rank * u.piece:(rank + 1) * u.piece])
                del full
                for p, o in zip(u.params, u.offsets):
                    n = p.numel()
                    p.data = u.weights[o:o + n].view(p.shape)          # the full copy of the parameter is dropped here
                    slot = GradSlot(u.grads[o:o + n].view(p.shape))
                    p.grad_slot = slot
                    u.slots.append(slot)
                    self.slots.append(slot)
                    self.unit_of[id(p)] = u
        self.master = self._model_shard.float().clone()

    def unit_table(self) -> list[tuple[str, int, int]]:
        """(name, elements before padding, piece length) per unit in shard-space order: what a checkpoint needs to
        re-cut the pieces for another world size."""
        return [(u.name, u.payload, u.piece) for u in self.units]

    # ---- FlatParams surface
    def piece_of(self, u: _Unit) -> torch.Tensor:
        return self._model_shard[u.shard_lo:u.shard_lo + u.piece]

    def grad_piece_of(self, u: _Unit) -> torch.Tensor:
        return self._grad_shard[u.shard_lo:u.shard_lo + u.piece]

    def grad_shard(self) -> torch.Tensor:
        return self._grad_shard

    def model_shard(self) -> torch.Tensor:
        return self._model_shard

    def offset_of(self, p):
        return None

    def mark_fresh(self) -> None:
        for s in self.slots:
            s.fresh = True

    def untouched_to_zero(self) -> None:
        """Only the units whose gradients live until the step (embedding, head): a layer's untouched parameters are
        zeroed when that layer's buffer is reduced."""
        for u in self.units:
            if not u.is_layer:
                for s in u.slots:
                    if s.fresh:
                        s.buf.zero_()
                        s.fresh = False

    def absorb_autograd_grads(self) -> None:
        for p, s in zip(self.params, self.slots):
            if p.grad is not None:
                if s.fresh:
                    s.buf.copy_(p.grad)
                    s.fresh = False
                else:
                    s.buf.add_(p.grad)
                p.grad = None


class FullShardComm:
    """Communicator for ``shard_strategy = "zero3"``: builds the ``ShardedFlat`` and drives gather / reduce-scatter
    from the model's unit hooks."""

    shards_optimizer = True
    full_shard = True

    def __init__(self, device, group=None):
        self.device = torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.cuda = self.device.type == "cuda"
        self.gloo = dist.get_backend(group) == "gloo"
        self.side = torch.cuda.Stream(device=self.device) if self.cuda else None
        self.flat: ShardedFlat | None = None
        self.opt = None
        self._ready: dict[int, object] = {}        # unit index -> event: its gather has finished (side stream)
        self._grads_free = [None, None]            # rotating gradient buffer -> event: its reduce-scatter has finished
        self._tmp = None
        self.stats = {"gathers": 0, "reduces": 0}

    # ---- engine interface
    def build_flat(self, model) -> ShardedFlat:
        self.flat = ShardedFlat(model, self.rank, self.world, alloc=self._alloc())
        self._ready.clear()
        self._grads_free = [None, None]
        for layer in model.layers:          # frozen parameters of a partly trainable layer also identify its unit
            ps = list(layer.parameters())
            u = next((self.flat.unit_of[id(q)] for q in ps if id(q) in self.flat.unit_of), None)
            if u is not None:
                for q in ps:
                    self.flat.unit_of.setdefault(id(q), u)
        head = next((u for u in self.flat.units if u.name == "head"), None)
        if head is not None:
            self.flat.unit_of.setdefault(id(model.norm), head)
        big = max((u.piece for u in self.flat.units if u.is_layer), default=0)
        self._tmp = [torch.zeros(big, dtype=torch.float32, device=self.device) for _ in range(2)]
        return self.flat

    def allocate_flat_buffers(self, model):
        return None

    def attach(self, flat, opt) -> None:
        if flat is not self.flat:
            raise RuntimeError("the engine must use the flat space built by build_flat")
        self.opt = opt
        # the model calls ONE pair of module-level hooks: a second fully sharded engine in the same process would
        # silently take them away from the first
        other = getattr(_llama.UNIT_PRE[0], "__self__", None)
        if other is not None and other is not self and getattr(other, "flat", None) is not None:
            raise RuntimeError("another fully sharded engine is active in this process: close() its communicator first")
        _llama.UNIT_PRE[0] = self._pre
        _llama.LAYER_BACKWARD_DONE[0] = self._layer_done

    def close(self) -> None:
        self.flat = self.opt = self._tmp = None
        if _llama.UNIT_PRE[0] == self._pre:
            _llama.UNIT_PRE[0] = None
        if _llama.LAYER_BACKWARD_DONE[0] == self._layer_done:
            _llama.LAYER_BACKWARD_DONE[0] = None

    def barrier(self) -> None:
        dist.barrier(self.group)

    def shards_written(self) -> None:
        """This rank's weight pieces were written outside the step protocol (construction, a checkpoint load). Nothing
        to do here: an all-gather reads the local piece in stream order and waits for the peers by itself."""

    # ---- collectives (every rank issues them in the same host order; on GPUs all of them on the side stream)
    def _all_gather(self, out: torch.Tensor, piece: torch.Tensor) -> None:
        if self.gloo:
            parts = [torch.empty_like(piece) for _ in range(self.world)]
            dist.all_gather(parts, piece.contiguous(), group=self.group)
            out.copy_(torch.cat(parts))
        else:
            dist.all_gather_into_tensor(out, piece, group=self.group)

    def _reduce_scatter(self, out: torch.Tensor, full: torch.Tensor) -> None:
        if self.gloo:
            dist.all_reduce(full, op=dist.ReduceOp.SUM, group=self.group)
            out.copy_(full[self.rank * out.numel():(self.rank + 1) * out.numel()])
        else:
            dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.SUM, group=self.group)

    def _on_side(self):
        """Context: the side stream, ordered after everything enqueued on the current stream so far."""
        if not self.cuda:
            return contextlib.nullcontext()
        ev = torch.cuda.Event()
        ev.record()
        self.side.wait_event(ev)
        return torch.cuda.stream(self.side)

    def _issue_gather(self, u: _Unit) -> None:
        """Start the all-gather of a unit into its buffer, unless the buffer already holds it."""
        f = self.flat
        if u.is_layer:
            if f.rot_owner[u.slot] == u.index:
                return
            f.rot_owner[u.slot] = u.index
        else:
            if u.valid:
                return
            u.valid = True
        with self._on_side():
            self._gather_unit(u)
            if self.cuda:
                ev = torch.cuda.Event()
                ev.record()
                self._ready[u.index] = ev
        self.stats["gathers"] += 1

    def _gather_unit(self, u: _Unit) -> None:
        self._all_gather(u.weights, self.flat.piece_of(u))

    def _alloc(self):
        return None

    def _wait_ready(self, u: _Unit) -> None:
        ev = self._ready.pop(u.index, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def _neighbour(self, u: _Unit, step: int):
        i = u.index + step
        return self.flat.units[i] if 0 <= i < len(self.flat.units) else None

    # ---- hooks from the model
    def _pre(self, param, backward: bool = False) -> None:
        """A unit is about to read its parameters (``param`` is any of them)."""
        u = self.flat.unit_of.get(id(param))
        if u is None:
            return
        self._issue_gather(u)
        self._wait_ready(u)
        if backward and u.is_layer:
            self._before_backward_writes(u)
        # next unit in execution order: gathered behind this unit's compute. Going backward only layers are needed
        # again (embedding backward reads no weights; the head ran just before)
        nxt = self._neighbour(u, -1 if backward else 1)
        if nxt is not None and (nxt.is_layer or not backward):
            self._issue_gather(nxt)

    def _layer_done(self, first_param) -> None:
        """All weight gradients of a layer are in its gradient buffer: reduce them into the shard gradient."""
        u = self.flat.unit_of.get(id(first_param))
        if u is not None and u.is_layer:
            self._reduce_unit(u)

    def _reduce_unit(self, u: _Unit) -> None:
        f = self.flat
        for s in u.slots:
            if s.fresh:                 # a parameter without a gradient this time
                s.buf.zero_()
        with self._on_side():
            self._reduce_op(u)
        u.reduced = True
        for s in u.slots:
            s.fresh = True
        self.stats["reduces"] += 1

    def _reduce_op(self, u: _Unit) -> None:
        """On the side stream: sum the unit's gradient buffers over the ranks onto this rank's piece."""
        dst = self.flat.grad_piece_of(u)
        if not u.reduced:
            self._reduce_scatter(dst, u.grads)
        else:
            tmp = self._tmp[u.slot][:u.piece] if u.is_layer else torch.empty_like(dst)
            self._reduce_scatter(tmp, u.grads)
            dst.add_(tmp)
        if self.cuda and u.is_layer:
            ev = torch.cuda.Event()
            ev.record()
            self._grads_free[u.slot] = ev

    def _before_backward_writes(self, u: _Unit) -> None:
        """A layer's backward is about to write its gradient buffer."""
        if self._grads_free[u.slot] is not None:
            # the previous owner's gradients must have left the buffer before this layer's wgrad kernels write it
            torch.cuda.current_stream().wait_event(self._grads_free[u.slot])
            self._grads_free[u.slot] = None

    def _step_begin(self) -> None:
        pass

    def _step_end(self) -> None:
        pass

    def idle_micro_step(self) -> None:
        """The collectives of one micro-batch's forward + backward with a zero gradient contribution: for a rank
        that has no micro-batch while the others have one."""
        units = self.flat.units
        for u in units:
            self._pre(u.params[0])
        for u in reversed(units):
            if u.is_layer:
                self._pre(u.params[0], backward=True)
                self._reduce_unit(u)

    # ---- the optimizer step
    def reduce_and_step(self, lr: float, grad_scale: float) -> None:
        f = self.flat
        self._step_begin()
        for u in f.units:
            if not u.is_layer:
                self._reduce_unit(u)
            elif not u.reduced:             # a step without any backward: that gradient is zero, not last step's
                f.grad_piece_of(u).zero_()
        if self.cuda:
            done = torch.cuda.Event()
            done.record(self.side)
            torch.cuda.current_stream().wait_event(done)
        self.opt.step(lr, grad_scale=grad_scale / self.world, grad=f.grad_shard())
        for u in f.units:
            u.valid = False
            u.reduced = False
        f.rot_owner = [None, None]
        self._ready.clear()
        self._step_end()

    # ---- whole-model access (checkpoints)
    @contextlib.contextmanager
    def gathered(self, writeback: bool = False):
        """Inside the block every parameter holds its full, current value (a temporary whole copy of the model; all
        ranks enter together). ``writeback``: values stored into the parameters inside the block become the new
        weights (this rank's pieces and their fp32 master copies are re-cut from them on exit)."""
        f = self.flat
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.side)
        temps = []
        with torch.no_grad():
            for u in f.units:
                t = torch.empty(u.numel, dtype=f.dtype, device=f.device)
                self._all_gather(t, f.piece_of(u))
                temps.append(t)
                for p, o in zip(u.params, u.offsets):
                    p.data = t[o:o + p.numel()].view(p.shape)
        try:
            yield
        finally:
            with torch.no_grad():
                for u, t in zip(f.units, temps):
                    if writeback:
                        f.piece_of(u).copy_(t[self.rank * u.piece:(self.rank + 1) * u.piece])
                    for p, o in zip(u.params, u.offsets):
                        p.data = u.weights[o:o + p.numel()].view(p.shape)
                    u.valid = False
                if writeback:
                    f.master.copy_(f.model_shard().float())
            f.rot_owner = [None, None]
            if writeback:
                self.shards_written()


class P2PFullShardComm(FullShardComm):
    """Full sharding over NVLink peer access (kernels: csrc/comm/p2p.cu) instead of NCCL.

    * This rank's weight pieces live in symmetric memory. A unit is gathered by ONE kernel that loads every rank's
      piece straight out of its memory (``gather_pull``): the pieces do not change between two optimizer steps, so a
      gather needs no handshake at all - only the optimizer step is bracketed by flag barriers.
    * The unit-sized gradient buffers live in symmetric memory. After a layer's backward: flag barrier (every rank's
      gradients of the layer are complete), then one kernel sums the ranks' buffers over this rank's slice onto the
      gradient of the shard space (``reduce_scatter_acc``). The barrier of the NEXT reduction tells a rank that all
      peers have finished reading the previous buffer, which is when its next owner may overwrite it.

    All of it runs on the side stream, behind the compute of the neighbouring layer. Every device-side wait is
    bounded and reports through the device error word (``check``).
    """

    def __init__(self, device, group=None):
        super().__init__(device, group)
        from ..ops import _lib
        from ..ops._lib import _VP, _I, _LL
        from .p2p import SymmetricBuffer
        import ctypes
        _lib.register("b200_p2p_barrier", [_VP, _I, _I, ctypes.c_uint, _VP])
        _lib.register("b200_p2p_gather_pull", [_VP, _VP, _LL, _LL, _I, _I, _VP])
        _lib.register("b200_p2p_reduce_scatter_acc_f32", [_VP, _VP, _LL, _LL, _I, _I, _I, _VP])
        _F = ctypes.c_float
        _lib.register("b200_p2p_rs_adamw_piece", [_VP, _LL, _VP, _VP, _VP, _VP, _VP, _LL, _I, _I, _F, _F, _F, _F, _F, _I,
                                                  _F, _I, _VP])
        self._fused = None            # {"lr", "gs"} during the last micro-batch of a step and the step that follows
        self._met = False             # an NCCL rendezvous has preceded the flag barriers since the last forward began
        self._rdv = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._lib = _lib
        self._SymmetricBuffer = SymmetricBuffer
        self.sig = SymmetricBuffer(64, torch.int32, self.device)
        self.epoch = 0
        self._sym: dict[int, object] = {}
        self._unprotected = None      # rotating gradient buffer read by the latest reduction, no barrier issued since
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def _alloc(self):
        def alloc(n, dtype, role):
            buf = self._SymmetricBuffer(max(int(n), 64), dtype, self.device)      # zero-filled, mapped on every rank
            self._sym[buf.tensor.data_ptr()] = buf
            return buf.tensor[:n]
        self._sym.clear()
        self._unprotected = None
        return alloc

    def close(self) -> None:
        super().close()
        self._sym.clear()

    def build_flat(self, model) -> ShardedFlat:
        flat = super().build_flat(model)
        self.shards_written()
        return flat

    def shards_written(self) -> None:
        """Peers read this rank's pieces straight out of its memory, and a pull gather involves no handshake: after
        writes outside the step protocol every rank waits until all of them have finished theirs (host barrier; these
        are start-up and checkpoint-load moments, not the training loop)."""
        torch.cuda.current_stream().synchronize()
        dist.barrier(self.group)

    def _pre(self, param, backward: bool = False) -> None:
        if not backward:
            self._met = False         # a new forward: this rank may have waited for its batch for any length of time
        super()._pre(param, backward)

    def _barrier(self) -> None:
        if not self._met:
            # ranks can be seconds apart here (a checkpoint being written, a batch late from disk) while the flag
            # barrier gives up after two: let NCCL, whose wait has no such bound, bring the streams together first
            dist.all_reduce(self._rdv, group=self.group)
            self._met = True
        self.epoch += 1
        self._lib.check(self._lib.kernels().b200_p2p_barrier(self.sig.c_ptrs, self.rank, self.world, self.epoch,
                                                             self._lib.stream()), "b200_p2p_barrier")

    def check(self) -> None:
        err = self._lib.take_device_error()
        if err:
            # the barrier that gave up switched this GPU's peer kernels off (csrc/comm/p2p.cu): nothing behind it ran
            from ..ops._lib import _VP
            self._lib.register("b200_p2p_clear_poison", [_VP])
            self._lib.check(self._lib.kernels().b200_p2p_clear_poison(self._lib.stream()), "b200_p2p_clear_poison")
            torch.cuda.synchronize()
            raise RuntimeError(f"peer-to-peer wait timed out on rank {self.rank} (device error code {err})")

    def _gather_unit(self, u: _Unit) -> None:
        f = self.flat
        es = f.model_shard().element_size()
        src = self._sym[f.model_shard().data_ptr()]
        self._lib.check(self._lib.kernels().b200_p2p_gather_pull(
            src.c_ptrs, self._lib.ptr(u.weights), u.shard_lo * es, u.piece * es, self.rank, self.world,
            self._lib.stream()), "b200_p2p_gather_pull")

    def _mark_protected(self) -> None:
        """Call right after a barrier on the side stream: every peer has finished its earlier reductions."""
        if self._unprotected is not None:
            ev = torch.cuda.Event()
            ev.record()
            self._grads_free[self._unprotected] = ev
            self._unprotected = None

    def _reduce_op(self, u: _Unit) -> None:
        self._barrier()
        self._mark_protected()
        src = self._sym[u.grads.data_ptr()]
        dst = self.flat.grad_piece_of(u)
        lib, ptr = self._lib.kernels(), self._lib.ptr
        if self._fused is not None:
            # the optimizer step follows this micro-batch: reduce + AdamW on this rank's piece in one kernel. Nobody
            # gathers this unit again before the step is over, so its weight piece may change now
            f, opt = self.flat, self.opt
            lo, hi = u.shard_lo, u.shard_lo + u.piece
            b1, b2 = opt.betas
            self._lib.check(lib.b200_p2p_rs_adamw_piece(
                src.c_ptrs, self.rank * u.piece, ptr(dst) if u.reduced else None, ptr(f.model_shard()[lo:hi]),
                ptr(f.master[lo:hi]), ptr(opt.state["m"][lo:hi]), ptr(opt.state["v"][lo:hi]), u.piece, self.rank,
                self.world, self._fused["lr"], b1, b2, opt.eps, opt.weight_decay, opt.step_count, self._fused["gs"],
                int(opt.decoupled), self._lib.stream()), "b200_p2p_rs_adamw_piece")
            u.stepped = True
        else:
            self._lib.check(lib.b200_p2p_reduce_scatter_acc_f32(
                src.c_ptrs, ptr(dst), self.rank * u.piece, u.piece, self.rank, self.world, int(u.reduced),
                self._lib.stream()), "b200_p2p_reduce_scatter_acc_f32")
        if u.is_layer:
            self._unprotected = u.slot

    def last_micro_batch(self, lr: float, grad_scale: float) -> None:
        """The optimizer step follows the micro-batch whose backward starts now (every rank is told the same)."""
        opt = self.opt
        if (opt.name in ("adam", "adamw", "adamw32bit", "paged_adamw", "paged_adamw32bit") and "m" in opt.state
                and self.flat.dtype == torch.bfloat16 and self._fused is None):
            opt.step_count += 1
            self._fused = {"lr": float(lr), "gs": float(grad_scale) / self.world}

    def reduce_and_step(self, lr: float, grad_scale: float) -> None:
        if self._fused is None:
            return super().reduce_and_step(lr, grad_scale)
        f = self.flat
        self._step_begin()
        for u in f.units:
            if not u.stepped:           # embedding and head (their gradients were still accumulating); a layer
                self._reduce_unit(u)    # whose backward did not run contributes its zeroed buffer
        done = torch.cuda.Event()
        done.record(self.side)
        torch.cuda.current_stream().wait_event(done)
        for u in f.units:
            u.valid = u.reduced = u.stepped = False
        f.rot_owner = [None, None]
        self._ready.clear()
        self._fused = None
        self._step_end()

    def _before_backward_writes(self, u: _Unit) -> None:
        if self._unprotected == u.slot:
            # the latest reduction read this very buffer (first layer of the previous micro-batch's backward order):
            # peers may still be reading it, and no later reduction's barrier has vouched for them yet
            with self._on_side():
                self._barrier()
                self._mark_protected()
        super()._before_backward_writes(u)

    def _step_begin(self) -> None:
        # peers may still be pulling weights for an evaluation pass: nobody's optimizer overwrites its pieces before
        # every rank has got here
        with self._on_side():
            self._barrier()
            self._mark_protected()

    def _step_end(self) -> None:
        # the new pieces of every rank are in place before anyone gathers them
        with self._on_side():
            self._barrier()
            self._mark_protected()
        self._grads_free = [None, None]
