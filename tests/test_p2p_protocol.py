"""Race check of the data-parallel peer-to-peer communicator (``parallel.p2p.P2PComm``) on the host, with the recorders
and the happens-before checker of ``tests/test_zero3_protocol.py``.

Default schedule: backward -> rendezvous + flag barrier -> ONE kernel (peers' gradient shards read, AdamW, new weights
stored into EVERY rank's weight buffer) -> flag barrier. Overlapped schedule (``B200_OVERLAP=1``): each finished layer
range is handed to the side stream (own flag words), which sums it over the ranks into a local buffer behind the
backward of the earlier layers; the kernel after backward updates the shard from that buffer and stores the new weights
into every rank's buffer. Memory is tracked per
segment of the flat parameter space (cut at parameter and shard boundaries), per rank: the kernel's peer loads of a
gradient segment must be ordered against the owner's weight-gradient writes of this and of the next step, and its peer
stores of a weight segment against every rank's compute that reads it. With the bf16 wire format every rank first
copies its gradient into a wire buffer that the peers read instead: the copy must follow the gradient writes, and the
next step's copy must follow every peer's read of this step's.
"""
import bisect

import pytest
import torch

from llm_distillery_b200.engine.trainer import DistillEngine, synthetic_batch
from llm_distillery_b200.models.llama import LlamaConfig, build_model
from llm_distillery_b200.parallel import p2p

from tests import test_zero3_protocol as zp
from tests.test_zero3_protocol import recorders  # noqa: F401  (fixture)


class Segments:
    """The flat space cut at every parameter start and every shard boundary."""

    def __init__(self, flat):
        cuts = sorted(set(flat.offsets) | {r * flat.shard_size for r in range(flat.world + 1)} | {0, flat.total})
        self.cuts = cuts

    def span(self, lo, hi):
        """Indices of the segments that intersect [lo, hi)."""
        if hi <= lo:
            return range(0)
        a = bisect.bisect_right(self.cuts, lo) - 1
        b = bisect.bisect_left(self.cuts, hi)
        return range(max(a, 0), max(b, 0))

    def below(self, hi):
        return self.span(0, hi)

    @property
    def all(self):
        return range(len(self.cuts) - 1)


class P2PKernels:
    def __init__(self, seg: Segments, shard_lo: int, shard_size: int, comm=None):
        self.seg, self.shard_lo, self.shard_size, self.comm = seg, shard_lo, shard_size, comm

    def _in_reduced(self, ptr):
        """Flat offset of a pointer into the communicator's summed-gradient buffer, or None."""
        red = getattr(self.comm, "_reduced", None)
        if red is None or ptr is None:
            return None
        off = int(getattr(ptr, "value", ptr) or 0) - red.data_ptr()
        return self.shard_lo + off // 4 if 0 <= off < red.numel() * 4 else None

    def b200_p2p_barrier(self, sig, rank, world, epoch, stream):
        zp.SIM.collective(("flag", sig, int(epoch)))
        return 0

    def b200_p2p_rs_adamw_ag(self, grads, own, wire16, models, master, m, v, lo, n, state_off, rank, world, *rest):
        segs = list(self.seg.span(lo, lo + n))
        assert state_off == lo - self.shard_lo
        if wire16 == 2:   # the sum is already in the local buffer
            assert self._in_reduced(own) == self.shard_lo
            reads = {("reduced", rank, k) for k in segs}
        elif wire16:      # own fp32 gradient + the peers' wire copies
            reads = {("grad", rank, k) for k in segs} | {("wire", r, k) for r in range(world) if r != rank for k in segs}
        else:
            reads = {("grad", r, k) for r in range(world) for k in segs}
        zp.SIM.add("reduce+adamw+allgather", reads=reads,
                   writes={("model", r, k) for r in range(world) for k in segs} | {("state", rank, k) for k in segs})
        return 0

    def b200_p2p_mark_step(self, counter, stream):
        return 0

    def b200_p2p_cast_wire(self, grad, wire, lo, n, stream):
        segs = list(self.seg.span(lo, lo + n))
        rank = zp.SIM.rank
        zp.SIM.add("cast wire", reads={("grad", rank, k) for k in segs}, writes={("wire", rank, k) for k in segs})
        return 0

    def b200_p2p_reduce_scatter_f32(self, src, out, lo, n, rank, world, scale, max_ctas, stream):
        segs = list(self.seg.span(lo, lo + n))
        where = self._in_reduced(out)
        if where is not None:
            assert where == lo          # the buffer is indexed like the shard
            writes = {("reduced", rank, k) for k in segs}
        else:
            writes = {("tmp", rank, 0)}
        zp.SIM.add("reduce", reads={("grad", r, k) for r in range(world) for k in segs}, writes=writes)
        return 0

    def b200_p2p_allgather(self, dst, local, lo_bytes, nbytes, rank, world, skip_self, stream):
        segs = list(self.seg.span(self.shard_lo, self.shard_lo + self.shard_size))
        peers = [r for r in range(world) if not (skip_self and r == rank)]
        zp.SIM.add("allgather", reads={("model", rank, k) for k in segs},
                   writes={("model", r, k) for r in peers for k in segs})
        return 0


class TracedP2P(p2p.P2PComm):
    fused = True

    def _fused(self):                 # the real check also wants bf16 weights; the schedule is the same
        return self.fused and self.opt.name == "adamw"

    def range_ready(self, lo):
        S = zp.SIM
        S.end_window()
        super().range_ready(lo)
        if self._ov is not None:       # what is left of this backward touches only the parameters below `lo`
            below = self.segments.below(lo)
            S.begin_window({("model", self.rank, k) for k in below}, {("grad", self.rank, k) for k in below})


def trace_rank(monkeypatch, rank, world, layers, steps, overlap, optimizer="adamw", wire=True):
    zp.SIM = S = zp.Sim(rank, world)
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=layers,
                      num_attention_heads=2, num_key_value_heads=1, max_position_embeddings=32)
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=1)
    comm = TracedP2P("cpu")
    comm._wire16 = wire
    comm._overlap_enabled = overlap
    comm._buckets = 64                # hand every layer over on its own
    comm.side = zp.FakeStream("S")
    accum = max(len(st) for st in steps)
    eng = DistillEngine(model, loss="kl", temperature=1.0, optimizer=optimizer, lr=1e-3, grad_accum=accum, comm=comm)
    flat = eng.flat
    if wire:        # the traced model is fp32 (CPU); the schedule of the bf16 wire copy is the same
        comm.wire_buf = zp.FakeSym(flat.total, torch.bfloat16, "cpu")
    comm.segments = seg = Segments(flat)
    monkeypatch.setattr(zp._lib, "kernels", lambda: P2PKernels(seg, flat.shard_lo, flat.shard_size, comm))
    monkeypatch.setattr(zp._lib, "ptr", lambda t: 0 if t is None else t.data_ptr())   # the recorders tell buffers apart
    real_step = eng.opt.step

    def traced_step(lr=None, grad_scale=1.0, grad=None):
        mine = seg.span(flat.shard_lo, flat.shard_lo + flat.shard_size)
        S.add("optimizer", "M", reads={("tmp", rank, 0)}, writes={("model", rank, k) for k in mine})
        return real_step(lr, grad_scale, grad)
    eng.opt.step = traced_step
    hb = synthetic_batch(cfg.vocab_size, 1, 16, 4, seed=rank)
    everything = ({("model", rank, k) for k in seg.all}, {("grad", rank, k) for k in seg.all})
    for st in steps:
        for j, kind in enumerate(st):
            if kind == "eval":
                S.begin_window(everything[0], set())
                eng.eval_batch(hb)
                S.end_window()
                continue
            S.begin_window(*everything)          # forward + backward of the micro-batch
            eng.micro_step(hb.to_device("cpu"), last=(j + 1 == len(st)))
            S.end_window()
        eng.optimizer_step()
    return S.ops


def run(monkeypatch, world, layers, steps, overlap, optimizer="adamw", wire=True):
    traces = [trace_rank(monkeypatch, r, world, layers, steps, overlap, optimizer, wire) for r in range(world)]
    kinds = {op["kind"] for t in traces for op in t}
    assert "arrive" in kinds and ("reduce+adamw+allgather" in kinds or optimizer != "adamw")
    if overlap and optimizer == "adamw":
        assert any(op["kind"] == "reduce" and op["stream"] == "S" for t in traces for op in t)
    return zp.find_races(traces)


STEPS = {"plain": [["train"], ["train"], ["train"]], "accumulation": [["train", "train"], ["train", "train"]],
         "validation between": [["train"], ["eval", "train"], ["eval", "train", "train"]]}


@pytest.mark.parametrize("overlap", [False, True], ids=["after backward", "behind backward"])
@pytest.mark.parametrize("layers", [2, 3])
@pytest.mark.parametrize("name", list(STEPS))
def test_no_unordered_conflicting_accesses(recorders, monkeypatch, name, layers, overlap):  # noqa: F811
    races = run(monkeypatch, 2, layers, STEPS[name], overlap)
    assert not races, f"{len(races)} unordered pairs, e.g.\n" + "\n".join(races[:8])


def test_three_ranks_and_the_unfused_optimizers(recorders, monkeypatch):  # noqa: F811
    assert not run(monkeypatch, 3, 2, STEPS["accumulation"], True)
    assert not run(monkeypatch, 2, 2, STEPS["plain"], False, optimizer="sgd")


@pytest.mark.parametrize("overlap", [False, True])
def test_fp32_exchange_without_the_wire_copy(recorders, monkeypatch, overlap):  # noqa: F811
    assert not run(monkeypatch, 2, 3, STEPS["accumulation"], overlap, wire=False)


@pytest.mark.parametrize("what", ["main-stream barriers", "side-stream wait for backward"])
def test_the_checker_sees_a_removed_ordering(recorders, monkeypatch, what):  # noqa: F811
    if what == "main-stream barriers":
        monkeypatch.setattr(p2p.P2PComm, "barrier", lambda self: None)
        races = run(monkeypatch, 2, 2, STEPS["plain"], False)
        # peers read the wire copy, not the fp32 gradient: without barriers those reads race with the owner's copy
        assert any(r.startswith("('model'") for r in races) and any(r.startswith("('wire'") for r in races), races[:5]
        races = run(monkeypatch, 2, 2, STEPS["plain"], False, wire=False)
        assert any(r.startswith("('model'") for r in races) and any(r.startswith("('grad'") for r in races), races[:5]
    else:
        monkeypatch.setattr(zp.FakeStream, "wait_event", lambda self, ev: None)
        races = run(monkeypatch, 2, 2, STEPS["plain"], True)
        assert any(r.startswith("('grad'") for r in races), races[:5]
