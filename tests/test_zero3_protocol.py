"""Race check of the peer-access full-sharding protocol, on the host, without a GPU.

``P2PFullShardComm`` orders its kernels with stream order, events between the main and the side stream, flag barriers
between ranks and (once per step) an NCCL rendezvous. A mistake in that ordering would show on a GPU only as a rare
wrong gradient. Here the REAL communicator and engine run on CPU tensors while ``torch.cuda`` streams / events, the
process group, symmetric memory and the kernel library are replaced by recorders; every rank's run yields a trace of
operations (stream, event waits, barrier epochs, what memory each kernel reads and writes - including the peers').
The traces are joined into one happens-before graph (stream order, event record -> wait, "every rank has arrived"
-> "barrier / collective completes") and every pair of conflicting accesses to the same buffer - a peer's pull of a
weight piece against the optimizer's write, a peer's read of a gradient buffer against the next layer's weight-gradient
kernels, a gather into a rotating buffer against the compute that still reads it - must be ordered by the graph.

The compute of a unit is entered as a window (a marker when it starts, one when the next hook fires) that reads the
unit's gathered weights and, in backward, writes its gradient buffer.
"""
import contextlib

import pytest
import torch
import torch.distributed as dist

from llm_distillery_b200.engine.trainer import DistillEngine, synthetic_batch
from llm_distillery_b200.models.llama import LlamaConfig, build_model
from llm_distillery_b200.ops import _lib
from llm_distillery_b200.parallel import fsdp, p2p

SIM = None          # the recorder of the rank whose schedule is being traced


class Sim:
    def __init__(self, rank: int, world: int):
        self.rank, self.world = rank, world
        self.ops: list[dict] = []
        self.last = {"M": None, "S": None}
        self.cur = "M"
        self.unit = None
        self.window = None
        self.ncoll = {"nccl": 0, "host": 0}
        self.nsym = 0

    def add(self, kind, stream=None, reads=(), writes=(), deps=(), coll=None, phase=None) -> int:
        stream = stream or self.cur
        d = [x for x in deps if x is not None]
        if self.last[stream] is not None:
            d.append(self.last[stream])
        op = {"i": len(self.ops), "rank": self.rank, "stream": stream, "kind": kind, "reads": set(reads),
              "writes": set(writes), "deps": d, "coll": coll, "phase": phase}
        self.ops.append(op)
        self.last[stream] = op["i"]
        return op["i"]

    def collective(self, key, stream=None) -> None:
        """Two nodes: arrival (ordered after this stream's past) and completion (after EVERY rank's arrival)."""
        self.add("arrive", stream, coll=key, phase="arrive")
        self.add("complete", stream, coll=key, phase="complete")

    # ---- compute windows on the main stream
    def begin_window(self, reads, writes) -> None:
        self.window = (set(reads), set(writes))
        self.add("compute-begin", "M", reads, writes)

    def end_window(self) -> None:
        if self.window is not None:
            self.add("compute-end", "M", *self.window)
            self.window = None


# ------------------------------------------------------------------------------------------------ recorders
class FakeEvent:
    def __init__(self, *a, **k):
        self.after = None

    def record(self, stream=None):
        self.after = SIM.last[stream.name if stream is not None else SIM.cur]


class FakeStream:
    def __init__(self, name="S", **k):
        self.name = name if isinstance(name, str) else "S"
        self.cuda_stream = 0

    def wait_event(self, ev):
        SIM.add("wait", self.name, deps=[ev.after])

    def wait_stream(self, other):
        SIM.add("wait", self.name, deps=[SIM.last[other.name]])

    def synchronize(self):
        pass


@contextlib.contextmanager
def fake_stream_ctx(s):
    prev, SIM.cur = SIM.cur, s.name
    try:
        yield
    finally:
        SIM.cur = prev


class FakeSym:
    def __init__(self, numel, dtype, device, group=None):
        self.tensor = torch.zeros(numel, dtype=dtype)
        SIM.nsym += 1                       # allocation order is the same on every rank: the count names the buffer
        self.ptrs, self.c_ptrs = [], ("sym", SIM.nsym)


def _weights_obj(rank, u):
    return ("W", rank, u.slot) if u.is_layer else ("Wd", rank, u.name)


def _grads_obj(rank, u):
    return ("G", rank, u.slot) if u.is_layer else ("Gd", rank, u.name)


class FakeKernels:
    """Stands in for the kernel library: every launcher records what its kernel touches, on the current stream."""

    def b200_p2p_barrier(self, sig, rank, world, epoch, stream):
        SIM.collective(("flag", sig, int(epoch)))          # flag words of one symmetric buffer, one epoch
        return 0

    def b200_p2p_gather_pull(self, src, dst, off, nbytes, rank, world, stream):
        u = SIM.unit
        SIM.add("gather", reads={("shard", r, u.index) for r in range(world)}, writes={_weights_obj(rank, u)})
        return 0

    def b200_p2p_reduce_scatter_acc_f32(self, src, out, lo, n, rank, world, accumulate, stream):
        u = SIM.unit
        SIM.add("reduce", reads={_grads_obj(r, u) for r in range(world)}, writes={("gshard", rank, u.index)})
        return 0

    def b200_p2p_rs_adamw_piece(self, src, lo, acc, model, master, m, v, n, rank, world, *rest):
        u = SIM.unit
        SIM.add("reduce+adamw", reads={_grads_obj(r, u) for r in range(world)} | {("gshard", rank, u.index)},
                writes={("shard", rank, u.index), ("state", rank, u.index)})
        return 0

    def __getattr__(self, name):      # any other launcher: not part of this protocol
        raise AttributeError(name)


class Traced(fsdp.P2PFullShardComm):
    """The real communicator; only adds the compute windows and tells the recorder which unit a kernel works on."""
    fuse = True

    def _embed_unit(self):
        return next((u for u in self.flat.units if u.name == "embed"), None)

    def _pre(self, param, backward=False):
        SIM.end_window()
        super()._pre(param, backward)
        u = self.flat.unit_of.get(id(param))
        if u is None:
            return
        writes = set()
        if backward and u.is_layer:
            writes.add(_grads_obj(self.rank, u))
        if not backward and u.name == "head" and torch.is_grad_enabled():
            # this window runs on through the loss head's forward and backward, up to the last layer's backward
            writes.add(_grads_obj(self.rank, u))
            emb = self._embed_unit()
            if emb is not None:
                writes.add(_grads_obj(self.rank, emb))       # tied LM head: its gradient lands in the embedding's buffer
        SIM.begin_window({_weights_obj(self.rank, u)}, writes)

    def _layer_done(self, first_param):
        SIM.end_window()
        super()._layer_done(first_param)
        u = self.flat.unit_of.get(id(first_param))
        first_layer = next(x for x in self.flat.units if x.is_layer)
        emb = self._embed_unit()
        if u is first_layer and emb is not None:             # what follows the first layer's backward: embedding gradient
            SIM.begin_window(set(), {_grads_obj(self.rank, emb)})

    def idle_micro_step(self):
        super().idle_micro_step()
        SIM.end_window()

    def reduce_and_step(self, lr, grad_scale):
        SIM.end_window()
        super().reduce_and_step(lr, grad_scale)

    def _reduce_unit(self, u):
        SIM.end_window()      # a rank without a batch gets here without a layer-done hook; its zero fill ends with this
        super()._reduce_unit(u)

    def _gather_unit(self, u):
        SIM.unit = u
        super()._gather_unit(u)

    def _reduce_op(self, u):
        SIM.unit = u
        super()._reduce_op(u)

    def last_micro_batch(self, lr, grad_scale):
        if self.fuse and self._fused is None:                # the real check also wants bf16 weights; the schedule is the same
            self.opt.step_count += 1
            self._fused = {"lr": float(lr), "gs": float(grad_scale) / self.world}


@pytest.fixture
def recorders(monkeypatch):
    monkeypatch.setattr(torch.cuda, "Event", FakeEvent)
    monkeypatch.setattr(torch.cuda, "Stream", FakeStream)
    monkeypatch.setattr(torch.cuda, "stream", fake_stream_ctx)
    monkeypatch.setattr(torch.cuda, "current_stream", lambda *a, **k: FakeStream(SIM.cur))
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    monkeypatch.setattr(dist, "get_rank", lambda group=None: SIM.rank)
    monkeypatch.setattr(dist, "get_world_size", lambda group=None: SIM.world)
    monkeypatch.setattr(dist, "get_backend", lambda group=None: "nccl")

    def host_barrier(group=None, **k):
        SIM.ncoll["host"] += 1
        SIM.collective(("host", SIM.ncoll["host"]), "M")

    def all_reduce(t, op=None, group=None, **k):
        SIM.ncoll["nccl"] += 1
        SIM.collective(("nccl", SIM.ncoll["nccl"]))
    monkeypatch.setattr(dist, "barrier", host_barrier)
    monkeypatch.setattr(dist, "all_reduce", all_reduce)
    monkeypatch.setattr(p2p, "SymmetricBuffer", FakeSym)
    monkeypatch.setattr(_lib, "kernels", lambda: FakeKernels())
    monkeypatch.setattr(_lib, "stream", lambda: None)
    monkeypatch.setattr(_lib, "ptr", lambda t: 0)
    monkeypatch.setattr(_lib, "register", lambda *a, **k: None)
    monkeypatch.setattr(_lib, "take_device_error", lambda: 0)
    yield
    global SIM
    SIM = None


def trace_rank(rank, world, layers, tied, steps, fuse):
    """Runs one rank's whole schedule. ``steps``: a list of steps, each a list of micro-batch kinds - "train",
    "idle:<rank>" (that rank has no batch), "eval" (a validation pass under no_grad)."""
    global SIM
    SIM = Sim(rank, world)
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=layers,
                      num_attention_heads=2, num_key_value_heads=1, max_position_embeddings=32, tie_word_embeddings=tied)
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=1)
    comm = Traced("cpu")
    comm.fuse = fuse
    comm.cuda, comm.side = True, FakeStream("S")
    accum = max(sum(1 for k in st if k != "eval") for st in steps)
    eng = DistillEngine(model, loss="kl", temperature=1.0, optimizer="adamw", lr=1e-3, grad_accum=accum, comm=comm)
    real_step = eng.opt.step
    units = comm.flat.units

    def traced_step(lr=None, grad_scale=1.0, grad=None):
        SIM.add("optimizer", "M", reads={("gshard", rank, u.index) for u in units},
                writes={("shard", rank, u.index) for u in units} | {("state", rank, u.index) for u in units})
        return real_step(lr, grad_scale, grad)
    eng.opt.step = traced_step
    hb = synthetic_batch(cfg.vocab_size, 1, 16, 4, seed=rank)
    for st in steps:
        micro = [k for k in st if k != "eval"]
        seen = 0
        for kind in st:
            if kind == "eval":
                eng.eval_batch(hb)
                SIM.end_window()
                continue
            seen += 1
            last = seen == len(micro)
            if kind == f"idle:{rank}":
                eng.idle_micro_step(last=last)
            else:
                eng.micro_step(hb.to_device("cpu"), last=last)
        eng.optimizer_step()
    SIM.end_window()
    comm.close()
    return SIM.ops


# ------------------------------------------------------------------------------------------------ the checker
def find_races(traces: list[list[dict]]) -> list[str]:
    """Joins the ranks' traces into one happens-before graph and returns a description of every pair of conflicting
    accesses (same buffer, at least one write) that the graph leaves unordered."""
    gid, nodes = {}, []
    for ops in traces:
        for op in ops:
            gid[(op["rank"], op["i"])] = len(nodes)
            nodes.append(op)
    preds = [set() for _ in nodes]
    for n, op in enumerate(nodes):
        for d in op["deps"]:
            preds[n].add(gid[(op["rank"], d)])
    arrive, complete = {}, {}
    for n, op in enumerate(nodes):
        if op["coll"] is not None:
            (arrive if op["phase"] == "arrive" else complete).setdefault(op["coll"], []).append(n)
    world = len(traces)
    for key, arr in arrive.items():
        # the protocol is symmetric: every rank takes part in every barrier / collective, exactly once
        assert len(arr) == world and len(complete[key]) == world, (key, len(arr), len(complete[key]))
        for c in complete[key]:
            preds[c].update(arr)
    # ancestors as bit sets, in topological order
    succs = [[] for _ in nodes]
    indeg = [len(p) for p in preds]
    for n, ps in enumerate(preds):
        for q in ps:
            succs[q].append(n)
    order = [n for n, d in enumerate(indeg) if d == 0]
    anc = [0] * len(nodes)
    k = 0
    while k < len(order):
        n = order[k]
        k += 1
        for m in succs[n]:
            anc[m] |= anc[n] | (1 << n)
            indeg[m] -= 1
            if indeg[m] == 0:
                order.append(m)
    assert len(order) == len(nodes), "the happens-before graph has a cycle"
    by_obj = {}
    for n, op in enumerate(nodes):
        for o in op["reads"]:
            by_obj.setdefault(o, []).append((n, False))
        for o in op["writes"]:
            by_obj.setdefault(o, []).append((n, True))
    races = []
    for obj, acc in by_obj.items():
        for x in range(len(acc)):
            a, aw = acc[x]
            for y in range(x + 1, len(acc)):
                b, bw = acc[y]
                if a == b or not (aw or bw):
                    continue
                if not ((anc[b] >> a) & 1 or (anc[a] >> b) & 1):
                    A, B = nodes[a], nodes[b]
                    races.append(f"{obj}: rank {A['rank']} {A['stream']} {A['kind']}#{A['i']} ({'W' if aw else 'R'}) || "
                                 f"rank {B['rank']} {B['stream']} {B['kind']}#{B['i']} ({'W' if bw else 'R'})")
    return races


def run(world, layers, tied, steps, fuse):
    traces = [trace_rank(r, world, layers, tied, steps, fuse) for r in range(world)]
    kinds = {op["kind"] for t in traces for op in t}
    assert {"gather", "arrive", "compute-begin"} <= kinds and (("reduce+adamw" in kinds) == fuse or not fuse)
    return find_races(traces)


SCHEDULES = {
    "one micro-batch per step": [["train"], ["train"], ["train"]],
    "accumulation of two": [["train", "train"], ["train", "train"]],
    "validation between steps and inside an accumulation": [["train"], ["eval", "train", "eval", "train"], ["eval"], ["train"]],
    "a rank without a batch, last and not last": [["train", "idle:1"], ["idle:1", "train"], ["train", "train"]],
}


@pytest.mark.parametrize("fuse", [True, False], ids=["fused", "unfused"])
@pytest.mark.parametrize("layers,tied", [(2, False), (3, False), (3, True), (1, False)])
@pytest.mark.parametrize("name", list(SCHEDULES))
def test_no_unordered_conflicting_accesses(recorders, name, layers, tied, fuse):
    races = run(2, layers, tied, SCHEDULES[name], fuse)
    assert not races, f"{len(races)} unordered pairs, e.g.\n" + "\n".join(races[:8])


def test_three_ranks(recorders):
    assert not run(3, 3, False, SCHEDULES["accumulation of two"], True)


def test_the_checker_sees_a_missing_barrier(recorders, monkeypatch):
    """Without the barrier that protects a gradient buffer read by the latest reduction, the next backward's writes
    into that buffer race with the peers' reads: the checker must say so."""
    monkeypatch.setattr(Traced, "_before_backward_writes",
                        lambda self, u: fsdp.FullShardComm._before_backward_writes(self, u))
    races = run(2, 3, False, SCHEDULES["accumulation of two"], False)
    assert any(r.startswith("('G'") for r in races), races[:5]


MUTATIONS = {
    # what is taken out of the protocol -> the buffer kind on which the checker must then find a race
    "no barrier after the optimizer step": ("_step_end", lambda self: None, "shard"),
    "no wait for the previous owner's reduction": ("_before_backward_writes", lambda self, u: None, "G"),
    "compute does not wait for its gather": ("_wait_ready", lambda self, u: None, "W"),
    "side stream does not wait for the main stream": ("_on_side", lambda self: fake_stream_ctx(self.side), "G"),
}


@pytest.mark.parametrize("name", list(MUTATIONS))
def test_the_checker_sees_each_removed_ordering(recorders, monkeypatch, name):
    attr, repl, kind = MUTATIONS[name]
    monkeypatch.setattr(Traced, attr, repl)
    races = run(2, 3, False, SCHEDULES["accumulation of two"], True)
    assert any(r.startswith(f"('{kind}'") for r in races), (name, races[:5])
