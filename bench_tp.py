#!/usr/bin/env python
"""Multi-GPU benchmarks of the tensor-parallel path (one rank per GPU, launched by torch.distributed.run):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        bench_tp.py gemms   [--tokens 8192] [--model llama-3-70b] [--iters 10]
        bench_tp.py collect [--model llama-3-70b] [--seq 8192] [--batch 1] [--topk 128] [--steps 3] [--layers N]
        bench_tp.py p2p     [--iters 10]
        bench_tp.py head    [--rows 32768] [--hidden 4096] [--vocab 128256] [--topk 200] [--iters 10]
        bench_tp.py zero3   [--iters 10]

gemms    the four linear layers of one decoder block at tensor-parallel width N: fused all-gather->GEMM and
         GEMM->reduce-scatter kernels against NCCL all_gather / reduce_scatter + torch.matmul (cuBLAS), with the
         roofline  max(FLOPs / measured bf16 peak, bytes over NVLink / 770 GB/s per direction).
collect  teacher collection throughput (tokens/s) of the tensor-parallel forward + vocabulary-parallel top-K,
         random-init weights, synthetic token ids (``--layers`` below the model's depth is a smoke run, flagged in the
         output and not a benchmark number).
head     the fused vocabulary-parallel LM head + distillation loss (forward and backward) over N vocabulary slices
         against cuBLAS + PyTorch ops + NCCL all-reduce, KL and JSD at T = 1 and 2.
zero3    the kernels of full parameter sharding on one decoder layer of TinyLlama-1.1B and Llama-3-8B: pull gather,
         reduce-scatter-accumulate and reduce-scatter + AdamW, against NCCL all_gather / reduce_scatter.
p2p      peer-to-peer all-reduce (reduce-scatter + all-gather kernels) against NCCL all_reduce, bus bandwidth.

Timing: CUDA events on the launching stream after warm-up, a barrier before each timed call, median per rank, MAX
over ranks. Inputs of the GEMM cases are far larger than L2. One JSON line per case from rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from llm_distillery_b200.models.llama import preset  # noqa: E402
from llm_distillery_b200.ops import _lib  # noqa: E402
from llm_distillery_b200.parallel.tp import TPGroup, TPLlama, padded_seq_len  # noqa: E402

NVLINK_GBS = 770.0   # measured peer copy bandwidth per direction on this pool


def peak_tflops() -> tuple[float, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


def timed_max(fn, iters: int, warmup: int = 3) -> float:
    """Median ms per call on this rank, then the maximum over ranks."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def emit(rank: int, **kw) -> None:
    err = _lib.take_device_error()
    if err:
        kw["device_error"] = err
    if rank == 0:
        print(json.dumps(kw), flush=True)


def bench_gemms(args, dev, rank, world) -> None:
    cfg = preset(args.model)
    T, h = args.tokens, cfg.hidden_size
    d, H, Hkv, f = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
    Ts = T // world
    grp = TPGroup(dev, T, h)
    pk, src = peak_tflops()
    gen = torch.Generator(device=dev).manual_seed(rank)

    def rnd(*shape):
        return (torch.randn(shape, device=dev, generator=gen) * 0.05).to(torch.bfloat16)

    link_bytes = T * h * 2 * (world - 1) / world      # what one rank must receive (AG) or send (RS)
    for name, n_local in (("qkv", (H + 2 * Hkv) * d // world), ("gate_up", 2 * f // world)):
        w = rnd(n_local, h)
        x_shard = rnd(Ts, h)
        full = torch.empty((T, h), dtype=torch.bfloat16, device=dev)

        def fused():
            grp.slab(T, h).copy_(x_shard)
            return grp.ag_gemm(w, T)

        def copy_only():
            grp.slab(T, h).copy_(x_shard)

        def nccl():
            dist.all_gather_into_tensor(full, x_shard)
            return full @ w.t()

        ms_f = timed_max(fused, args.iters) - timed_max(copy_only, args.iters)
        ms_n = timed_max(nccl, args.iters)
        flops = 2.0 * T * n_local * h
        ideal = max(flops / (pk * 1e9), link_bytes / (NVLINK_GBS * 1e6))
        emit(rank, case=f"ag_gemm {name}", tp=world, shape=[T, n_local, h], ms_fused=round(ms_f, 4), ms_nccl_cublas=round(ms_n, 4),
             speedup=round(ms_n / ms_f, 3), tflops=round(flops / ms_f / 1e9, 1), roofline_ms=round(ideal, 4),
             frac_of_roofline=round(ideal / ms_f, 3), roofline=f"max(FLOPs/{pk} TF/s of {src}, bytes/{NVLINK_GBS} GB/s)")
    for name, k_local in (("o_proj", H * d // world), ("down", f // world)):
        w = rnd(h, k_local)
        x = rnd(T, k_local)
        res = rnd(Ts, h)
        out = torch.empty((Ts, h), dtype=torch.bfloat16, device=dev)

        def fused():
            return grp.gemm_rs(x, w, residual=res)

        def nccl():
            y = x @ w.t()
            dist.reduce_scatter_tensor(out, y)
            return out.add_(res)

        ms_f = timed_max(fused, args.iters)
        ms_n = timed_max(nccl, args.iters)
        flops = 2.0 * T * h * k_local
        ideal = max(flops / (pk * 1e9), link_bytes / (NVLINK_GBS * 1e6))
        emit(rank, case=f"gemm_rs {name}", tp=world, shape=[T, h, k_local], ms_fused=round(ms_f, 4), ms_nccl_cublas=round(ms_n, 4),
             speedup=round(ms_n / ms_f, 3), tflops=round(flops / ms_f / 1e9, 1), roofline_ms=round(ideal, 4),
             frac_of_roofline=round(ideal / ms_f, 3), roofline=f"max(FLOPs/{pk} TF/s of {src}, bytes/{NVLINK_GBS} GB/s)")


def bench_collect_replicas(args, dev, rank, world, cfg, full_depth) -> None:
    """Every rank holds the WHOLE teacher and collects its own batches (what ``tp_size = 0`` picks when the model fits
    one GPU: a 70 B teacher in bf16 is 131 GiB of 180 GB): no communication, aggregate = sum over the ranks."""
    import numpy as np
    from llm_distillery_b200.collect.collector import TeacherCollector
    from llm_distillery_b200.models.llama import build_model
    B, L = args.batch, args.seq
    model = build_model(cfg, dtype=torch.bfloat16, device=dev, seed=None)
    model.init_weights(seed=rank)
    collector = TeacherCollector(model, topk=args.topk, crop_to_size=cfg.vocab_size, enable_topk=True)

    class _Convo:      # every position of every sequence is a content row
        length = L

        @staticmethod
        def content_indices():
            return np.arange(L, dtype=np.int64)
    convos = [_Convo() for _ in range(B)]
    toks = np.random.default_rng(rank).integers(0, cfg.vocab_size, (B, L)).astype(np.int64)

    def step():
        with torch.no_grad():
            collector.fetch(collector.submit(toks, convos))     # rows in pinned host memory when this returns

    n0 = _lib.LAUNCH_COUNT[0]
    ms = timed_max(step, args.steps, warmup=max(1, args.warmup))
    launches = (_lib.LAUNCH_COUNT[0] - n0) // (args.steps + max(1, args.warmup))
    toks_all = B * L * world
    emit(rank, metric="teacher collect tokens/s", value=round(toks_all / ms * 1e3, 1), unit="tokens/s", n_gpus=world,
         ms_per_step=round(ms, 3), dtype="bf16", data="synthetic token ids, random-init weights",
         config={"model": args.model, "layers": cfg.num_hidden_layers, "parallelism": f"{world} replicas (tp1)",
                 "batch_per_gpu": B, "seq_len": L, "topk": args.topk,
                 "peak_mem_gb": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 1)},
         smoke_only=bool(cfg.num_hidden_layers != full_depth), gpu_launches_per_step=int(launches),
         fwd_tflops_per_gpu=round(cfg.flops_per_token_fwd(L) * B * L / ms / 1e9, 1))


def bench_collect(args, dev, rank, world) -> None:
    over = {"num_hidden_layers": args.layers} if args.layers else {}
    cfg = preset(args.model, **over)
    full_depth = preset(args.model).num_hidden_layers
    if args.replicas:
        return bench_collect_replicas(args, dev, rank, world, cfg, full_depth)
    B = args.batch
    L = padded_seq_len(B, args.seq, world)
    grp = TPGroup(dev, B * L, cfg.hidden_size, topk=args.topk)
    model = TPLlama.random_init(cfg, grp, seed=0)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (B, L), generator=g)
    pin = ids.pin_memory()
    host_lp = torch.empty((B * L, args.topk), dtype=torch.float16).pin_memory()
    host_ix = torch.empty((B * L, args.topk), dtype=torch.int32).pin_memory()

    def step():
        dev_ids = pin.to(dev, non_blocking=True)
        lp, ix = model.topk_logprobs(dev_ids, args.topk)
        if rank == 0:   # the writer rank takes the rows to pinned host memory, as the collector does
            host_lp.copy_(lp, non_blocking=True)
            host_ix.copy_(ix, non_blocking=True)

    n0 = _lib.LAUNCH_COUNT[0]
    ms = timed_max(step, args.steps, warmup=max(1, args.warmup))
    launches = (_lib.LAUNCH_COUNT[0] - n0) // (args.steps + max(1, args.warmup))
    toks = B * L
    emit(rank, metric="teacher collect tokens/s", value=round(toks / ms * 1e3, 1), unit="tokens/s", n_gpus=world,
         ms_per_step=round(ms, 3), dtype="bf16", data="synthetic token ids, random-init weights",
         config={"model": args.model, "layers": cfg.num_hidden_layers, "parallelism": f"tp{world}", "batch": B,
                 "seq_len": L, "topk": args.topk},
         smoke_only=bool(cfg.num_hidden_layers != full_depth), gpu_launches_per_step=int(launches),
         fwd_tflops_per_gpu=round(cfg.flops_per_token_fwd(L) * toks / ms / 1e9 / world, 1))


def bench_head(args, dev, rank, world) -> None:
    """Fused vocabulary-parallel loss head (forward + backward) against the unfused library path: cuBLAS logits of
    the slice, fp32 softmax statistics with NCCL all-reduces, the loss in PyTorch ops, autograd backward, NCCL
    all-reduce of dH."""
    from llm_distillery_b200.loss import divergence as dv
    from llm_distillery_b200.loss.head import sort_teacher_rows
    from llm_distillery_b200.parallel.vp_head import VocabParallelHead
    M, h, V, K = args.rows, args.hidden, args.vocab, args.topk
    g = torch.Generator(device=dev).manual_seed(5)          # same stream on every rank: replicated inputs
    Hc = (torch.randn((M, h), device=dev, generator=g) * 0.5).to(torch.bfloat16)
    ids = torch.randint(0, V, (M, K), device=dev, generator=g, dtype=torch.int32)
    u = torch.log_softmax(torch.randn((M, K), device=dev, generator=g) * 2, -1)
    ids, u = sort_teacher_rows(ids, u)
    grp = TPGroup(dev, M, h)
    head = VocabParallelHead(grp, M, h, K, V)
    gw = torch.Generator(device=dev).manual_seed(100 + rank)
    Ws = (torch.randn((head.vl, h), device=dev, generator=gw) * 0.02).to(torch.bfloat16)
    dW = torch.zeros((head.vl, h), dtype=torch.float32, device=dev)
    pk, src = peak_tflops()
    for kind in ("kl", "jsd"):
        for T in (1.0, 2.0):
            def fused():
                return head.loss_and_grads(Hc, Ws, ids, u, kind, T, dW=dW)

            def unfused():
                Hr = Hc.detach().requires_grad_(True)
                Wr = Ws.detach().requires_grad_(True)
                z = (Hr @ Wr.t()).float() / T
                m = z.detach().max(-1).values
                dist.all_reduce(m, op=dist.ReduceOp.MAX)
                se = torch.exp(z - m[:, None]).sum(-1)
                se_all = se.detach().clone()
                dist.all_reduce(se_all)
                lse = m + torch.log(se + (se_all - se.detach()))
                local = ids.long() - head.lo
                inside = (local >= 0) & (local < head.valid)
                zk_part = torch.where(inside, torch.gather(z, 1, local.clamp(0, head.valid - 1)), torch.zeros((), device=dev))
                zk_all = zk_part.detach().clone()
                dist.all_reduce(zk_all)
                zk = zk_part + (zk_all - zk_part.detach())
                s, t = dv.student_teacher_logprobs(lse, zk, u, ids.long() < V, T)
                rows = dv.loss_rows(kind, s, t)
                rows.mean().backward()
                dist.all_reduce(Hr.grad)
                return rows

            ms_f = timed_max(fused, args.iters)
            ms_u = timed_max(unfused, max(3, args.iters // 2))
            flops = 4 * 2.0 * M * head.vl * h       # pass 1, pass 2, dgrad, wgrad on the slice
            link = M * h * 2 * (world - 1) / world * 2 + (world - 1) * M * K * 4
            ideal = max(flops / (pk * 1e9), link / (NVLINK_GBS * 1e6))
            emit(rank, case=f"vocab-parallel head {kind} T={T}", tp=world, shape=[M, h, V, K], ms_fused=round(ms_f, 3),
                 ms_unfused=round(ms_u, 3), speedup=round(ms_u / ms_f, 2), tflops_per_gpu=round(flops / ms_f / 1e9, 1),
                 roofline_ms=round(ideal, 3), frac_of_roofline=round(ideal / ms_f, 3),
                 roofline=f"max(4 GEMMs/{pk} TF/s of {src}, link bytes/{NVLINK_GBS} GB/s)")


def bench_p2p(args, dev, rank, world) -> None:
    from llm_distillery_b200.parallel.p2p import P2PComm, SymmetricBuffer
    comm = P2PComm(dev)
    for mib in (1, 16, 128, 1024):
        n = mib * (1 << 20) // 4
        buf = SymmetricBuffer(n, torch.float32, dev)
        ref = torch.zeros(n, dtype=torch.float32, device=dev)
        ms_p = timed_max(lambda: comm.allreduce_(buf, 1.0 / world), args.iters)
        ms_n = timed_max(lambda: dist.all_reduce(ref), args.iters)
        bus = lambda ms: 2.0 * (world - 1) / world * n * 4 / ms / 1e6
        emit(rank, case="allreduce fp32", mib=mib, tp=world, ms_p2p=round(ms_p, 4), ms_nccl=round(ms_n, 4),
             busbw_p2p_gbs=round(bus(ms_p), 1), busbw_nccl_gbs=round(bus(ms_n), 1))
        del buf


def bench_dpstep(args, dev, rank, world) -> None:
    """The pieces of the data-parallel optimizer step on a flat parameter space of ``--params`` elements (default: the
    1.1 B of TinyLlama): bf16 wire cast, the fused reduce-scatter + AdamW + all-gather kernel in its three gradient
    modes, and reduce-scatter / all-gather alone. Every timed call is bracketed by the flag barriers of a real step."""
    from llm_distillery_b200.parallel.p2p import P2PComm, SymmetricBuffer
    comm = P2PComm(dev)
    n = (int(args.params) // (256 * world)) * (256 * world)
    per = n // world
    lo = rank * per
    grad = SymmetricBuffer(n, torch.float32, dev)
    wire = SymmetricBuffer(n, torch.bfloat16, dev)
    model = SymmetricBuffer(n, torch.bfloat16, dev)
    grad.tensor.normal_(0, 1e-3)
    master = torch.zeros(per, dtype=torch.float32, device=dev)
    m = torch.zeros_like(master)
    v = torch.zeros_like(master)
    reduced = torch.zeros_like(master)
    shard16 = torch.zeros(per, dtype=torch.bfloat16, device=dev)
    K = _lib.kernels()
    st = _lib.stream

    def cast():
        for a, b in ((0, lo), (lo + per, n)):
            if b > a:
                _lib.check(K.b200_p2p_cast_wire(_lib.ptr(grad.tensor), _lib.ptr(wire.tensor), a, b - a, st()), "cast")

    def fused(mode):
        def run():
            comm.barrier()
            src = wire.c_ptrs if mode == 1 else grad.c_ptrs
            own = _lib.ptr(grad.tensor) if mode == 1 else (_lib.ptr(reduced) if mode == 2 else None)
            _lib.check(K.b200_p2p_rs_adamw_ag(src, own, mode, model.c_ptrs, _lib.ptr(master), _lib.ptr(m), _lib.ptr(v), lo,
                                              per, 0, rank, world, 1e-5, 0.9, 0.99, 1e-8, 0.0, 1, 1.0 / world, 1, 0, st()),
                       "fused")
            comm.barrier()
        return run

    def rs_only():
        comm.barrier()
        comm.reduce_scatter(grad, reduced, lo, 1.0)
        comm.barrier()

    def ag_only():
        comm.barrier()
        comm.allgather(model, shard16, lo, skip_self=True)
        comm.barrier()

    def two_barriers():
        comm.barrier()
        comm.barrier()

    gb = lambda b, ms: round(b / ms / 1e6, 1)
    inbound16, inbound32 = (world - 1) * per * 2, (world - 1) * per * 4
    for name, fn, note in (
            ("two flag barriers", two_barriers, {}),
            ("bf16 wire cast", cast, {"hbm_gbs": None}),
            ("fused, bf16 wire", fused(1), {"nvlink_in_gbs": inbound16, "nvlink_out_gbs": inbound16}),
            ("fused, fp32 wire", fused(0), {"nvlink_in_gbs": inbound32, "nvlink_out_gbs": inbound16}),
            ("fused, gradient already summed (AdamW + all-gather)", fused(2), {"nvlink_out_gbs": inbound16}),
            ("reduce-scatter alone, fp32", rs_only, {"nvlink_in_gbs": inbound32}),
            ("all-gather alone, bf16", ag_only, {"nvlink_out_gbs": inbound16})):
        ms = timed_max(fn, args.iters)
        extra = {k: (gb(b, ms) if b else None) for k, b in note.items()}
        emit(rank, case=name, world=world, params=n, ms=round(ms, 4), **extra)


def bench_zero3(args, dev, rank, world) -> None:
    """The three kernels of full parameter sharding on one decoder layer's worth of parameters, against the NCCL
    collectives they replace: pull gather (bf16), reduce-scatter-accumulate (fp32), reduce-scatter + AdamW (fp32)."""
    import ctypes
    from llm_distillery_b200.ops._lib import _VP, _I, _LL
    from llm_distillery_b200.parallel.p2p import P2PComm, SymmetricBuffer
    _F = ctypes.c_float
    _lib.register("b200_p2p_gather_pull", [_VP, _VP, _LL, _LL, _I, _I, _VP])
    _lib.register("b200_p2p_reduce_scatter_acc_f32", [_VP, _VP, _LL, _LL, _I, _I, _I, _VP])
    _lib.register("b200_p2p_rs_adamw_piece", [_VP, _LL, _VP, _VP, _VP, _VP, _VP, _LL, _I, _I, _F, _F, _F, _F, _F, _I, _F,
                                              _I, _VP])
    lib = _lib.kernels()
    comm = P2PComm(dev)
    for name in ("tinyllama-1.1b", "llama-3-8b"):
        c = preset(name)
        per_layer = (c.q_size + 2 * c.kv_size) * c.hidden_size + c.hidden_size * c.q_size + 3 * c.hidden_size * c.intermediate_size
        numel = (per_layer + 256 * world - 1) // (256 * world) * (256 * world)
        piece = numel // world
        shard = SymmetricBuffer(piece, torch.bfloat16, dev)
        grads = SymmetricBuffer(numel, torch.float32, dev)
        full = torch.empty(numel, dtype=torch.bfloat16, device=dev)
        out = torch.zeros(piece, dtype=torch.float32, device=dev)
        master, m, v = (torch.zeros(piece, dtype=torch.float32, device=dev) for _ in range(3))
        gfull = torch.zeros(numel, dtype=torch.float32, device=dev)

        def pull():
            _lib.check(lib.b200_p2p_gather_pull(shard.c_ptrs, _lib.ptr(full), 0, piece * 2, rank, world, _lib.stream()), "pull")

        def rs_acc():
            comm.barrier()
            _lib.check(lib.b200_p2p_reduce_scatter_acc_f32(grads.c_ptrs, _lib.ptr(out), rank * piece, piece, rank, world, 1,
                                                           _lib.stream()), "rs")

        def rs_adam():
            comm.barrier()
            _lib.check(lib.b200_p2p_rs_adamw_piece(grads.c_ptrs, rank * piece, None, _lib.ptr(shard.tensor), _lib.ptr(master),
                                                   _lib.ptr(m), _lib.ptr(v), piece, rank, world, 1e-5, 0.9, 0.99, 1e-8, 2e-8,
                                                   1, 1.0 / world, 1, _lib.stream()), "rs_adamw")

        def nccl_ag():
            dist.all_gather_into_tensor(full, shard.tensor)

        def nccl_rs():
            dist.reduce_scatter_tensor(out, gfull)

        ms = {k: timed_max(f, args.iters) for k, f in (("pull", pull), ("nccl_ag", nccl_ag), ("rs_acc", rs_acc),
                                                       ("nccl_rs", nccl_rs), ("rs_adamw", rs_adam))}
        link = (world - 1) / world          # share of the bytes that crosses NVLink
        emit(rank, case="zero3 layer kernels", model=name, world=world, layer_params=numel,
             ms={k: round(x, 4) for k, x in ms.items()},
             gather_in_gbs=round(numel * 2 * link / ms["pull"] / 1e6, 1) if world > 1 else None,
             gather_write_gbs=round(numel * 2 / ms["pull"] / 1e6, 1),
             rs_in_gbs=round(piece * 4 * (world - 1) / ms["rs_acc"] / 1e6, 1) if world > 1 else None,
             rs_adamw_hbm_gbs=round(piece * (4 * world + 24 + 2) / ms["rs_adamw"] / 1e6, 1))
        del shard, grads, full, out, master, m, v, gfull
    comm.check()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("cmd", choices=["gemms", "collect", "p2p", "head", "zero3", "dpstep"])
    ap.add_argument("--params", type=float, default=1.1e9, help="dpstep: elements of the flat parameter space")
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--model", default="llama-3-70b")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--topk", type=int, default=128)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--replicas", action="store_true",
                    help="collect: every rank holds the whole teacher (no tensor parallelism), aggregate over the ranks")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    {"gemms": bench_gemms, "collect": bench_collect, "p2p": bench_p2p, "head": bench_head,
     "zero3": bench_zero3, "dpstep": bench_dpstep}[args.cmd](args, dev, rank, world)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
