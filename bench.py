#!/usr/bin/env python
"""Headline benchmark: distilled-student training throughput (tokens/s) on the TinyLlama-1.1B self-distillation
configuration - seq 2048, micro-batch 8 per GPU, teacher top-200 targets, forward KL at T = 2, AdamW, data-parallel
over N GPUs of one node (weak scaling) - on synthetic token data and random-init weights.

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Prints ONE JSON line from rank 0. ``value`` is device-timed (CUDA events, max over ranks) with the step's inputs
already on the device; ``e2e`` repeats the measurement through the public per-step API with the inputs copied
from pinned host memory and the loss read back every step. ``--impl reference`` runs the unmodified reference tree
from ``baseline/_ref`` through its own ``StudentModel.train_chunk`` (``baseline/reference_arm.py``); ``--impl baseline`` runs the reference's op sequence on the
libraries that are installed (HF Llama on cuBLAS/SDPA, full fp32 logits, torch AdamW, NCCL DDP).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "student train tokens/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="ours", choices=["ours", "reference", "baseline"])
    ap.add_argument("--model", type=str, default="tinyllama-1.1b")
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--topk", type=int, default=200)
    ap.add_argument("--temperature", type=float, default=2.0)
    ap.add_argument("--loss", type=str, default="kl")
    ap.add_argument("--comm", type=str, default="p2p", choices=["p2p", "nccl"])
    ap.add_argument("--grad-accum", type=int, default=1, help="micro-batches per optimizer step")
    ap.add_argument("--shard", type=str, default="ddp", choices=["ddp", "fsdp", "zero3"],
                    help="ddp/fsdp: weights replicated (fsdp shards the optimizer state); zero3: weights and gradients sharded too")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-collect", action="store_true")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.lines: list[str] = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args) -> int:
    """Runs the unmodified reference tree kept under ``baseline/_ref`` (``baseline/reference_arm.py`` says what stands
    in for the packages this image lacks), or prints the ``unavailable`` line when that cannot be done."""
    from baseline import reference_arm as ra
    return ra.run(args, ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))))


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        print(f"bench.py --gpus {args.gpus} must be launched with torch.distributed.run (WORLD_SIZE={world})",
              file=sys.stderr)
        return 2
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from llm_distillery_b200.models.llama import preset
    cfg = preset(args.model)
    B, L, K = args.micro_batch, args.seq_len, args.topk
    A = max(1, args.grad_accum)
    tokens_per_step = B * L * world * A

    if args.impl == "baseline":
        from baseline.hf_baseline import BaselineRunner
        runner = BaselineRunner(cfg, dev, world, temperature=args.temperature, topk=K, loss=args.loss, shard=args.shard,
                                grad_accum=A)
        launches_of = lambda: 0  # noqa: E731
    else:
        from llm_distillery_b200.engine.trainer import DistillEngine
        from llm_distillery_b200.models.llama import build_model
        from llm_distillery_b200.ops import _lib
        from llm_distillery_b200.parallel.ddp import make_comm
        model = build_model(cfg, dtype=torch.bfloat16, device=dev, seed=1234)
        comm = make_comm(args.comm, dev, shard_strategy=args.shard) if world > 1 else None
        eng = DistillEngine(model, loss=args.loss, temperature=args.temperature, optimizer="adamw", lr=1e-5,
                            crop_to_size=cfg.vocab_size, grad_accum=A, comm=comm)

        class Runner:
            def device_step(self, db):
                for k in range(A):
                    loss, _ = eng.micro_step(db, last=(k + 1 == A))
                eng.optimizer_step()
                return loss

            def e2e_step(self, hb):
                return eng.train_step([hb] * A)

            def to_device(self, hb):
                return hb.to_device(dev)

            def collect_setup(self):
                # self-distillation config: the teacher has the student's architecture (weights shared here)
                from llm_distillery_b200.collect.collector import TeacherCollector
                self.collector = TeacherCollector(model, topk=K, crop_to_size=cfg.vocab_size)

            def collect_step(self, tokens_np, convos):
                return self.collector.content_logprobs(tokens_np, convos)

            def collect_many(self, toks, convos, n):
                """n batches the way the pipeline runs them: batch i+1 is queued before batch i's rows are taken."""
                pending, last = None, None
                for i in range(n):
                    t = self.collector.submit(toks[i % len(toks)], convos)
                    if pending is not None:
                        last = self.collector.fetch(pending)
                    pending = t
                return self.collector.fetch(pending)
        runner = Runner()
        launches_of = lambda: _lib.LAUNCH_COUNT[0]  # noqa: E731

    from llm_distillery_b200.engine.trainer import synthetic_batch
    pool = [synthetic_batch(cfg.vocab_size, B, L, K, seed=100 + 7 * rank + i, device=dev,
                            reference_fields=(args.loss == "reference")).pin() for i in range(2)]
    dev_pool = [runner.to_device(hb) for hb in pool]
    h2d_bytes = pool[0].nbytes()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------- device-timed arm
    for i in range(args.warmup):
        runner.device_step(dev_pool[i % 2])
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    l0 = launches_of()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last = None
    for i in range(args.steps):
        last = runner.device_step(dev_pool[i % 2])
    e1.record()
    barrier()
    launches = launches_of() - l0
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    final_loss = float(last.item())

    # ---------------- end-to-end arm (pinned host inputs, loss read back every step)
    e2e = None
    if not args.skip_e2e:
        for i in range(max(1, args.warmup // 2)):
            runner.e2e_step(pool[i % 2]).item()
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            final_loss = float(runner.e2e_step(pool[i % 2]).item())
        barrier()
        dt = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        e2e = {"value": tokens_per_step * args.steps / float(dt.item()), "unit": "tokens/s",
               "ms_per_step": 1e3 * float(dt.item()) / args.steps, "h2d_bytes_per_step": h2d_bytes * A,
               "d2h_bytes_per_step": 4}
    clocks = sampler.stop() if rank == 0 else None

    # ---------------- what the gradient exchange leaves exposed: device time from the end of backward to the end of
    # the step (reduce + optimizer + weight all-gather), a few extra steps with the phase timer on, max over ranks
    exposed = exchange = None
    if args.impl == "ours" and hasattr(runner, "device_step"):
        eng.timer.enabled = True
        barrier()                       # rank 0 comes late from stopping the clock sampler: without this its peers
        runner.device_step(dev_pool[0])  # would count that wait as exposed time in their first probe step
        barrier()
        eng.timer.summary()
        n_probe = 3
        if comm is not None and hasattr(comm, "time_exchange"):
            comm.time_exchange = True
        for i in range(n_probe):
            runner.device_step(dev_pool[i % 2])
        barrier()
        phases = eng.timer.summary()
        eng.timer.enabled = False
        xms = comm.exchange_ms() if comm is not None and hasattr(comm, "exchange_ms") else None
        if comm is not None and hasattr(comm, "time_exchange"):
            comm.time_exchange = False
        t = torch.tensor([phases.get("reduce+optimizer", 0.0) / n_probe, -1.0 if xms is None else xms], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        exposed = float(t[0].item())
        exchange = None if float(t[1].item()) < 0 else float(t[1].item())

    # ---------------- teacher collection arm (second half of the metric): tokens in -> top-K rows in pinned host memory
    collect = None
    if not args.skip_collect and hasattr(runner, "collect_step"):
        import numpy as np

        class _Convo:      # every position of every sequence is a content row
            length = L

            @staticmethod
            def content_indices():
                return np.arange(L, dtype=np.int64)
        convos = [_Convo() for _ in range(B)]
        toks = [np.random.default_rng(50 + rank + i).integers(0, cfg.vocab_size, (B, L)).astype(np.int64) for i in range(2)]
        with torch.no_grad():
            runner.collect_topk = K
            runner.collect_setup()
            for i in range(4):          # pinned buffers, the copy stream and the top-K workspace are first touched here
                runner.collect_step(toks[i % 2], convos)
            barrier()
            t0 = time.perf_counter()
            n_col = max(8, args.steps // 2)
            d2h = 0
            if hasattr(runner, "collect_many"):
                hv, hi, _ = runner.collect_many(toks, convos, n_col)
            else:
                for i in range(n_col):
                    hv, hi, _ = runner.collect_step(toks[i % 2], convos)
            d2h = hv.numel() * hv.element_size() + hi.numel() * hi.element_size()
            barrier()
        dt = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        collect = {"metric": "teacher collect tokens/s", "value": tokens_per_step * n_col / float(dt.item()),
                   "unit": "tokens/s", "ms_per_batch": 1e3 * float(dt.item()) / n_col, "batches": n_col,
                   "h2d_bytes_per_batch": B * L * 8, "d2h_bytes_per_batch": d2h,
                   "config": {"teacher": args.model, "batch": B, "seq_len": L, "topk": K, "parallelism": f"dp{world}",
                              "rows": "all positions are content rows"}}

    err = 0
    if args.impl == "ours":
        from llm_distillery_b200.ops import _lib
        err = _lib.take_device_error()
    if rank == 0:
        value = tokens_per_step * args.steps / (ms_total / 1e3)
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids + synthetic top-K teacher targets, random-init weights",
            "impl": args.impl,
            "config": {"model": args.model, "global_batch": B * world * A, "micro_batch_per_gpu": B, "grad_accum": A, "seq_len": L,
                       "parallelism": f"dp{world}" + ("" if args.shard == "ddp" or world == 1 else f"-{args.shard}"),
                       "peak_mem_gb": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 2),
                       # whole device, symmetric (peer-mapped) buffers included, which the allocator's peak does not see
                       "device_mem_used_gb": round((lambda fr, tot: (tot - fr) / 2 ** 30)(*torch.cuda.mem_get_info(dev)), 2),
                       "loss": f"{args.loss} T={args.temperature}", "topk": K,
                       "optimizer": "adamw (fp32 master + state)", "comm": args.comm if world > 1 else "none",
                       "l2": "no flush: each step streams ~2.2 GB of weights and >20 GB of activations, far above the 126 MB L2"},
            "e2e": e2e, "exposed_comm_ms": exposed, "exchange_ms": exchange, "collect": collect, "gpu_launches": launches, "clocks": clocks, "final_loss": final_loss, "device_error": err,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
