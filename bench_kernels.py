#!/usr/bin/env python
"""Kernel micro-benchmarks with roofline fractions against the measured box peaks (MEASURED_PEAKS.json when
present, else the documented fallback of 6.65 TB/s and 1.59 PFLOP/s).

    python bench_kernels.py gemm --m 16384 --n 2048 --k 2048 [--layout nt|nn|tn] [--iters 20]
    python bench_kernels.py attn --batch 8 --seq 2048 --heads 32 --kv-heads 4 --dim 64 [--bwd]
    python bench_kernels.py head --rows 16384 --hidden 2048 --vocab 32000 --topk 200
    python bench_kernels.py elementwise --rows 16384 --hidden 2048 --ffn 5632
    python bench_kernels.py topk --rows 4096 --vocab 32000 --topk 200     (top-K extraction, merge, remap)
    python bench_kernels.py all            (the model shapes of the headline benchmark)

Timing: CUDA events on the launching stream, warm-up first, L2 flushed between timed iterations by writing a
256 MB buffer (its time is excluded: one event pair per iteration). One JSON line per case.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from llm_distillery_b200.ops import basic, attention, _lib  # noqa: E402


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "tflops_sustained": d.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


_FLUSH = None


def timed(fn, iters: int, warmup: int = 3, flush: bool = True) -> float:
    """Median milliseconds per call."""
    global _FLUSH
    if flush and _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            _FLUSH.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def report(name, ms, flops=None, bytes_=None, **extra):
    pk = peaks()
    out = {"kernel": name, "ms": round(ms, 4), **extra}
    if flops:
        tf = flops / ms / 1e9
        out.update(tflops=round(tf, 1), frac_of_peak=round(tf / pk["tflops"], 3), peak=f"{pk['tflops']} TF/s of {pk['source']}")
    if bytes_:
        gbs = bytes_ / ms / 1e6
        out.update(gbs=round(gbs, 1), frac_of_hbm=round(gbs / pk["hbm_gbs"], 3), hbm=f"{pk['hbm_gbs']} GB/s of {pk['source']}")
    err = _lib.take_device_error()
    if err:
        out["device_error"] = err
    print(json.dumps(out), flush=True)


def bench_gemm(M, N, K, layout, iters, compare=True):
    a_mn, b_mn = {"nt": (False, False), "nn": (False, True), "tn": (True, True)}[layout]
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda").bfloat16()
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda").bfloat16()
    out = torch.empty((M, N), device="cuda", dtype=torch.bfloat16)
    extra = {}
    if layout == "tn":
        # the weight-gradient GEMM as the trainer runs it: fp32 accumulation into the gradient buffer
        acc = torch.zeros((M, N), device="cuda", dtype=torch.float32)
        ms = timed(lambda: basic.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=acc, accumulate=True), iters)
        extra["output"] = "fp32 +="
    else:
        ms = timed(lambda: basic.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out), iters)
    if compare:
        A, B = (a.t() if a_mn else a), (b if b_mn else b.t())
        extra["cublas_ms"] = round(timed(lambda: torch.matmul(A, B, out=out), iters), 4)
        if layout == "tn":
            extra["cublas_note"] = "bf16 output, no accumulation"
    report(f"gemm_{layout}", ms, flops=2.0 * M * N * K, shape=[M, N, K], **extra)


def bench_fused(rows, hidden, ffn, heads, kv_heads, dim, iters):
    """The GEMMs whose epilogues absorb an elementwise kernel, each against its two-kernel path on the same operands:
    gate / up projection + SwiGLU, down-projection dgrad + SwiGLU backward, q/k/v projection + rotary embedding."""
    x = torch.randn(rows, hidden, device="cuda").bfloat16()
    w_gu = (torch.randn(2 * ffn, hidden, device="cuda") * 0.02).bfloat16()
    w_d = (torch.randn(hidden, ffn, device="cuda") * 0.02).bfloat16()
    dy = torch.randn(rows, hidden, device="cuda").bfloat16()
    gu, _ = basic.linear_swiglu_fwd(x, w_gu)
    fl = 2.0 * rows * hidden * 2 * ffn
    ms = timed(lambda: basic.linear_swiglu_fwd(x, w_gu), iters)
    ms2 = timed(lambda: basic.swiglu_fwd(basic.linear_fwd(x, w_gu)), iters)
    report("gate_up_gemm+swiglu", ms, flops=fl, shape=[rows, 2 * ffn, hidden], two_kernels_ms=round(ms2, 4))
    ms = timed(lambda: basic.linear_dgrad_swiglu_bwd(dy, w_d, gu), iters)
    ms2 = timed(lambda: basic.swiglu_bwd(gu, basic.linear_dgrad(dy, w_d)), iters)
    report("down_dgrad+swiglu_bwd", ms, flops=2.0 * rows * hidden * ffn, shape=[rows, ffn, hidden],
           two_kernels_ms=round(ms2, 4))
    n = (heads + 2 * kv_heads) * dim
    w_qkv = (torch.randn(n, hidden, device="cuda") * 0.02).bfloat16()
    pos = (torch.arange(rows, device="cuda", dtype=torch.int32) % 2048)
    cos, sin = basic.rope_tables(2048, dim, 10000.0, "cuda")
    ms = timed(lambda: basic.linear_rope_fwd(x, w_qkv, pos, cos, sin, heads + kv_heads, dim), iters)
    ms2 = timed(lambda: basic.rope_(basic.linear_fwd(x, w_qkv), pos, cos, sin, heads + kv_heads, dim), iters)
    report("qkv_gemm+rope", ms, flops=2.0 * rows * hidden * n, shape=[rows, n, hidden], two_kernels_ms=round(ms2, 4))


def _sm_clock_mhz():
    """SM clock right now (read through NVML; None when it is not available)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
        return int(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
    except Exception:  # noqa: BLE001
        return None


def bench_attn(B, L, H, Hkv, d, iters, bwd, library=True):
    """This repository's kernels, then the library kernels on the same tensors: flash_attn 2.8 (the reference's
    ``attn_implementation="flash_attention_2"``) and torch SDPA (its fallback)."""
    qkv = torch.randn(B * L, (H + 2 * Hkv) * d, device="cuda").bfloat16()
    out, lse = attention.attention_fwd(qkv, B, L, H, Hkv, d)
    fl = 4.0 * B * H * L * L * d / 2
    ms = timed(lambda: attention.attention_fwd(qkv, B, L, H, Hkv, d), iters)
    report("flash_attn_fwd", ms, flops=fl, shape=[B, L, H, Hkv, d], sm_mhz=_sm_clock_mhz())
    dout = torch.randn_like(out)
    if bwd:
        ms = timed(lambda: attention.attention_bwd(dout, qkv, out, lse, B, L, H, Hkv, d), iters)
        report("flash_attn_bwd", ms, flops=2.5 * fl, shape=[B, L, H, Hkv, d], sm_mhz=_sm_clock_mhz())
    if not library:
        return
    q4 = qkv.view(B, L, H + 2 * Hkv, d)
    q, k, v = (q4[:, :, :H].contiguous().requires_grad_(bwd), q4[:, :, H:H + Hkv].contiguous().requires_grad_(bwd),
               q4[:, :, H + Hkv:].contiguous().requires_grad_(bwd))
    do4 = dout.view(B, L, H, d)
    try:
        from flash_attn import flash_attn_func
        o = flash_attn_func(q, k, v, causal=True)
        ms = timed(lambda: flash_attn_func(q, k, v, causal=True), iters)
        report("library flash_attn 2 fwd", ms, flops=fl, shape=[B, L, H, Hkv, d], sm_mhz=_sm_clock_mhz())
        if bwd:
            ms = timed(lambda: torch.autograd.grad(o, (q, k, v), do4, retain_graph=True), iters)
            report("library flash_attn 2 bwd", ms, flops=2.5 * fl, shape=[B, L, H, Hkv, d], sm_mhz=_sm_clock_mhz())
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"kernel": "library flash_attn 2", "unavailable": f"{type(e).__name__}: {e}"[:200]}), flush=True)
    try:
        import torch.nn.functional as F
        qs, ks, vs = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        f = lambda: F.scaled_dot_product_attention(qs, ks, vs, is_causal=True, enable_gqa=True)  # noqa: E731
        o = f()
        ms = timed(f, iters)
        report("library torch sdpa fwd", ms, flops=fl, shape=[B, L, H, Hkv, d], sm_mhz=_sm_clock_mhz())
        if bwd:
            dos = do4.transpose(1, 2)
            ms = timed(lambda: torch.autograd.grad(o, (q, k, v), dos, retain_graph=True), iters)
            report("library torch sdpa bwd", ms, flops=2.5 * fl, shape=[B, L, H, Hkv, d], sm_mhz=_sm_clock_mhz())
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"kernel": "library torch sdpa", "unavailable": f"{type(e).__name__}: {e}"[:200]}), flush=True)


def bench_head(M, h, V, K, iters, T=2.0):
    from llm_distillery_b200.loss import head
    from llm_distillery_b200.models.llama import GradSlot
    Hc = torch.randn(M, h, device="cuda").bfloat16().requires_grad_()
    W = (torch.randn(V, h, device="cuda") * 0.02).bfloat16().requires_grad_()
    W.grad_slot = GradSlot(torch.zeros(V, h, device="cuda"))
    ids = torch.rand(M, V, device="cuda").topk(K, -1).indices.sort(-1).values.int() if V * M < 2 ** 30 else \
        torch.stack([torch.randperm(V, device="cuda")[:K].sort().values for _ in range(M)]).int()
    u = torch.log_softmax(torch.randn(M, K, device="cuda") * 3, -1)

    def fwd():
        return head.fused_distill_rows(Hc, W, ids, u, "kl", T, V)

    def fwd_bwd():
        Hc.grad = None
        fwd().sum().backward()

    gemm_fl = 2.0 * M * V * h
    with torch.no_grad():
        report("distill_head_fwd", timed(fwd, iters), flops=gemm_fl, shape=[M, h, V, K])
    report("distill_head_fwd_bwd", timed(fwd_bwd, iters), flops=4 * gemm_fl, shape=[M, h, V, K],
           note="4 GEMM-equivalents: stats, recompute, dH, dW")


def bench_elementwise(rows, h, f, iters):
    x = torch.randn(rows, h, device="cuda").bfloat16()
    w = torch.ones(h, device="cuda").bfloat16()
    y, _, rstd = basic.rmsnorm_fwd(x, w, 1e-5)
    report("rmsnorm_fwd", timed(lambda: basic.rmsnorm_fwd(x, w, 1e-5), iters), bytes_=2 * rows * h * 2, shape=[rows, h])
    report("rmsnorm_bwd", timed(lambda: basic.rmsnorm_bwd(y, x, w, rstd, x), iters), bytes_=4 * rows * h * 2, shape=[rows, h])
    gu = torch.randn(rows, 2 * f, device="cuda").bfloat16()
    act = basic.swiglu_fwd(gu)
    report("swiglu_fwd", timed(lambda: basic.swiglu_fwd(gu), iters), bytes_=3 * rows * f * 2, shape=[rows, f])
    report("swiglu_bwd", timed(lambda: basic.swiglu_bwd(gu, act), iters), bytes_=5 * rows * f * 2, shape=[rows, f])
    pos = torch.arange(rows, device="cuda", dtype=torch.int32) % 2048
    cos, sin = basic.rope_tables(2048, 64, 10000.0, "cuda")
    q = torch.randn(rows, h + 512, device="cuda").bfloat16()
    report("rope", timed(lambda: basic.rope_(q, pos, cos, sin, (h + 256) // 64, 64), iters), bytes_=2 * rows * (h + 256) * 2,
           shape=[rows, h + 256])
    n = 64 << 20
    from llm_distillery_b200.engine.optim import FlatOptimizer, FlatParams
    p = torch.nn.Parameter(torch.randn(n, device="cuda").bfloat16())
    opt = FlatOptimizer(FlatParams([p]), "adamw", lr=1e-4)
    report("adamw", timed(lambda: opt.step(), iters), bytes_=n * 30, shape=[n])


def bench_topk_family(rows, V, K, iters):
    """Exact top-K log-prob extraction, multi-teacher merge and cross-tokenizer remap against their library / CPU
    statements (the CPU loops are timed on 256 rows and scaled)."""
    import time
    from llm_distillery_b200.ops import topk as tk
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    logits = torch.randn((rows, V), device=dev, generator=g) * 3
    ms = timed(lambda: tk.topk_logprob(logits, V, K), iters)
    ms_t = timed(lambda: torch.topk(torch.log_softmax(logits, -1), K, dim=-1), max(3, iters // 2))
    report("topk_logprob", ms, bytes_=rows * V * 4.0, shape=[rows, V, K], torch_ms=round(ms_t, 4),
           speedup_vs_torch=round(ms_t / ms, 2), note="torch = log_softmax + topk on the same fp32 logits")
    a_lp, a_id = tk.topk_logprob(logits, V, K)
    b_lp, b_id = tk.topk_logprob(logits.roll(1, 0) + 0.5 * torch.randn_like(logits), V, K)
    a_lp, b_lp = a_lp.float(), b_lp.float()
    ms = timed(lambda: tk.topk_merge(a_lp, a_id, b_lp, b_id), iters, flush=False)
    sub = 256
    ca = [t[:sub].cpu() for t in (a_lp, a_id, b_lp, b_id)]
    t0 = time.perf_counter()
    tk.topk_merge(*ca)
    cpu_ms = (time.perf_counter() - t0) * 1e3 * rows / sub
    report("topk_merge", ms, bytes_=rows * K * 8.0 * 3, shape=[rows, K], cpu_loop_ms=round(cpu_ms, 1),
           speedup_vs_cpu_loop=round(cpu_ms / ms, 1), note="CPU = per-row unique + index_add + sort (the reference's merge rule)")
    table = torch.randint(-1, 32000, (V,), device=dev, generator=g, dtype=torch.int32)
    ms = timed(lambda: tk.remap_topk(a_lp, a_id, table, K), iters, flush=False)
    t0 = time.perf_counter()
    tk.remap_topk(ca[0], ca[1], table.cpu(), K)
    cpu_ms = (time.perf_counter() - t0) * 1e3 * rows / sub
    report("remap_topk", ms, bytes_=rows * K * 8.0 * 2, shape=[rows, K, V], cpu_loop_ms=round(cpu_ms, 1),
           speedup_vs_cpu_loop=round(cpu_ms / ms, 1), note="CPU = per-row table lookup + unique + index_add + sort")


def bench_trie_walk(iters):
    """Teacher-vocabulary -> student-vocabulary table of a 32 000-token teacher against a 128 256-token student
    (synthetic byte-fallback vocabularies): the trie-walk kernel against the per-token Python walk."""
    import random
    import time
    from llm_distillery_b200.align.aligner import ByteTrie
    from llm_distillery_b200.ops import topk as tk
    rng = random.Random(0)
    alpha = bytes(range(97, 123)) + b" \xc3\xa9"

    def words(n):
        return [bytes(rng.choice(alpha) for _ in range(rng.randint(2, 12))) for _ in range(n)]
    student = [bytes([b]) for b in range(256)] + words(128256 - 256)
    teacher = [bytes([b]) for b in range(256)] + words(32000 - 256)
    trie = ByteTrie()
    for i, b in enumerate(student):
        trie.insert(b, i)
    flat = trie.flatten()
    t0 = time.perf_counter()
    want = [trie.longest_prefix(b) for b in teacher]
    cpu_ms = (time.perf_counter() - t0) * 1e3
    got, _ = tk.trie_walk(flat, teacher, "cuda")
    assert got.cpu().tolist() == want
    # device-resident inputs: time the kernel, not the upload of the trie
    g = {k: torch.from_numpy(v).cuda() for k, v in flat.items()}
    import numpy as np
    lens = np.fromiter((len(b) for b in teacher), dtype=np.int64, count=len(teacher))
    off = np.zeros(len(teacher) + 1, dtype=np.int64)
    np.cumsum(lens, out=off[1:])
    tb = torch.from_numpy(np.frombuffer(b"".join(teacher), dtype=np.uint8).copy()).cuda()
    to = torch.from_numpy(off).cuda()
    out = torch.empty(len(teacher), dtype=torch.int32, device="cuda")
    lib = _lib.kernels()

    def run():
        _lib.check(lib.b200_trie_walk(_lib.ptr(g["edge_start"]), _lib.ptr(g["edge_byte"]), _lib.ptr(g["edge_child"]),
                                      _lib.ptr(g["node_value"]), g["node_value"].numel(), _lib.ptr(tb), _lib.ptr(to),
                                      len(teacher), _lib.ptr(out), None, _lib.stream()), "b200_trie_walk")
    ms = timed(run, iters)
    report("trie_walk", ms, shape=[len(teacher), len(student), int(g["node_value"].numel())], cpu_loop_ms=round(cpu_ms, 1),
           speedup_vs_cpu_loop=round(cpu_ms / ms, 1), bytes_walked=int(off[-1]),
           note="shape = teacher tokens, student tokens, trie nodes; CPU = dictionary trie walked token by token in Python")


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8192); g.add_argument("--n", type=int, default=8192)
    g.add_argument("--k", type=int, default=8192); g.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"])
    a = sub.add_parser("attn")
    a.add_argument("--batch", type=int, default=8); a.add_argument("--seq", type=int, default=2048)
    a.add_argument("--heads", type=int, default=32); a.add_argument("--kv-heads", type=int, default=4)
    a.add_argument("--dim", type=int, default=64); a.add_argument("--bwd", action="store_true")
    a.add_argument("--no-library", action="store_true", help="this repository's kernels only (for profiler captures)")
    h = sub.add_parser("head")
    h.add_argument("--rows", type=int, default=16384); h.add_argument("--hidden", type=int, default=2048)
    h.add_argument("--vocab", type=int, default=32000); h.add_argument("--topk", type=int, default=200)
    e = sub.add_parser("elementwise")
    e.add_argument("--rows", type=int, default=16384); e.add_argument("--hidden", type=int, default=2048)
    e.add_argument("--ffn", type=int, default=5632)
    t = sub.add_parser("topk")
    t.add_argument("--rows", type=int, default=4096); t.add_argument("--vocab", type=int, default=32000)
    t.add_argument("--topk", type=int, default=200)
    fu = sub.add_parser("fused")
    fu.add_argument("--rows", type=int, default=16384); fu.add_argument("--hidden", type=int, default=2048)
    fu.add_argument("--ffn", type=int, default=5632); fu.add_argument("--heads", type=int, default=32)
    fu.add_argument("--kv-heads", type=int, default=4); fu.add_argument("--dim", type=int, default=64)
    sub.add_parser("all")
    for s in (g, a, h, e, t, fu, sub.choices["all"]):
        s.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    if args.cmd == "gemm":
        bench_gemm(args.m, args.n, args.k, args.layout, args.iters)
    elif args.cmd == "attn":
        bench_attn(args.batch, args.seq, args.heads, args.kv_heads, args.dim, args.iters, args.bwd,
                   library=not args.no_library)
    elif args.cmd == "head":
        bench_head(args.rows, args.hidden, args.vocab, args.topk, args.iters)
    elif args.cmd == "elementwise":
        bench_elementwise(args.rows, args.hidden, args.ffn, args.iters)
    elif args.cmd == "topk":
        bench_topk_family(args.rows, args.vocab, args.topk, args.iters)
        bench_trie_walk(args.iters)
    elif args.cmd == "fused":
        bench_fused(args.rows, args.hidden, args.ffn, args.heads, args.kv_heads, args.dim, args.iters)
    else:
        for shp, lay in [((8192, 8192, 8192), "nt"), ((16384, 2560, 2048), "nt"), ((16384, 2048, 2048), "nt"),
                         ((16384, 11264, 2048), "nt"), ((16384, 2048, 5632), "nt"), ((16384, 2048, 2560), "nn"),
                         ((16384, 2048, 11264), "nn"), ((16384, 5632, 2048), "nn"), ((2560, 2048, 16384), "tn"),
                         ((11264, 2048, 16384), "tn"), ((2048, 5632, 16384), "tn"), ((2048, 2048, 16384), "tn")]:
            bench_gemm(*shp, lay, args.iters)
        bench_attn(8, 2048, 32, 4, 64, args.iters, True)
        bench_attn(2, 4096, 32, 8, 128, args.iters, True)
        bench_head(16384, 2048, 32000, 200, max(3, args.iters // 4))
        bench_elementwise(16384, 2048, 5632, args.iters)
        bench_fused(16384, 2048, 5632, 32, 4, 64, args.iters)
        bench_topk_family(4096, 32000, 200, max(3, args.iters // 2))
        bench_trie_walk(max(3, args.iters // 2))


if __name__ == "__main__":
    main()
