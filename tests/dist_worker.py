"""Worker run under torch.distributed.run by tests/test_dist.py. Modes:
  cpu_engine  gloo ranks on CPU: ddp and fsdp(all-reduce comm) training equals single-process training on the
              concatenated micro-batches
  gpu_p2p     NCCL + NVLink P2P ranks: P2P all-reduce equals NCCL all-reduce; a P2P-communicated training run equals
              the NCCL-communicated one
Prints "WORKER_OK" on rank 0 when every check passed."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from llm_distillery_b200.engine.trainer import DistillEngine, synthetic_batch  # noqa: E402
from llm_distillery_b200.models.llama import LlamaConfig, build_model  # noqa: E402
from llm_distillery_b200.parallel.ddp import make_comm  # noqa: E402


def tiny(dtype, device):
    cfg = LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                      num_key_value_heads=1, max_position_embeddings=128)
    return build_model(cfg, dtype=dtype, device=device, seed=5), cfg


def run_steps(comm, dtype, device, rank, world, steps, opt="adamw", B=2, L=128):
    model, cfg = tiny(dtype, device)
    eng = DistillEngine(model, loss="kl", temperature=2.0, optimizer=opt, lr=1e-3, comm=comm)
    for s in range(steps):
        hb = synthetic_batch(cfg.vocab_size, B, L, 16, seed=100 * s + rank)
        eng.train_step([hb])
    return torch.cat([p.detach().float().reshape(-1).cpu() for p in model.parameters()])


def cpu_engine():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    out = {}
    for strat in ("ddp", "fsdp"):
        comm = make_comm("gloo", "cpu", shard_strategy=strat)
        out[strat] = run_steps(comm, torch.float32, "cpu", rank, world, 3)
    # single process on all ranks' batches with grad averaging == summing losses / world
    model, cfg = tiny(torch.float32, "cpu")
    eng = DistillEngine(model, loss="kl", temperature=2.0, optimizer="adamw", lr=1e-3, grad_accum=world)
    for s in range(3):
        eng.train_step([synthetic_batch(cfg.vocab_size, 2, 128, 16, seed=100 * s + r) for r in range(world)])
    ref = torch.cat([p.detach().float().reshape(-1) for p in model.parameters()])
    for strat, got in out.items():
        err = (got - ref).abs().max().item()
        assert err < 2e-5, (strat, err)
    gathered = [torch.empty_like(out["ddp"]) for _ in range(world)]
    dist.all_gather(gathered, out["fsdp"])
    assert all(torch.equal(g, gathered[0]) for g in gathered), "ranks diverged"
    if rank == 0:
        print("WORKER_OK")
    dist.destroy_process_group()


def gpu_p2p():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from llm_distillery_b200.ops import _lib
    from llm_distillery_b200.parallel.p2p import P2PComm, SymmetricBuffer
    comm = P2PComm(dev)
    n = 1 << 20
    buf = SymmetricBuffer(n + 12, torch.float32, dev)
    g = torch.Generator(device=dev).manual_seed(rank)
    buf.tensor.copy_(torch.randn(n + 12, device=dev, generator=g))
    ref = buf.tensor.clone()
    dist.all_reduce(ref)
    comm.allreduce_(buf, 1.0)
    torch.cuda.synchronize()
    assert _lib.take_device_error() == 0
    assert torch.allclose(buf.tensor, ref, atol=1e-5, rtol=1e-5), (buf.tensor - ref).abs().max()
    for opt in ("adamw", "sgd"):
        a = run_steps(P2PComm(dev), torch.bfloat16, dev, rank, world, 3, opt)
        b = run_steps(make_comm("nccl", dev), torch.bfloat16, dev, rank, world, 3, opt)
        torch.cuda.synchronize()
        assert _lib.take_device_error() == 0
        err = (a - b).abs().max().item()
        assert err < 2e-2, (opt, err)
        flat = a.to(dev)
        parts = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(parts, flat)
        assert all(torch.equal(p, parts[0]) for p in parts), "ranks hold different weights"
    if rank == 0:
        print("WORKER_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    {"cpu_engine": cpu_engine, "gpu_p2p": gpu_p2p}[sys.argv[1]]()
