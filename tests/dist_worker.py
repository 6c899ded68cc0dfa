"""Worker run under torch.distributed.run by tests/test_dist.py. Modes:
  cpu_engine  gloo ranks on CPU: ddp and fsdp(all-reduce comm) training equals single-process training on the
              concatenated micro-batches
  cpu_zero3   gloo ranks on CPU: full parameter sharding (weights gathered per unit, gradients reduce-scattered per
              layer) equals single-process training, with gradient accumulation, an evaluation between steps, a rank
              without a micro-batch, tied embeddings, a frozen layer and a checkpoint taken through the gathered view
  cpu_cli_zero3  gloo ranks on CPU: the command-line pipeline trains the same student replicated and fully sharded
  gpu_cli_zero3  the same pipeline on two GPUs in bf16
  cpu_cli_zero3_chunked  the same with a cache that holds only part of the data (collect / train / state per chunk)
  cpu_cli_zero3_three / cpu_cli_zero3_accum  the same on three ranks / with an accumulation that straddles epochs
  cpu_cli_zero3_variants  gradient checkpointing, shuffled order, reference loss, frozen layer, other optimizers
  cpu_cli_rank_loss  a rank's process ends between two steps of the command-line run: the other saves state, status 3
  cpu_cli_sync  the dataset changes between two runs: only the new conversations are collected, the store is re-keyed
  cpu_cli_resume  a fully sharded run stopped after one epoch and taken up again equals the uninterrupted run
  cpu_cli_config3  two teachers (one cross-tokenizer), tied-embedding student, JSD, fully sharded, planner-chosen widths
  gpu_zero3   GPU ranks: full parameter sharding, over NCCL and over the peer-access kernels, equals the replicated run
  gpu_p2p     NCCL + NVLink P2P ranks: P2P all-reduce equals NCCL all-reduce; a P2P-communicated training run equals
              the NCCL-communicated one
  cpu_tp      gloo ranks on CPU: the tensor-parallel teacher's top-K log-probs equal the unsharded model's
  cpu_vp_head gloo ranks on CPU: the vocabulary-parallel loss head equals the unsharded head (loss, dH, dW)
  cpu_rank_loss  three gloo ranks, one leaves between steps: the others find out through the heartbeat and leave
  cpu_cli_tp  gloo ranks on CPU: the command-line pipeline with tp_size = 2 stores what a single process stores
  gpu_tp      NVLink ranks: fused all-gather->GEMM and GEMM->reduce-scatter equal NCCL + matmul; the tensor-parallel
              teacher's top-K log-probs equal the single-GPU model's
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


def _tiny3(dtype, device, tied):
    moe = dict(model_type="mixtral", num_local_experts=4, num_experts_per_tok=2) if os.environ.get("Z3_MOE") == "1" else {}
    if os.environ.get("Z3_FAMILY") == "olmo2":       # norms behind the branches, none in front: models/sandwich.py
        moe = {}
        tied = False
        extra = dict(model_type="olmo2", pre_norm=False, post_norm=True, qk_norm_full=True)
    elif os.environ.get("Z3_FAMILY") == "glm4":
        extra = dict(model_type="glm4", post_norm=True, attention_bias=True, partial_rotary_factor=0.5, rope_interleaved=True)
    else:
        extra = {}
    moe = dict(moe, **extra)
    cfg = LlamaConfig(vocab_size=512, hidden_size=128, intermediate_size=256, num_hidden_layers=3, num_attention_heads=2,
                      num_key_value_heads=1, max_position_embeddings=128, tie_word_embeddings=tied, **moe)
    model = build_model(cfg, dtype=dtype, device=device, seed=7)
    if cfg.num_local_experts:
        with torch.no_grad():          # decisive routing: the sharded and the single-process run must pick the same experts
            for l in model.layers:
                l.router.mul_(25.0)
    return model, cfg


def _zero3_case(device, dtype, rank, world, tied, freeze, comm_factory, accum=2, steps=3, L=64, close=False):
    """Returns (weights after training under the communicator, loss of an evaluation batch between the steps)."""
    model, cfg = _tiny3(dtype, device, tied)
    if freeze:
        for p in model.layers[1].parameters():
            p.requires_grad_(False)
    comm = comm_factory()
    eng = DistillEngine(model, loss="kl", temperature=2.0, optimizer="adamw", lr=1e-3, grad_accum=accum, comm=comm)
    ev = None
    for s in range(steps):
        for m in range(accum):
            if s == 1 and m == 1 and rank == world - 1 and world > 1:
                eng.idle_micro_step(last=(m + 1 == accum))   # the last rank has no second micro-batch in step 1
                continue
            hb = synthetic_batch(cfg.vocab_size, 2, L, 16, seed=1000 * s + 10 * m + rank)
            # step 2 leaves it to the engine's count whether this is the last micro-batch (unfused update)
            eng.micro_step(hb.to_device(device), last=(m + 1 == accum) if s < 2 else None)
        eng.optimizer_step()
        if s == 0:
            ev = float(eng.eval_batch(synthetic_batch(cfg.vocab_size, 2, L, 16, seed=77))[0])
    with eng.full_parameters():
        w = torch.cat([p.detach().float().reshape(-1).cpu() for p in model.parameters()])
    stats = dict(getattr(comm, "stats", {}))
    if close and hasattr(comm, "close"):
        comm.close()
    return w, ev, (stats if close else eng)


def _zero3_reference(device, dtype, world, tied, freeze, accum=2, steps=3, L=64):
    model, cfg = _tiny3(dtype, device, tied)
    if freeze:
        for p in model.layers[1].parameters():
            p.requires_grad_(False)
    eng = DistillEngine(model, loss="kl", temperature=2.0, optimizer="adamw", lr=1e-3, grad_accum=accum * world)
    ev = None
    for s in range(steps):
        for m in range(accum):
            for r in range(world):
                if s == 1 and m == 1 and r == world - 1 and world > 1:
                    continue
                eng.micro_step(synthetic_batch(cfg.vocab_size, 2, L, 16, seed=1000 * s + 10 * m + r).to_device(device))
        eng.optimizer_step()
        if s == 0:
            ev = float(eng.eval_batch(synthetic_batch(cfg.vocab_size, 2, L, 16, seed=77))[0])
    return torch.cat([p.detach().float().reshape(-1).cpu() for p in model.parameters()]), ev


def cpu_zero3():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from llm_distillery_b200.parallel.fsdp import FullShardComm
    eng = None
    for tied, freeze in ((False, False), (True, False), (False, True)):
        if eng is not None:
            eng.comm.close()        # one fully sharded engine per process at a time
        got, ev, eng = _zero3_case("cpu", torch.float32, rank, world, tied, freeze,
                                   lambda: make_comm("gloo", "cpu", shard_strategy="zero3"))
        assert isinstance(eng.comm, FullShardComm)
        ref, ev_ref = _zero3_reference("cpu", torch.float32, world, tied, freeze)
        err = (got - ref).abs().max().item()
        assert err < 2e-5, (tied, freeze, err)
        assert abs(ev - ev_ref) < 1e-4 * max(1.0, abs(ev_ref)), (ev, ev_ref)
        flat = eng.flat
        n_params = sum(p.numel() for p in flat.params)
        # every rank keeps 1/world of the weights, master weights, gradient and moments
        assert flat.master.numel() == flat.shard_size and flat.shard_size * world == flat.total
        assert flat.shard_size < n_params / world * 1.2 + 4096
        assert eng.opt.state["m"].numel() == flat.shard_size
    # a checkpoint written through the gathered view loads into a fresh, differently initialised engine
    import tempfile
    from llm_distillery_b200.ckpt import hf as ckpt
    d = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(d, src=0)
    with eng.full_parameters():
        ckpt.save_trainer_state(d[0], eng.model if rank == 0 else None, eng.opt, eng.schedule, {"k": 1})
    dist.barrier()
    model2, cfg = _tiny3(torch.float32, "cpu", False)
    for p in model2.layers[1].parameters():
        p.requires_grad_(False)
    with torch.no_grad():
        for p in model2.parameters():
            p.add_(0.5)
    try:        # a second fully sharded engine while the first is still active is refused
        DistillEngine(_tiny3(torch.float32, "cpu", False)[0], loss="kl", optimizer="adamw",
                      comm=make_comm("gloo", "cpu", shard_strategy="zero3"))
        raise AssertionError("two active fully sharded engines were accepted")
    except RuntimeError as e:
        assert "close()" in str(e)
    master1, v1, steps1 = eng.flat.master.clone(), eng.opt.state["v"].clone(), eng.opt.step_count
    eng.comm.close()
    eng2 = DistillEngine(model2, loss="kl", temperature=2.0, optimizer="adamw", lr=1e-3, grad_accum=2,
                         comm=make_comm("gloo", "cpu", shard_strategy="zero3"))
    with eng2.full_parameters(writeback=True):
        ckpt.load_model_state(d[0], model2)
    ckpt.load_trainer_state(d[0], None, eng2.opt, eng2.schedule)
    assert torch.equal(eng2.flat.master, master1) and eng2.opt.step_count == steps1
    assert torch.equal(eng2.opt.state["v"], v1)
    with eng2.full_parameters():
        w2 = torch.cat([p.detach().float().reshape(-1) for p in model2.parameters()])
    assert torch.equal(w2, got), (w2 - got).abs().max()
    # HuggingFace-layout checkpoint with the shard files written by the ranks side by side
    hf_dir = os.path.join(d[0], "hf")
    with eng2.full_parameters():
        ckpt.save_hf_model(model2, hf_dir, writer=(rank, world), max_shard_bytes=200_000)
    dist.barrier()
    if rank == 0:
        import json
        files = sorted(f for f in os.listdir(hf_dir) if f.endswith(".safetensors"))
        assert len(files) >= world, files
        index = json.load(open(os.path.join(hf_dir, "model.safetensors.index.json")))
        assert set(index["weight_map"].values()) == set(files)
        back = ckpt.load_hf_model(hf_dir, dtype=torch.float32)
        wb = torch.cat([p.detach().float().reshape(-1) for p in back.parameters()])
        assert torch.equal(wb, got)
    if rank == 0:
        print("WORKER_OK")
    dist.destroy_process_group()


def _late_rank_step(dev, rank, world, comm_factory):
    """One rank arrives three seconds late at a step - longer than the two seconds a device-side wait lasts. The
    communicators bring the streams together through NCCL first, so no wait runs out."""
    import time
    from llm_distillery_b200.ops import _lib
    model, cfg = _tiny3(torch.bfloat16, dev, False)
    comm = comm_factory()
    eng = DistillEngine(model, loss="kl", temperature=2.0, optimizer="adamw", lr=1e-3, comm=comm)
    for s in range(3):
        if s == 1 and rank == world - 1:
            time.sleep(3.0)
        loss = eng.train_step([synthetic_batch(cfg.vocab_size, 2, 128, 16, seed=50 + s + rank)])
    torch.cuda.synchronize()
    assert _lib.take_device_error() == 0, "a bounded wait ran out although every rank was alive"
    assert torch.isfinite(loss).all()
    if hasattr(comm, "close"):
        comm.close()


def gpu_zero3():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from llm_distillery_b200.ops import _lib
    for tied in (False, True):
        b, ev_b, _ = _zero3_case(dev, torch.bfloat16, rank, world, tied, False,
                                 lambda: make_comm("nccl", dev, shard_strategy="ddp"), L=128, close=True)
        for kind in ("nccl", "p2p"):        # library collectives, then the peer-access kernels
            a, ev_a, stats = _zero3_case(dev, torch.bfloat16, rank, world, tied, False,
                                         lambda: make_comm(kind, dev, shard_strategy="zero3"), L=128, close=True)
            torch.cuda.synchronize()
            assert _lib.take_device_error() == 0
            err = (a - b).abs().max().item()
            assert err < 2e-2, (kind, tied, err)
            assert abs(ev_a - ev_b) < 2e-2 * max(1.0, abs(ev_b)), (kind, ev_a, ev_b)
            assert stats["gathers"] > 0 and stats["reduces"] > 0
            flat = a.to(dev)
            parts = [torch.empty_like(flat) for _ in range(world)]
            dist.all_gather(parts, flat)
            assert all(torch.equal(p, parts[0]) for p in parts), "ranks hold different weights"
    _late_rank_step(dev, rank, world, lambda: make_comm("p2p", dev, shard_strategy="zero3"))
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
    _late_rank_step(dev, rank, world, lambda: P2PComm(dev))
    # training through the vocabulary-parallel head (fused kernels, peer loads) against replicated heads
    finals = {}
    for vp in (False, True):
        model, cfg = tiny(torch.bfloat16, dev)
        eng = DistillEngine(model, loss="kl", temperature=2.0, optimizer="adamw", lr=1e-3, comm=P2PComm(dev),
                            crop_to_size=500, vocab_parallel=vp, max_rows_per_rank=256)
        for s in range(3):
            eng.train_step([synthetic_batch(cfg.vocab_size, 2, 128 if rank == 0 else 96, 16, seed=100 * s + rank)])
        finals[vp] = torch.cat([p.detach().float().reshape(-1) for p in model.parameters()])
    torch.cuda.synchronize()
    assert _lib.take_device_error() == 0
    err = (finals[True] - finals[False]).abs().max().item()
    assert err < 2e-2, ("vocabulary-parallel training", err)
    if rank == 0:
        print("WORKER_OK")
    dist.destroy_process_group()


def _tp_model_check(dev, dtype, rank, world, k, atol):
    from llm_distillery_b200.ops import topk as topk_ops
    from llm_distillery_b200.parallel.tp import TPGroup, TPLlama, padded_seq_len
    cfg = LlamaConfig(vocab_size=1000, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2 if world <= 2 else 4, max_position_embeddings=1024)
    if world > 2:
        cfg.num_attention_heads = 2 * world
        cfg.num_key_value_heads = world
        cfg.hidden_size = 64 * cfg.num_attention_heads
    if os.environ.get("TP_QKNORM") == "1":       # Qwen3-style per-head q/k norms: local to a head, so to a rank
        cfg.qk_norm, cfg.model_type = True, "qwen3"
    if os.environ.get("TP_VARIANT") == "partial_nope":     # three quarters of a head rotate; the second layer not at all
        cfg.partial_rotary_factor, cfg.no_rope_layers, cfg.model_type = 0.75, [1, 0], "smollm3"
    full = build_model(cfg, dtype=dtype, device=dev, seed=11)
    if cfg.qk_norm:
        gq = torch.Generator().manual_seed(5)        # the same values on every rank
        with torch.no_grad():
            for l in full.layers:
                l.q_norm.copy_(torch.empty(cfg.head_dim).uniform_(0.5, 1.5, generator=gq).to(dtype))
                l.k_norm.copy_(torch.empty(cfg.head_dim).uniform_(0.5, 1.5, generator=gq).to(dtype))
    B = 2
    L = padded_seq_len(B, 100, world)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab_size, (B, L), generator=g)
    vocab = 990          # cropped vocabulary that does not divide evenly
    grp = TPGroup(dev, B * L, cfg.hidden_size, topk=k, dtype=dtype)
    tpm = TPLlama.from_full(full, grp, vocab=vocab)
    for _ in range(2):   # twice: buffers and epochs are reused
        lp, ix = tpm.topk_logprobs(ids, k)
    with torch.no_grad():
        hs = full.hidden_states(ids.to(dev))
        logits = hs.float() @ full.lm_head[:vocab].float().t()
    ref_lp, ref_ix = topk_ops.topk_logprob(logits.contiguous(), vocab, k)
    if dev != "cpu":
        torch.cuda.synchronize()
        from llm_distillery_b200.ops import _lib
        assert _lib.take_device_error() == 0
    # compare as sparse distributions: probability mass per id
    full_lp = torch.log_softmax(logits[:, :vocab], -1)
    got = torch.gather(full_lp, 1, ix.long().to(full_lp.device))
    err = (got - lp.float().to(got.device)).abs().max().item()
    assert err < atol, ("tp log-probs vs unsharded log-softmax at the returned ids", err)
    top_ref = ref_lp.float()[:, -1]
    assert (lp.float()[:, -1].to(top_ref.device) - top_ref).abs().max().item() < atol, "K-th value differs"
    return err


def cpu_tp():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    _tp_model_check("cpu", torch.float32, rank, world, 16, 1e-2)
    if rank == 0:
        print("WORKER_OK")
    dist.destroy_process_group()


def _vp_head_check(dev, dtype, rank, world, atol):
    """Vocabulary-parallel head against the unsharded head on every rank: per-row loss, dH, this rank's dW rows."""
    from llm_distillery_b200.loss.head import fused_distill_rows, sort_teacher_rows
    from llm_distillery_b200.parallel.tp import TPGroup
    from llm_distillery_b200.parallel.vp_head import VocabParallelHead
    M, h, V, K = 256 * world, 256, 1000, 24
    g = torch.Generator().manual_seed(7)
    Hc = (torch.randn((M, h), generator=g) * 0.5).to(dtype).to(dev)
    W = (torch.randn((V + 24, h), generator=g) * 0.05).to(dtype).to(dev)
    ids = torch.stack([torch.randperm(V + 20, generator=g)[:K] for _ in range(M)]).to(torch.int32)   # some ids >= vocab
    u = torch.log_softmax(torch.randn((M, K), generator=g) * 2, -1)
    ids, u = sort_teacher_rows(ids, u)
    ids, u = ids.to(dev), u.to(dev)
    grp = TPGroup(dev, M, h, dtype=dtype)
    head = VocabParallelHead(grp, M, h, K, V)
    for kind, T in (("kl", 2.0), ("jsd", 1.0), ("rkl", 1.0)):
        Ws = torch.zeros((head.vl, h), dtype=dtype, device=dev)
        Ws[: head.valid] = W[head.lo: head.lo + head.valid]
        loss, dH, dW = head.loss_and_grads(Hc, Ws, ids, u, kind, T)
        Hr = Hc.detach().clone().requires_grad_(True)
        Wr = W.detach().clone().requires_grad_(True)
        ref = fused_distill_rows(Hr, Wr, ids, u, kind, T, vocab=V)
        ref.mean().backward()
        if dev != "cpu":
            torch.cuda.synchronize()
            from llm_distillery_b200.ops import _lib
            assert _lib.take_device_error() == 0
        e1 = (loss - ref.detach()).abs().max().item()
        e2 = (dH.float() - Hr.grad.float()).abs().max().item() / max(Hr.grad.float().abs().max().item(), 1e-12)
        wref = Wr.grad.float()[head.lo: head.lo + head.valid]
        e3 = (dW[: head.valid] - wref).abs().max().item() / max(wref.abs().max().item(), 1e-12)
        assert e1 < atol and e2 < 10 * atol and e3 < 10 * atol, (kind, e1, e2, e3)


def cpu_vp_head():
    dist.init_process_group("gloo")
    _vp_head_check("cpu", torch.float32, dist.get_rank(), dist.get_world_size(), 1e-4)
    if dist.get_rank() == 0:
        print("WORKER_OK")
    dist.destroy_process_group()


def cpu_vp_training():
    """Data-parallel training through the vocabulary-parallel head equals training through replicated heads."""
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    finals = {}
    for vp in (False, True):
        model, cfg = tiny(torch.float32, "cpu")
        comm = make_comm("gloo", "cpu", shard_strategy="ddp")
        eng = DistillEngine(model, loss="jsd", temperature=1.5, optimizer="adamw", lr=1e-3, comm=comm, crop_to_size=500,
                            vocab_parallel=vp, max_rows_per_rank=512)
        losses = []
        for s in range(3):
            # ranks get different numbers of rows (rank 1 has a shorter batch): the head pads to the step's maximum
            hb = synthetic_batch(cfg.vocab_size, 2, 128 if rank == 0 else 96, 16, seed=100 * s + rank)
            losses.append(float(eng.train_step([hb])))
        finals[vp] = (torch.cat([p.detach().float().reshape(-1) for p in model.parameters()]), losses)
    err = (finals[True][0] - finals[False][0]).abs().max().item()
    assert err < 5e-5, err
    assert all(abs(a - b) < 1e-3 * max(1.0, abs(b)) for a, b in zip(finals[True][1], finals[False][1])), finals
    if rank == 0:
        print("WORKER_OK")
    dist.destroy_process_group()


def cpu_rank_loss():
    """Rank 2 leaves between steps (no kernel or collective of its own in flight) without marking its record."""
    import datetime
    import time
    from llm_distillery_b200.obs.watchdog import Heartbeat, RankFailure
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=20))
    rank, world = dist.get_rank(), dist.get_world_size()
    hb = Heartbeat(os.path.join(sys.argv[2], "hb"), rank, world, interval=0.1, timeout=1.5)
    x = torch.ones(4)
    try:
        for step in range(200):
            hb.beat(step, "train")
            hb.check()
            if rank == 2 and step == 3:
                os._exit(0)
            try:
                dist.all_reduce(x)
            except RuntimeError as e:      # the collective ended with an error: ask the heartbeat who is gone
                deadline = time.time() + 5.0
                while time.time() < deadline and not hb.scan():
                    time.sleep(0.1)
                hb.check()
                raise e
            time.sleep(0.05)
        raise AssertionError("the lost rank was never noticed")
    except RankFailure as e:
        assert e.ranks == [2], e
        print(f"SURVIVOR_OK rank {rank}: {e}", flush=True)
        hb.close("done")
        os._exit(0)


def cpu_cli_tp():
    """The whole pipeline under two gloo ranks with a tensor-parallel teacher (tp_size = 2): what lands in the HDF5
    store equals a single-process collection of the same teacher."""
    import json
    import numpy as np
    from llm_distillery_b200 import cli
    from llm_distillery_b200.data.h5store import H5Store
    from llm_distillery_b200.models.llama import preset
    from llm_distillery_b200.utils import synthetic
    root = sys.argv[2]
    rank = int(os.environ["RANK"])
    conf = {"cache_folder": os.path.join(root, "cache"), "dataset_path": os.path.join(root, "train.jsonl"),
            "validation_dataset_path": os.path.join(root, "val.jsonl"), "teacher_models_folder": os.path.join(root, "teachers"),
            "student_path": os.path.join(root, "student"), "context_len": 96, "crop_distr_to_size": 400, "save_topK": 20,
            "enable_topK": True, "device": "cpu", "num_epochs": 1, "num_warmup_steps": 2, "batch_size": 2,
            "grad_accum_batches": 1, "temperature": 1.0, "lr": 1e-3, "optimizer": "adamw", "data_order": "sorted",
            "training_precision": "fp32", "validate_every_n_epochs": 1, "save_student_every_n_epochs": 1,
            "freeze_layers": [], "loss": "kl", "max_cache_size_gb": 320, "tp_size": 2}
    if rank == 0:
        tok = os.path.join(root, "tok")
        synthetic.make_tokenizer(tok, 400)
        tcfg = preset("plumbing-teacher", vocab_size=512, hidden_size=64, intermediate_size=176, max_position_embeddings=512)
        scfg = preset("plumbing-student", vocab_size=512, hidden_size=64, intermediate_size=176, max_position_embeddings=512)
        synthetic.make_model_dir(os.path.join(root, "teachers", "teacher_a"), tcfg, tok, seed=1, batch_size=4)
        synthetic.make_model_dir(os.path.join(root, "student"), scfg, tok, seed=2)
        synthetic.make_dataset(os.path.join(root, "train.jsonl"), 10, seed=3)
        synthetic.make_dataset(os.path.join(root, "val.jsonl"), 4, seed=4)
        with open(os.path.join(root, "config.json"), "w") as f:
            json.dump(conf, f)
    dist.init_process_group("gloo")
    dist.barrier()
    out = cli.main(["--config", os.path.join(root, "config.json")])
    assert out["trained_samples"] == 10, out
    if rank == 0:
        # single-process collection of the same data into another cache folder
        os.environ["WORLD_SIZE"] = "1"
        conf1 = dict(conf, cache_folder=os.path.join(root, "cache1"), tp_size=1)
        with open(os.path.join(root, "config1.json"), "w") as f:
            json.dump(conf1, f)
        cli.main(["--config", os.path.join(root, "config1.json")])
        a = H5Store(os.path.join(root, "cache", "dataset"))
        b = H5Store(os.path.join(root, "cache1", "dataset"))
        ids = a.get_dataset_ids()
        assert sorted(ids) == sorted(b.get_dataset_ids()) and len(ids) == 10
        for cid in ids:
            va, ia = a.load_id(cid)
            vb, ib = b.load_id(cid)
            assert va.shape == vb.shape and a.get_sha(cid) == b.get_sha(cid)
            assert np.abs(va.astype(np.float32) - vb.astype(np.float32)).max() < 2e-2
            assert (ia == ib).mean() > 0.97      # near-ties may swap under another summation order
        print("WORKER_OK")


def _cli_zero3(device: str, precision: str, tol: float, tp: int, hidden: int, ffn: int, extra: dict | None = None):
    """The command-line pipeline under two ranks, student trained once replicated and once fully sharded: five
    batches over two ranks, so the last step has a rank without a micro-batch; the saved students are equal."""
    import json
    from llm_distillery_b200 import cli
    from llm_distillery_b200.ckpt.hf import load_hf_state_dict
    from llm_distillery_b200.models.llama import preset
    from llm_distillery_b200.utils import synthetic
    root = sys.argv[2]
    rank = int(os.environ["RANK"])
    conf = {"dataset_path": os.path.join(root, "train.jsonl"),
            "validation_dataset_path": os.path.join(root, "val.jsonl"), "teacher_models_folder": os.path.join(root, "teachers"),
            "student_path": os.path.join(root, "student"), "context_len": 96, "crop_distr_to_size": 400, "save_topK": 20,
            "enable_topK": True, "device": device, "num_epochs": 2, "num_warmup_steps": 2, "batch_size": 2,
            "grad_accum_batches": 1, "temperature": 1.0, "lr": 1e-3, "optimizer": "adamw", "data_order": "sorted",
            "training_precision": precision, "validate_every_n_epochs": 1, "save_student_every_n_epochs": 1,
            "freeze_layers": [], "loss": "kl", "max_cache_size_gb": 320, "tp_size": tp, "save_final_state": True}
    conf.update(extra or {})
    os.environ["B200_TRACE"] = "1"          # phase timers on: the per-rank skew figures are gathered and logged
    if rank == 0:
        tok = os.path.join(root, "tok")
        synthetic.make_tokenizer(tok, 400)
        kw = dict(vocab_size=512, hidden_size=hidden, intermediate_size=ffn, max_position_embeddings=512)
        synthetic.make_model_dir(os.path.join(root, "teachers", "teacher_a"), preset("plumbing-teacher", **kw), tok, seed=1,
                                 batch_size=4)
        synthetic.make_model_dir(os.path.join(root, "student"), preset("plumbing-student", **kw), tok, seed=2)
        synthetic.make_dataset(os.path.join(root, "train.jsonl"), 10, seed=3)
        synthetic.make_dataset(os.path.join(root, "val.jsonl"), 4, seed=4)
        for strat in ("ddp", "zero3"):
            with open(os.path.join(root, f"config_{strat}.json"), "w") as f:
                json.dump(dict(conf, cache_folder=os.path.join(root, f"cache_{strat}"), shard_strategy=strat), f)
    if device == "cpu":
        dist.init_process_group("gloo")
    else:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dist.barrier()
    finals = {}
    for strat in ("ddp", "zero3"):
        out = cli.main(["--config", os.path.join(root, f"config_{strat}.json")])
        assert out["trained_samples"] == 20, out
        dist.barrier()
        if rank == 0:
            base = os.path.join(root, f"cache_{strat}", "student", "trained")
            final = [d for d in os.listdir(base) if d.endswith("final")]
            assert len(final) == 1, os.listdir(base)
            finals[strat] = load_hf_state_dict(os.path.join(base, final[0]))
            with open(os.path.join(root, f"cache_{strat}", "metrics.jsonl")) as f:
                logged = [json.loads(line) for line in f if line.strip()]
            assert any("Perf/rank skew ms" in rec for rec in logged), logged[:3]
            with open(os.path.join(root, f"cache_{strat}", "student", "states", "trainer_state.json")) as f:
                st = json.load(f)
            assert len(st["config_hash"]) == 16 and "rng_state" in st and st["world"] == int(os.environ["WORLD_SIZE"])
    if device != "cpu":
        from llm_distillery_b200.ops import _lib
        torch.cuda.synchronize()
        assert _lib.take_device_error() == 0
    if rank == 0:
        init = load_hf_state_dict(os.path.join(root, "student"))
        moved = 0.0
        for k, v in finals["ddp"].items():
            err = (v.float() - finals["zero3"][k].float()).abs().max().item()
            assert err < tol, (k, err)
            assert torch.isfinite(v.float()).all(), k
            moved = max(moved, (v.float() - init[k].float()).abs().max().item())
        assert moved > 1e-4, "training did not change the student"
        print("WORKER_OK")


def cpu_cli_zero3():
    _cli_zero3("cpu", "fp32", 1e-5, tp=2, hidden=64, ffn=176)


def cpu_cli_zero3_three():
    """Three ranks, five batches per epoch: the last step of an epoch has one rank without a batch."""
    _cli_zero3("cpu", "fp32", 1e-5, tp=1, hidden=64, ffn=176)


def cpu_cli_zero3_accum():
    """Gradient accumulation whose step size (batch 2 x 2 micro-batches x 2 ranks = 8 samples) does not divide the ten
    samples of an epoch: steps straddle epochs and the run ends with a partial step."""
    _cli_zero3("cpu", "fp32", 1e-5, tp=1, hidden=64, ffn=176, extra={"grad_accum_batches": 2})


def cpu_cli_zero3_variants():
    """Gradient checkpointing (the layer is recomputed from gathered weights in backward), shuffled data order, the
    reference's weighted loss, a frozen layer and an 8-bit optimizer name, replicated against fully sharded."""
    _cli_zero3("cpu", "fp32", 1e-5, tp=1, hidden=64, ffn=176,
               extra={"grad_checkpointing": True, "data_order": "shuffle", "loss": "reference", "temperature": 2.0,
                      "freeze_layers": ["layers.1."], "optimizer": os.environ.get("Z3_OPT", "adamw")})


def cpu_cli_zero3_chunked():
    """The cache holds only part of the data at a time: collect a chunk, train on it, save the trainer state, next chunk
    (state loaded back) - replicated against fully sharded, whose state goes through the gathered view each time."""
    _cli_zero3("cpu", "fp32", 1e-5, tp=1, hidden=64, ffn=176, extra={"max_cache_size_gb": 0.00002})


def cpu_cli_resume():
    """A fully sharded two-rank run stops after one epoch with its trainer state saved; the same command asking for two
    epochs picks the state up (weights through the gathered view, per-rank optimizer pieces, counters) and ends where
    an uninterrupted two-epoch run ends."""
    import json
    from llm_distillery_b200 import cli
    from llm_distillery_b200.ckpt.hf import load_hf_state_dict
    from llm_distillery_b200.models.llama import preset
    from llm_distillery_b200.utils import synthetic
    root = sys.argv[2]
    rank = int(os.environ["RANK"])
    conf = {"dataset_path": os.path.join(root, "train.jsonl"), "validation_dataset_path": os.path.join(root, "val.jsonl"),
            "teacher_models_folder": os.path.join(root, "teachers"), "student_path": os.path.join(root, "student"),
            "context_len": 96, "crop_distr_to_size": 400, "save_topK": 20, "enable_topK": True, "device": "cpu",
            "num_epochs": 1, "num_warmup_steps": 0, "lr_scheduler": "constant", "batch_size": 2, "grad_accum_batches": 1,
            "temperature": 1.0, "lr": 1e-3, "optimizer": "adamw", "data_order": "sorted", "training_precision": "fp32",
            "freeze_layers": [], "loss": "kl", "max_cache_size_gb": 320, "shard_strategy": "zero3", "save_final_state": True}
    if rank == 0:
        tok = os.path.join(root, "tok")
        synthetic.make_tokenizer(tok, 400)
        kw = dict(vocab_size=512, hidden_size=64, intermediate_size=176, max_position_embeddings=512)
        synthetic.make_model_dir(os.path.join(root, "teachers", "teacher_a"), preset("plumbing-teacher", **kw), tok, seed=1,
                                 batch_size=4)
        synthetic.make_model_dir(os.path.join(root, "student"), preset("plumbing-student", **kw), tok, seed=2)
        synthetic.make_dataset(os.path.join(root, "train.jsonl"), 8, seed=3)
        synthetic.make_dataset(os.path.join(root, "val.jsonl"), 4, seed=4)
        for name, extra in (("stop", {"cache_folder": os.path.join(root, "cache_a")}),
                            ("go_on", {"cache_folder": os.path.join(root, "cache_a"), "num_epochs": 2}),
                            ("whole", {"cache_folder": os.path.join(root, "cache_b"), "num_epochs": 2})):
            with open(os.path.join(root, f"config_{name}.json"), "w") as f:
                json.dump(dict(conf, **extra), f)
    dist.init_process_group("gloo")
    dist.barrier()

    def final(cache):
        base = os.path.join(root, cache, "student", "trained")
        names = [d for d in os.listdir(base) if d.endswith("final")]
        return {k: v.clone() for k, v in load_hf_state_dict(os.path.join(base, names[0])).items()}
    out = cli.main(["--config", os.path.join(root, "config_stop.json")])
    assert out["trained_samples"] == 8, out
    dist.barrier()
    first = final("cache_a") if rank == 0 else None
    out = cli.main(["--config", os.path.join(root, "config_go_on.json")])
    assert out["trained_samples"] == 16 and out["tokens_collected"] == 0, out      # nothing collected again; 8 more trained
    dist.barrier()
    resumed = final("cache_a") if rank == 0 else None
    out = cli.main(["--config", os.path.join(root, "config_whole.json")])
    assert out["trained_samples"] == 16, out
    dist.barrier()
    if rank == 0:
        whole = final("cache_b")
        for k, v in whole.items():
            err = (v.float() - resumed[k].float()).abs().max().item()
            assert err < 1e-5, (k, err)
        moved = max((first[k].float() - resumed[k].float()).abs().max().item() for k in first)
        assert moved > 1e-4, ("the second epoch changed nothing", moved)
        print("WORKER_OK")


def cpu_cli_sync():
    """The dataset changes between two runs on two ranks: two conversations are dropped, the rest is reordered, three
    new ones arrive. The second run collects only the new ones, renames / removes the old entries by their content
    SHA, and the store ends up equal to a fresh collection of the new dataset."""
    import json
    import numpy as np
    from llm_distillery_b200 import cli
    from llm_distillery_b200.data.h5store import H5Store
    from llm_distillery_b200.models.llama import preset
    from llm_distillery_b200.utils import synthetic
    root = sys.argv[2]
    rank = int(os.environ["RANK"])
    conf = {"dataset_path": os.path.join(root, "train.jsonl"), "validation_dataset_path": os.path.join(root, "val.jsonl"),
            "teacher_models_folder": os.path.join(root, "teachers"), "student_path": os.path.join(root, "student"),
            "context_len": 96, "crop_distr_to_size": 400, "save_topK": 20, "enable_topK": True, "device": "cpu",
            "num_epochs": 1, "num_warmup_steps": 0, "batch_size": 2, "grad_accum_batches": 1, "lr": 1e-3,
            "optimizer": "adamw", "data_order": "sorted", "training_precision": "fp32", "freeze_layers": [], "loss": "kl",
            "max_cache_size_gb": 320, "cache_folder": os.path.join(root, "cache")}
    if rank == 0:
        tok = os.path.join(root, "tok")
        synthetic.make_tokenizer(tok, 400)
        kw = dict(vocab_size=512, hidden_size=64, intermediate_size=176, max_position_embeddings=512)
        synthetic.make_model_dir(os.path.join(root, "teachers", "teacher_a"), preset("plumbing-teacher", **kw), tok, seed=1,
                                 batch_size=4)
        synthetic.make_model_dir(os.path.join(root, "student"), preset("plumbing-student", **kw), tok, seed=2)
        rows = synthetic.make_dataset(os.path.join(root, "all.jsonl"), 12, seed=3)
        synthetic.make_dataset(os.path.join(root, "val.jsonl"), 4, seed=4)
        with open(os.path.join(root, "train.jsonl"), "w", encoding="utf-8") as f:
            for r in rows[:9]:
                f.write(json.dumps(r, ensure_ascii=False) + "\n")
        with open(os.path.join(root, "config.json"), "w") as f:
            json.dump(conf, f)
        with open(os.path.join(root, "config_fresh.json"), "w") as f:
            json.dump(dict(conf, cache_folder=os.path.join(root, "cache_fresh")), f)
    dist.init_process_group("gloo")
    dist.barrier()
    out = cli.main(["--config", os.path.join(root, "config.json")])
    def total(n):           # tokens collected by all ranks together
        t = torch.tensor([float(n)])
        dist.all_reduce(t)
        return float(t.item())
    first_tokens = total(out["tokens_collected"])
    assert out["trained_samples"] == 9 and first_tokens > 0
    dist.barrier()
    if rank == 0:
        rows = [json.loads(line) for line in open(os.path.join(root, "all.jsonl"), encoding="utf-8")]
        new = [rows[7], rows[9], rows[0], rows[10], rows[3], rows[4], rows[11], rows[5], rows[8], rows[6]]   # 1, 2 dropped
        with open(os.path.join(root, "train.jsonl"), "w", encoding="utf-8") as f:
            for r in new:
                f.write(json.dumps(r, ensure_ascii=False) + "\n")
    dist.barrier()
    out = cli.main(["--config", os.path.join(root, "config.json")])
    assert out["trained_samples"] == 10, out
    again = total(out["tokens_collected"])
    assert 0 < again < 0.6 * first_tokens, (again, first_tokens)                 # three conversations of ten
    dist.barrier()
    if rank == 0:
        os.environ["WORLD_SIZE"] = "1"
        cli.main(["--config", os.path.join(root, "config_fresh.json")])
        a, b = H5Store(os.path.join(root, "cache", "dataset")), H5Store(os.path.join(root, "cache_fresh", "dataset"))
        assert sorted(a.get_dataset_ids()) == sorted(b.get_dataset_ids()) == list(range(10))
        for cid in range(10):
            assert a.get_sha(cid) == b.get_sha(cid), cid
            va, ia = a.load_id(cid)
            vb, ib = b.load_id(cid)
            assert va.shape == vb.shape and np.abs(va - vb).max() < 2e-2 and (ia == ib).mean() > 0.97
        print("WORKER_OK")


def cpu_cli_rank_loss():
    """The command line on two ranks; rank 1's process ends right after its second optimizer step. Rank 0 meets the loss
    as a failed collective, asks the heartbeats, saves what it can without a peer and leaves with status 3."""
    import datetime
    import json
    from llm_distillery_b200 import cli
    from llm_distillery_b200.models.llama import preset
    from llm_distillery_b200.models.student import StudentModel
    from llm_distillery_b200.utils import synthetic
    root = sys.argv[2]
    rank = int(os.environ["RANK"])
    conf = {"dataset_path": os.path.join(root, "train.jsonl"), "validation_dataset_path": os.path.join(root, "val.jsonl"),
            "teacher_models_folder": os.path.join(root, "teachers"), "student_path": os.path.join(root, "student"),
            "context_len": 96, "crop_distr_to_size": 400, "save_topK": 20, "enable_topK": True, "device": "cpu",
            "num_epochs": 2, "num_warmup_steps": 0, "batch_size": 2, "grad_accum_batches": 1, "lr": 1e-3,
            "optimizer": "adamw", "data_order": "sorted", "training_precision": "fp32", "freeze_layers": [], "loss": "kl",
            "max_cache_size_gb": 320, "cache_folder": os.path.join(root, os.environ.get("RL_CACHE", "cache")),
            "shard_strategy": os.environ.get("RL_STRATEGY", "ddp")}
    if rank == 0:
        tok = os.path.join(root, "tok")
        synthetic.make_tokenizer(tok, 400)
        kw = dict(vocab_size=512, hidden_size=64, intermediate_size=176, max_position_embeddings=512)
        synthetic.make_model_dir(os.path.join(root, "teachers", "teacher_a"), preset("plumbing-teacher", **kw), tok, seed=1,
                                 batch_size=4)
        synthetic.make_model_dir(os.path.join(root, "student"), preset("plumbing-student", **kw), tok, seed=2)
        synthetic.make_dataset(os.path.join(root, "train.jsonl"), 8, seed=3)
        synthetic.make_dataset(os.path.join(root, "val.jsonl"), 2, seed=4)
    if rank == 0:
        with open(os.path.join(root, "config.json"), "w") as f:
            json.dump(conf, f)
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=20))
    dist.barrier()
    real, count = StudentModel._optimizer_step, [0]

    def step(self):
        real(self)
        count[0] += 1
        if rank == 1 and count[0] == int(os.environ.get("RL_AT", "2")) and os.environ.get("RL_LEAVE", "1") == "1":   # between two steps: nothing in flight
            if os.environ.get("RL_MODE") == "stop":      # a stop request that reaches only this rank (yet)
                import signal
                cli.handle_termination(signal.SIGTERM, None)
                return
            print("RANK 1 LEAVES", flush=True)
            os._exit(0)
    StudentModel._optimizer_step = step
    out = cli.main(["--config", os.path.join(root, "config.json")])
    if os.environ.get("RL_MODE") == "stop" and os.environ.get("RL_LEAVE", "1") == "1":
        assert out == {"stopped": True, "trained_samples": 4 * int(os.environ.get("RL_AT", "2"))}, out
        dist.barrier()
        if rank == 0:
            print("WORKER_OK")
        return
    if os.environ.get("RL_LEAVE", "1") == "1":
        print(f"rank {rank} finished the run although its peer left", flush=True)
    else:
        assert out["trained_samples"] == 16, out
        if "RL_CACHE" not in os.environ:
            assert out["tokens_collected"] == 0, out                                  # the cache is reused as it is
        if rank == 0:
            print("WORKER_OK")


def cpu_cli_config3():
    """The multi-teacher cross-tokenizer configuration in small: two teachers, one with another tokenizer (mapped onto the
    student vocabulary through the byte trie), a student with tied embeddings trained with JSD on the merged targets,
    fully sharded over two gloo ranks; tensor-parallel width and sharding both left to the planner. The result equals
    the single-process run of the same configuration."""
    import json
    import numpy as np
    from llm_distillery_b200 import cli
    from llm_distillery_b200.ckpt.hf import load_hf_state_dict
    from llm_distillery_b200.data.h5store import H5Store
    from llm_distillery_b200.models.llama import preset
    from llm_distillery_b200.utils import synthetic
    root = sys.argv[2]
    rank = int(os.environ["RANK"])
    if rank == 0:
        synthetic.make_tokenizer(os.path.join(root, "tok_a"), 400, seed=0)
        synthetic.make_tokenizer(os.path.join(root, "tok_b"), 700, seed=5, extra_merges_text="quartz sphinx wizard " * 50)
        kw = dict(hidden_size=64, intermediate_size=176, max_position_embeddings=128)
        synthetic.make_model_dir(os.path.join(root, "teachers", "t_same"), preset("plumbing-teacher", vocab_size=512, **kw),
                                 os.path.join(root, "tok_a"), seed=1, batch_size=4, add_bos=False)
        synthetic.make_model_dir(os.path.join(root, "teachers", "t_other"), preset("plumbing-teacher", vocab_size=768, **kw),
                                 os.path.join(root, "tok_b"), seed=2, batch_size=4, add_bos=False)
        synthetic.make_model_dir(os.path.join(root, "student"),
                                 preset("plumbing-student", vocab_size=512, num_hidden_layers=3, tie_word_embeddings=True, **kw),
                                 os.path.join(root, "tok_a"), seed=3)
        synthetic.make_dataset(os.path.join(root, "train.jsonl"), 9, seed=3)
        synthetic.make_dataset(os.path.join(root, "val.jsonl"), 3, seed=4)
        conf = {"dataset_path": os.path.join(root, "train.jsonl"), "validation_dataset_path": os.path.join(root, "val.jsonl"),
                "teacher_models_folder": os.path.join(root, "teachers"), "student_path": os.path.join(root, "student"),
                "context_len": 96, "crop_distr_to_size": 400, "save_topK": 16, "device": "cpu", "num_epochs": 2,
                "batch_size": 2, "grad_accum_batches": 2, "lr": 1e-3, "optimizer": "adamw", "training_precision": "fp32",
                "freeze_layers": [], "loss": "jsd", "cross_tokenizer": True, "data_order": "sorted", "tp_size": int(os.environ.get("C3_TP", "0"))}
        for name, extra in (("sharded", {"shard_strategy": "zero3"}), ("auto", {"shard_strategy": "auto"}), ("single", {})):
            with open(os.path.join(root, f"config_{name}.json"), "w") as f:
                json.dump(dict(conf, cache_folder=os.path.join(root, f"cache_{name}"), **extra), f)
    dist.init_process_group("gloo")
    dist.barrier()
    finals = {}
    for name in ("sharded", "auto"):
        out = cli.main(["--config", os.path.join(root, f"config_{name}.json")])
        assert out["trained_samples"] == 18, out
        dist.barrier()
        if rank == 0:
            base = os.path.join(root, f"cache_{name}", "student", "trained")
            final = [d for d in os.listdir(base) if d.endswith("final")]
            finals[name] = load_hf_state_dict(os.path.join(base, final[0]))
    if rank == 0:
        os.environ["WORLD_SIZE"] = "1"
        out = cli.main(["--config", os.path.join(root, "config_single.json")])
        assert out["trained_samples"] == 18
        base = os.path.join(root, "cache_single", "student", "trained")
        single = load_hf_state_dict(os.path.join(base, [d for d in os.listdir(base) if d.endswith("final")][0]))
        assert "lm_head.weight" not in single                       # tied embeddings stay tied in the checkpoint
        for k, v in single.items():
            # same data, same schedule; one process sums the two batches of a step in another order than two ranks do,
            # and AdamW turns a last-bit difference of a near-zero gradient into a visible one (lr = 1e-3)
            for name, sd in finals.items():
                err = (v.float() - sd[k].float()).abs().max().item()
                assert err < 3e-4, (name, k, err)
            err = (finals["sharded"][k].float() - finals["auto"][k].float()).abs().max().item()
            assert err < 2e-5, ("sharded vs planner-chosen", k, err)
        a, b = H5Store(os.path.join(root, "cache_sharded", "dataset")), H5Store(os.path.join(root, "cache_single", "dataset"))
        assert sorted(a.get_dataset_ids()) == sorted(b.get_dataset_ids()) and len(a.get_dataset_ids()) == 9
        for cid in a.get_dataset_ids():
            va, ia = a.load_id(cid)
            vb, ib = b.load_id(cid)
            assert va.shape == vb.shape and ia.max() < 400
            fin = np.isfinite(va) & np.isfinite(vb)
            assert (np.isfinite(va) == np.isfinite(vb)).all() and np.abs(va[fin] - vb[fin]).max() < 2e-2
            mass = np.exp(va).sum(-1)
            assert (mass <= 2.0 + 1e-2).all()                       # two teachers' probabilities summed, never more
        print("WORKER_OK")


def gpu_cli_zero3():
    """Same on two GPUs in bf16: data-parallel collection replicas, NVLink data parallelism / full sharding."""
    _cli_zero3("cuda", "bf16", 3e-2, tp=1, hidden=256, ffn=688)


def gpu_tp():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from llm_distillery_b200.ops import _lib
    from llm_distillery_b200.parallel.tp import TPGroup
    T, h, n_col, k_row = 512 * world, 512, 768, 640
    grp = TPGroup(dev, T, h)
    Ts = T // world
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    for it in range(3):
        x_shard = torch.randn((Ts, h), device=dev, generator=gen).to(torch.bfloat16)
        w_col = (torch.randn((n_col, h), device=dev, generator=gen) * 0.05).to(torch.bfloat16)
        grp.slab(T, h).copy_(x_shard)
        y = grp.ag_gemm(w_col, T)
        parts = [torch.empty_like(x_shard) for _ in range(world)]
        dist.all_gather(parts, x_shard)
        ref = (torch.cat(parts).float() @ w_col.float().t())
        torch.cuda.synchronize()
        assert _lib.take_device_error() == 0
        err = (y.float() - ref).abs().max().item()
        assert err < 0.06, ("ag_gemm", it, err)
        grp.slab(T, h).copy_(x_shard)
        y32 = grp.ag_gemm(w_col, T, out_f32=True)
        assert (y32 - ref).abs().max().item() < 2e-3, "ag_gemm fp32 output"
        xa = torch.randn((T, k_row), device=dev, generator=gen).to(torch.bfloat16)
        w_row = (torch.randn((h, k_row), device=dev, generator=gen) * 0.05).to(torch.bfloat16)
        res = torch.randn((Ts, h), device=dev, generator=gen).to(torch.bfloat16)
        out = grp.gemm_rs(xa, w_row, residual=res)
        # every rank's partial is rounded to bf16 before the sum, like the kernel's staging
        part = (xa.float() @ w_row.float().t()).to(torch.bfloat16).float()
        dist.all_reduce(part)
        ref2 = part[rank * Ts:(rank + 1) * Ts] + res.float()
        torch.cuda.synchronize()
        assert _lib.take_device_error() == 0
        err2 = (out.float() - ref2).abs().max().item()
        assert err2 < 0.08, ("gemm_rs", it, err2)
    del grp
    _tp_model_check(dev, torch.bfloat16, rank, world, 32, 0.05)
    _vp_head_check(dev, torch.bfloat16, rank, world, 5e-3)
    if rank == 0:
        print("WORKER_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    {"cpu_engine": cpu_engine, "gpu_p2p": gpu_p2p, "cpu_tp": cpu_tp, "gpu_tp": gpu_tp, "cpu_cli_tp": cpu_cli_tp,
     "cpu_vp_head": cpu_vp_head, "cpu_vp_training": cpu_vp_training, "cpu_rank_loss": cpu_rank_loss, "cpu_zero3": cpu_zero3, "gpu_zero3": gpu_zero3,
     "cpu_cli_zero3": cpu_cli_zero3, "gpu_cli_zero3": gpu_cli_zero3, "cpu_cli_config3": cpu_cli_config3,
     "cpu_cli_zero3_chunked": cpu_cli_zero3_chunked, "cpu_cli_resume": cpu_cli_resume, "cpu_cli_zero3_three": cpu_cli_zero3_three,
     "cpu_cli_zero3_accum": cpu_cli_zero3_accum, "cpu_cli_zero3_variants": cpu_cli_zero3_variants,
     "cpu_cli_sync": cpu_cli_sync, "cpu_cli_rank_loss": cpu_cli_rank_loss}[sys.argv[1]]()
