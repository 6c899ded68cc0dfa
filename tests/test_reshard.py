"""Trainer state saved under one world size resumes under another: the per-rank optimizer slices are re-cut."""
import torch

from llm_distillery_b200.ckpt import hf as ckpt
from llm_distillery_b200.engine.optim import FlatOptimizer, FlatParams
from llm_distillery_b200.models.llama import LlamaConfig, build_model

CFG = LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=136, num_hidden_layers=2, num_attention_heads=2,
                  num_key_value_heads=1, max_position_embeddings=64)


def _rank(rank, world, steps, seed=3):
    model = build_model(CFG, dtype=torch.float32, device="cpu", seed=1)
    flat = FlatParams([p for p in model.parameters()], shard=(rank, world))
    opt = FlatOptimizer(flat, "adamw", lr=1e-2)
    g = torch.Generator().manual_seed(seed)
    for _ in range(steps):
        flat.grad.copy_(torch.randn(flat.grad.shape, generator=g)[: flat.total] if flat.grad.numel() == flat.total else 0)
        opt.step(1e-2, grad_scale=1.0)
    return model, flat, opt


def _full(flat_opts, key):
    parts = [(o.flat.master if key == "master" else o.state[key]) for o in flat_opts]
    return torch.cat(parts)


def test_two_rank_state_loads_into_one_rank_and_back(tmp_path):
    world = 2
    ranks = []
    for r in range(world):
        model, flat, opt = _rank(r, world, steps=3)
        ranks.append((model, flat, opt))
    # every rank holds the same weights after the all-gather a real step would do: emulate it
    full_master = torch.cat([o.flat.master for _, _, o in ranks])
    for model, flat, opt in ranks:
        flat.model.copy_(full_master[: flat.total].to(flat.dtype))
    d = str(tmp_path / "states")
    for model, flat, opt in ranks:
        ckpt.save_trainer_state(d, model, opt, None, {"num_trained_steps": 7})
    # ---- 2 -> 1
    m1 = build_model(CFG, dtype=torch.float32, device="cpu", seed=99)
    f1 = FlatParams([p for p in m1.parameters()], shard=(0, 1))
    o1 = FlatOptimizer(f1, "adamw", lr=1e-2)
    counters = ckpt.load_trainer_state(d, m1, o1, None)
    assert counters["num_trained_steps"] == 7 and o1.step_count == 3
    n = min(f1.total, full_master.numel())
    assert torch.equal(o1.flat.master[:n], full_master[:n])
    for k in ("m", "v"):
        assert torch.equal(o1.state[k][:n], torch.cat([o.state[k] for _, _, o in ranks])[:n])
    # ---- 1 -> 4
    d1 = str(tmp_path / "states1")
    ckpt.save_trainer_state(d1, m1, o1, None, {"num_trained_steps": 9})
    for r in range(4):
        m4 = build_model(CFG, dtype=torch.float32, device="cpu", seed=5)
        f4 = FlatParams([p for p in m4.parameters()], shard=(r, 4))
        o4 = FlatOptimizer(f4, "adamw", lr=1e-2)
        ckpt.load_trainer_state(d1, m4, o4, None)
        lo, hi = f4.shard_lo, min(f4.shard_lo + f4.shard_size, f1.total)
        if hi > lo:
            assert torch.equal(o4.flat.master[: hi - lo], o1.flat.master[lo:hi])
            assert torch.equal(o4.state["v"][: hi - lo], o1.state["v"][lo:hi])
        assert o4.step_count == 3


def test_block_quantised_state_is_not_cut(tmp_path):
    model, flat, opt = _rank(0, 1, steps=1)
    shards = [{"name": "adamw8bit", "step_count": 1, "master": flat.master, "state": {"m": torch.zeros(10, dtype=torch.uint8)},
               "shard": (0, 1), "total": flat.total}]
    assert ckpt.reshard_optimizer_state(shards, opt) is False


def _zero3_rank(rank, world, steps, seed_model=1):
    from llm_distillery_b200.parallel.fsdp import ShardedFlat
    model = build_model(CFG, dtype=torch.float32, device="cpu", seed=seed_model)
    flat = ShardedFlat(model, rank, world)
    opt = FlatOptimizer(flat, "adamw", lr=1e-2)
    for s in range(steps):
        # the same whole-unit gradient on every rank, of which each rank sees its pieces
        for u in flat.units:
            g = torch.Generator().manual_seed(1000 * s + u.index)
            full = torch.randn(u.payload, generator=g)
            full = torch.cat([full, torch.zeros(u.numel - u.payload)])
            flat.grad_piece_of(u).copy_(full[rank * u.piece:(rank + 1) * u.piece])
        opt.step(1e-2, grad_scale=1.0)
    return model, flat, opt


def _units_full(ranks, key):
    """{unit name: the unit's values without padding}, put together from every rank's pieces."""
    out = {}
    flat0 = ranks[0][1]
    for u in flat0.units:
        parts = []
        for _, flat, opt in ranks:
            t = flat.master if key == "master" else opt.state[key]
            uu = flat.units[u.index]
            parts.append(t[uu.shard_lo:uu.shard_lo + uu.piece])
        out[u.name] = torch.cat(parts)[:u.payload]
    return out


def test_fully_sharded_state_is_recut_for_another_world_size(tmp_path):
    old = [_zero3_rank(r, 2, steps=3) for r in range(2)]
    d = str(tmp_path / "states")
    for model, flat, opt in old:
        ckpt.save_trainer_state(d, None, opt, None, {"num_trained_steps": 5})
    want = {k: _units_full(old, k) for k in ("master", "m", "v")}
    for world in (3, 1):
        new = []
        for r in range(world):
            from llm_distillery_b200.parallel.fsdp import ShardedFlat
            model = build_model(CFG, dtype=torch.float32, device="cpu", seed=42)
            flat = ShardedFlat(model, r, world)
            opt = FlatOptimizer(flat, "adamw", lr=1e-2)
            counters = ckpt.load_trainer_state(d, None, opt, None)
            assert counters["num_trained_steps"] == 5 and opt.step_count == 3
            assert torch.equal(flat.model_shard(), flat.master.to(flat.dtype))
            new.append((model, flat, opt))
        for k in ("master", "m", "v"):
            got = _units_full(new, k)
            for name, t in want[k].items():
                assert torch.equal(got[name], t), (world, k, name)
    # a contiguous (ZeRO-1) engine does not take the per-unit state: its moments restart from the loaded weights
    m1 = build_model(CFG, dtype=torch.float32, device="cpu", seed=1)
    o1 = FlatOptimizer(FlatParams(list(m1.parameters()), shard=(0, 1)), "adamw", lr=1e-2)
    ckpt.load_trainer_state(d, None, o1, None)
    assert o1.step_count == 0 and float(o1.state["m"].abs().max()) == 0.0
