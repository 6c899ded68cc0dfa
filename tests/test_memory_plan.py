"""Memory planner: the closed-form footprints sit just below what the benchmark runs measured on B200s (the gap is
context, allocator slack and library workspaces - the planner's headroom), and the recommendation moves from
replicated weights to full sharding to gradient checkpointing as models grow."""
import pytest

from llm_distillery_b200.models.llama import preset
from llm_distillery_b200.parallel import memory

# (model, ranks, strategy, tokens per rank, top-K, device memory in use at the end of the benchmark run, GB)
MEASURED = [("llama-3-8b", 8, "zero3", 8192, 128, 67.45), ("llama-3-8b", 2, "zero3", 8192, 128, 118.6),
            ("tinyllama-1.1b", 2, "zero3", 16384, 200, 35.5), ("tinyllama-1.1b", 2, "ddp", 16384, 200, 37.2),
            ("tinyllama-1.1b", 1, "ddp", 16384, 200, 42.3), ("llama-3.2-1b", 2, "zero3", 16384, 200, 36.1),
            ("llama-3.2-1b", 2, "ddp", 16384, 200, 39.1)]


@pytest.mark.parametrize("model,world,strategy,tokens,topk,measured", MEASURED)
def test_estimate_is_close_below_the_measured_footprint(model, world, strategy, tokens, topk, measured):
    fp = memory.estimate(preset(model), world, strategy, tokens, topk=topk)
    assert fp.total_gb <= measured + 0.5
    assert measured - fp.total_gb <= memory.HEADROOM_GB


def test_sharding_shrinks_what_it_says_it_shrinks():
    cfg = preset("llama-3-8b")
    ddp_nccl = memory.estimate(cfg, 8, "ddp", 8192, comm="nccl")
    ddp = memory.estimate(cfg, 8, "ddp", 8192)
    z1 = memory.estimate(cfg, 8, "fsdp", 8192, comm="nccl")
    z3 = memory.estimate(cfg, 8, "zero3", 8192)
    assert ddp_nccl.optimizer_gb == pytest.approx(8 * ddp.optimizer_gb) and z1.optimizer_gb == pytest.approx(ddp.optimizer_gb)
    assert z3.weights_gb == pytest.approx(ddp.weights_gb / 8) and z3.gradients_gb == pytest.approx(ddp.gradients_gb / 8)
    assert z3.buffers_gb > 0 and z3.total_gb < ddp.total_gb < ddp_nccl.total_gb
    ck = memory.estimate(cfg, 8, "zero3", 8192, grad_checkpointing=True)
    assert ck.activations_gb < 0.1 * z3.activations_gb
    eight = memory.estimate(cfg, 8, "zero3", 8192, optimizer="adamw8bit")
    assert eight.optimizer_gb < 0.55 * z3.optimizer_gb


def test_recommendation_ladder():
    assert memory.recommend(preset("tinyllama-1.1b"), 8, 16384)[0] == "ddp"
    assert memory.recommend(preset("llama-3-8b"), 8, 8192)[0] == "ddp"
    pick, table = memory.recommend(preset("llama-3-8b"), 2, 32768)
    assert pick == "zero3+checkpointing" and not table["ddp"].fits() and not table["zero3"].fits()
    assert memory.recommend(preset("llama-3-70b"), 8, 4096)[0] == "none"                      # fp32 AdamW state of 70 B
    assert memory.recommend(preset("llama-3-70b"), 8, 4096, optimizer="adamw8bit")[0] == "zero3+checkpointing"
    assert memory.main(["--model", "llama-3-8b", "--world", "8", "--seq-len", "4096", "--micro-batch", "2"]) == 0


def test_student_memory_note_names_a_plan_that_fits():
    from types import SimpleNamespace
    from llm_distillery_b200.models.student import StudentModel
    from llm_distillery_b200.parallel.fsdp import FullShardComm

    def note(model, world, comm, batch, ctx, opt="adamw", ck=False):
        ns = SimpleNamespace(comm=comm, world=world, batch_size=batch, context_len=ctx, optimizer_name=opt,
                             grad_checkpointing=ck, model=SimpleNamespace(cfg=preset(model)))
        return StudentModel.memory_note(ns)
    ok = note("tinyllama-1.1b", 1, None, 8, 2048)
    assert "ddp, 1 rank(s)" in ok and "NOT fit" not in ok
    ddp8 = SimpleNamespace(shards_optimizer=True)
    big = note("llama-3-8b", 2, ddp8, 8, 4096)
    assert "fsdp" in big and "does NOT fit" in big and "shard_strategy zero3 and grad_checkpointing" in big
    z3 = SimpleNamespace(full_shard=True, shards_optimizer=True)
    assert "zero3, 8 rank(s)" in note("llama-3-8b", 8, z3, 2, 4096)
    assert "no built-in plan fits" in note("llama-3-70b", 8, z3, 1, 4096)


def test_shard_strategy_auto_resolves_from_the_student_config(tmp_path):
    import json
    from types import SimpleNamespace
    from llm_distillery_b200.cli import resolve_shard_strategy

    def run(model, world, batch, ctx, optimizer="adamw", ck=False, strategy="auto"):
        d = tmp_path / f"{model}-{world}-{batch}-{ctx}"
        d.mkdir(exist_ok=True)
        (d / "config.json").write_text(json.dumps(preset(model).to_hf_dict()))
        cfg = SimpleNamespace(shard_strategy=strategy, student_path=str(d), batch_size=batch, context_len=ctx,
                              save_topK=200, enable_topK=True, optimizer=optimizer, grad_checkpointing=ck)
        return resolve_shard_strategy(cfg, world), cfg
    assert run("tinyllama-1.1b", 8, 8, 2048)[0] == "ddp"
    pick, cfg = run("llama-3-8b", 2, 8, 4096)
    assert pick == "zero3" and cfg.shard_strategy == "zero3" and cfg.grad_checkpointing is True
    pick, cfg = run("llama-3-70b", 8, 1, 4096)                # nothing fits: the smallest plan, with a notice
    assert pick == "zero3" and cfg.grad_checkpointing is True
    pick, cfg = run("llama-3-8b", 1, 8, 4096)                 # one GPU: checkpointing is the only lever
    assert pick == "ddp" and cfg.grad_checkpointing is True
    assert run("llama-3-8b", 2, 8, 4096, strategy="fsdp")[0] == "fsdp"        # explicit values pass through
    cfg = SimpleNamespace(shard_strategy="auto", student_path=str(tmp_path / "missing"), batch_size=1, context_len=8,
                          save_topK=1, enable_topK=True, optimizer="adamw", grad_checkpointing=False)
    assert resolve_shard_strategy(cfg, 4) == "ddp"


def test_tensor_parallel_width_is_the_smallest_that_fits():
    t70, t8, tiny = preset("llama-3-70b"), preset("llama-3-8b"), preset("tinyllama-1.1b")
    # a 70 B teacher in bf16 is 131 GiB of weights: one B200 holds it, eight replicas collect without communication
    assert memory.teacher_footprint_gb(t70, 1, 8192, 128) < memory.HBM_GB - memory.HEADROOM_GB
    assert memory.recommend_tp([t70], 8, 8192, 128) == 1
    assert memory.recommend_tp([t70], 8, 65536, 128) == 2          # eight sequences of 8192 per forward: no longer
    assert memory.recommend_tp([t8, tiny], 8, 16384) == 1
    big = preset("llama-3-70b", num_hidden_layers=240)             # three times deeper: needs the weights split
    assert memory.recommend_tp([big], 8, 8192, 128) == 4
    assert memory.teacher_footprint_gb(t70, 8, 8192, 128) < 0.2 * memory.teacher_footprint_gb(t70, 1, 8192, 128)
    # only widths that divide the ranks, the heads, the KV heads and the FFN width are offered
    odd = preset("llama-3-70b", num_hidden_layers=240, num_key_value_heads=2)   # nothing fits: the widest valid
    assert memory.recommend_tp([odd], 8, 8192, 128) == 2

    from types import SimpleNamespace
    from llm_distillery_b200.cli import resolve_tp_size
    cfg = SimpleNamespace(tp_size=4, context_len=8192, save_topK=128, enable_topK=True, crop_distr_to_size=128256)
    assert resolve_tp_size(cfg, [], 8) == 4 and resolve_tp_size(cfg, [], 2) == 2 and resolve_tp_size(cfg, [], 1) == 1
