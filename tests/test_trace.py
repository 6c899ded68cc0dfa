"""Phase timers: CPU fallback, accumulation per phase, disabled timers cost nothing and record nothing."""
import time

from llm_distillery_b200.obs.trace import PhaseTimer


def test_cpu_phases_accumulate_and_reset():
    t = PhaseTimer(enabled=True, nvtx=False, device="cpu")
    for _ in range(3):
        with t.phase("a"):
            time.sleep(0.01)
    with t.phase("b"):
        pass
    s = t.summary()
    assert set(s) == {"a", "b"} and s["a"] >= 25.0 and s["b"] < 5.0
    assert t.summary() == {}


def test_disabled_timer_records_nothing():
    t = PhaseTimer(enabled=False, nvtx=False, device="cpu")
    with t.phase("a"):
        pass
    assert t.summary() == {}


def test_engine_reports_phase_times_on_cpu(monkeypatch):
    import torch
    from llm_distillery_b200.engine.trainer import DistillEngine, synthetic_batch
    from llm_distillery_b200.models.llama import LlamaConfig, build_model
    monkeypatch.setenv("B200_TRACE", "1")
    cfg = LlamaConfig(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=2,
                      num_key_value_heads=1, max_position_embeddings=64)
    eng = DistillEngine(build_model(cfg, dtype=torch.float32, device="cpu", seed=0), loss="kl", lr=1e-3)
    eng.train_step([synthetic_batch(cfg.vocab_size, 2, 32, 8, seed=1)])
    s = eng.timer.summary()
    assert {"forward+loss", "backward", "reduce+optimizer"} <= set(s) and all(v >= 0 for v in s.values())
