"""Learning-rate schedules as pure functions of the optimizer-step index.

``wsd`` is the reference's Warmup-Stable-Decay schedule (utils/finetuning_utils.py:16-43): half-cosine warm-up
0 -> lr over ``warmup`` steps, constant until ``int(total * decay_start)``, linear decay to ``final_lr``, then
``final_lr``. The other names follow ``transformers.get_scheduler`` semantics (linear warm-up): cosine, linear,
constant, constant_with_warmup, polynomial, cosine_with_restarts, inverse_sqrt.
"""
from __future__ import annotations

import math


class LRSchedule:
    def __init__(self, name: str, base_lr: float, total_steps: int, warmup_steps: int = 0, decay_start: float = 0.9,
                 final_lr: float = 5e-7):
        self.name = name.lower()
        self.base_lr = float(base_lr)
        self.total_steps = max(1, int(total_steps))
        self.warmup_steps = int(warmup_steps)
        self.decay_start_step = int(self.total_steps * decay_start)
        self.decay_steps = self.total_steps - self.decay_start_step
        self.final_lr = float(final_lr)
        self.step_index = 0
        known = ("wsd", "cosine", "linear", "constant", "constant_with_warmup", "polynomial", "cosine_with_restarts",
                 "inverse_sqrt")
        if self.name not in known:
            raise ValueError(f"Invalid lr_scheduler name: {name}; available: {known}")

    def lr_at(self, step: int) -> float:
        n, w, T = self.name, self.warmup_steps, self.total_steps
        if n == "wsd":
            if step < w:
                return self.base_lr * 0.5 * (1 + math.cos(math.pi + (step / w) * math.pi))
            if step <= self.decay_start_step:
                return self.base_lr
            if step < T:
                frac = (step - self.decay_start_step) / self.decay_steps
                return self.base_lr * (1 - frac * (1 - self.final_lr / self.base_lr))
            return self.final_lr
        if n == "constant":
            return self.base_lr
        warm = (step / max(1, w)) if step < w else None
        if warm is not None:
            return self.base_lr * warm
        if n == "constant_with_warmup":
            return self.base_lr
        if n == "inverse_sqrt":
            shift = max(1, w)
            return self.base_lr * math.sqrt(shift / max(1, step + shift - w)) if w else self.base_lr / math.sqrt(step + 1)
        prog = min(1.0, (step - w) / max(1, T - w))
        if n == "linear":
            return self.base_lr * max(0.0, 1.0 - prog)
        if n == "cosine":
            return self.base_lr * max(0.0, 0.5 * (1 + math.cos(math.pi * prog)))
        if n == "cosine_with_restarts":
            return self.base_lr * max(0.0, 0.5 * (1 + math.cos(math.pi * ((prog * 1.0) % 1.0))))
        if n == "polynomial":
            lr_end = 1e-7
            return (self.base_lr - lr_end) * (1 - prog) ** 1.0 + lr_end if step <= T else lr_end
        raise AssertionError(n)

    @property
    def lr(self) -> float:
        return self.lr_at(self.step_index)

    def step(self) -> float:
        self.step_index += 1
        return self.lr

    def state_dict(self) -> dict:
        return {"name": self.name, "step_index": self.step_index, "base_lr": self.base_lr,
                "total_steps": self.total_steps, "warmup_steps": self.warmup_steps,
                "decay_start_step": self.decay_start_step, "final_lr": self.final_lr}

    def load_state_dict(self, sd: dict) -> None:
        self.step_index = int(sd["step_index"])


def set_lr_scheduler(lr_scheduler_name: str, base_lr: float, num_warmup_steps: int, num_training_steps: int,
                     decay_start: float = 0.9, final_lr: float = 5e-7) -> LRSchedule:
    return LRSchedule(lr_scheduler_name, base_lr, num_training_steps, num_warmup_steps, decay_start, final_lr)
