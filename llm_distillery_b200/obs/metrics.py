"""Metrics: the reference's scalar names on the reference's step axis (samples trained), written to
``<cache>/metrics.jsonl`` and, when asked, to Weights & Biases in offline mode (there is no network on the box).

``Losses`` is the per-log-interval accumulator (reference: classes/losses.py): per-conversation loss dicts are
summed, logged as ``Loss/<key>`` or ``Val Loss/<key>`` averaged over the conversations accumulated, then emptied.
"""
from __future__ import annotations

import json
import os
import time

import torch


class MetricsLogger:
    def __init__(self, out_dir: str, backend: str = "jsonl", run_name: str = "", config: dict | None = None,
                 group: str = ""):
        os.makedirs(out_dir, exist_ok=True)
        self.path = os.path.join(out_dir, "metrics.jsonl")
        self._f = open(self.path, "a", encoding="utf-8")
        self.wandb_run = None
        if backend in ("wandb", "both"):
            try:
                os.environ.setdefault("WANDB_MODE", "offline")
                os.environ.setdefault("WANDB_SILENT", "true")
                import wandb
                self.wandb_run = wandb.init(project="student_training", name=run_name, config=config or {}, group=group,
                                            reinit=True, dir=out_dir)
            except Exception as e:  # noqa: BLE001 - metrics must never stop training
                print(f"wandb unavailable ({e}); logging to {self.path} only")
        self._f.write(json.dumps({"event": "run_start", "name": run_name, "time": time.time()}) + "\n")

    def log(self, scalars: dict, step: int) -> None:
        rec = {"step": int(step), "time": time.time()}
        for k, v in scalars.items():
            rec[k] = float(v.item() if isinstance(v, torch.Tensor) else v)
        self._f.write(json.dumps(rec) + "\n")
        self._f.flush()
        if self.wandb_run is not None:
            self.wandb_run.log({k: v for k, v in rec.items() if k not in ("step", "time")}, step=int(step))

    def finish(self) -> None:
        if self.wandb_run is not None:
            self.wandb_run.finish()
            self.wandb_run = None
        if not self._f.closed:
            self._f.close()


class Losses:
    def __init__(self, logger: MetricsLogger | None, validation: bool = False):
        self.logger = logger
        self.validation = validation
        self.loss_dict: dict[str, torch.Tensor] = {}
        self.num_steps_accumulated = 0

    def add_losses(self, new_losses: dict, count: int = 1) -> None:
        """``new_losses``: sums over ``count`` conversations (detached)."""
        if not new_losses:
            raise ValueError("No losses to add to the loss dictionary.")
        self.num_steps_accumulated += count
        for k, v in new_losses.items():
            if k == "train_loss":
                continue
            v = v.detach() if isinstance(v, torch.Tensor) else torch.tensor(float(v))
            self.loss_dict[k] = self.loss_dict[k] + v if k in self.loss_dict else v.clone()

    def empty(self) -> None:
        self.loss_dict = {}
        self.num_steps_accumulated = 0

    def averages(self) -> dict[str, float]:
        n = max(1, self.num_steps_accumulated)
        return {k: float(v) / n for k, v in self.loss_dict.items()}

    def log(self, step: int, average: bool = True) -> None:
        if self.logger is None or not self.loss_dict:
            return
        prefix = "Val Loss" if self.validation else "Loss"
        n = max(1, self.num_steps_accumulated) if average else 1
        self.logger.log({f"{prefix}/{k}": float(v) / n for k, v in self.loss_dict.items()}, step)

    def __str__(self) -> str:
        head = " Validation Losses:\n" if self.validation else " Training Losses:\n"
        return head + "".join(f"{k}: {float(v):.4f}\n" for k, v in self.loss_dict.items())
