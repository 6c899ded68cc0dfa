"""Student role: trains the student against the stored teacher distributions.

Bookkeeping follows the reference exactly (collect_and_finetune.py:178-208, classes/student/model.py:319-532):
every "step" counter is in SAMPLES (conversations), an optimizer step happens whenever the number of trained
samples reaches the next multiple of ``grad_accum * batch_size``, validation runs at step 0 and every
``validate_every_n_epochs * dataset_len`` samples on an endlessly cycling validation reader, checkpoints are
HF folders ``<cache>/student/trained/<model>_step_<N|final>``, and in chunked mode the trainer state is saved
after every chunk and restored at the next one.

What differs: the model, loss head and optimizer are this package's kernels driven by ``DistillEngine``; the
per-conversation Python loss loop is one fused head call per micro-batch; teacher batches arrive from a prefetch
thread in pinned memory; with several ranks each rank trains a different batch of the same global step and the
engine's communicator reduces the gradients; trainer state also resumes across process restarts.
"""
from __future__ import annotations

import math
import os
import time

import numpy as np
import torch

from ..ckpt import hf as ckpt
from ..engine.schedule import set_lr_scheduler
from ..engine.trainer import DistillEngine, HostBatch
from ..obs.console import progress, status
from ..obs.metrics import Losses, MetricsLogger
from .base_model import BaseModel


class StopRequested(Exception):
    """Raised out of the training loop after the trainer state has been saved on a stop request (SIGTERM / SIGINT)."""


class StudentModel(BaseModel):
    def __init__(self, model_path: str, paths, add_bos: bool, prompt_format: dict, batch_size: int,
                 interactive: bool = False):
        super().__init__(model_path, student=True, interactive=interactive)
        self.model = None
        self.engine: DistillEngine | None = None
        self.tokenizer_dir = self.model_path
        self.add_bos = add_bos
        self.prompt_format = prompt_format
        self.batch_size = batch_size
        self.paths = paths
        self.losses: Losses | None = None
        self.logger: MetricsLogger | None = None
        # hyper-parameters (set by cli.set_training_params)
        self.optimizer_name = "adamw"
        self.lr_scheduler_name = "wsd"
        self.lr = 0.0
        self.decay_start = 0.9
        self.final_lr = 5e-7
        self.alpha = 2.0
        self.loss_kind = "reference"
        self.num_epochs = 0
        self.total_training_steps = 0
        self.num_warmup_steps = 0
        self.grad_accum = 1
        self.num_grad_accum_batches = 0
        self.eff_batch_size = 0
        self.validation_every_steps = 0
        self.save_every_steps = 0
        # progress
        self.next_save_step = 0
        self.num_trained_steps = 0
        self.next_val_step = 0
        self.next_accum_step = 0
        self.saved_state = False
        self.val_batch_order_ids: list = []
        # misc
        self.freeze_layers: list = []
        self.training_precision_name = "bf16"
        self.data_order = "sorted"
        self.save_final_state = False
        self.grad_checkpointing = False
        self.multi_gpu = False
        self.use_fa2 = True
        self.wandb_comment = ""
        self.device_map_name = ""
        self.max_memory: dict = {}
        self.num_gpu0_layers = 0
        self.metrics_backend = "jsonl"
        self.comm = None           # parallel communicator (None = single GPU)
        self.rank, self.world = 0, 1
        self.seed = 0
        self.tokens_trained = 0
        self.train_seconds = 0.0
        self._rng = np.random.default_rng(0)

    # ------------------------------------------------------------------ model / optimizer
    def _dtype(self, device: torch.device) -> torch.dtype:
        """Compute dtype for ``training_precision`` (reference: classes/student/model.py:121-148).

        ``bf16``: bf16 tensor-core kernels, fp32 master weights and optimizer state. ``4bit`` / ``8bit``: the same
        compute, with the decoder layers' matrices frozen as NF4 / int8 weights (``_load_model``). ``fp32`` and
        ``fp16`` name compute types these kernels do not have: on a GPU they are refused rather than silently run in
        bf16. On CPU (the restatement that the tests and the plumbing configuration run) everything is fp32."""
        if device.type != "cuda":
            return torch.float32
        name = (self.training_precision_name or "bf16").lower()
        if name in ("fp32", "fp16"):
            raise ValueError(f"training_precision = {name!r} is not available on GPUs here: the kernels compute in bf16 "
                             "with fp32 accumulation, fp32 master weights and fp32 optimizer state. Set "
                             "training_precision to 'bf16' (or to '4bit' / '8bit' for frozen low-bit base weights).")
        return torch.bfloat16

    def _load_model(self) -> None:
        dev = torch.device(self.device)
        self.model = ckpt.load_hf_model(self.model_path, dtype=self._dtype(dev), device=dev)
        self.model.grad_checkpointing = bool(self.grad_checkpointing)
        name = (self.training_precision_name or "bf16").lower()
        if name in ("4bit", "8bit"):
            self.model.quantize_frozen_linears("nf4" if name == "4bit" else "int8")
            if self.rank == 0 and not getattr(self, "_quant_note_done", False):
                q = self.model.quant
                print(f"training_precision {name}: the decoder layers' matrices are frozen {q.kind} weights "
                      f"({q.packed_bytes() / 2 ** 30:.2f} GiB packed); embeddings, norms and the LM head train.")
                self._quant_note_done = True
        if self.freeze_layers:
            self.model.apply_freeze(self.freeze_layers)
        schedule = set_lr_scheduler(self.lr_scheduler_name, self.lr, self.num_warmup_steps, self.num_grad_accum_batches,
                                    self.decay_start, self.final_lr)
        if self.rank == 0 and dev.type == "cuda" and not getattr(self, "_memory_note_done", False):
            try:
                print(self.memory_note())
            except Exception as e:  # noqa: BLE001 - an estimate must never stop a run
                print(f"(memory estimate unavailable: {e})")
            self._memory_note_done = True
        self.engine = DistillEngine(self.model, loss=self.loss_kind, temperature=self.temperature, alpha=self.alpha,
                                    crop_to_size=self.crop_to_size, optimizer=self.optimizer_name, lr=self.lr,
                                    betas=(0.9, 0.99), weight_decay=2e-8, grad_accum=self.grad_accum, schedule=schedule,
                                    comm=self.comm, vocab_parallel=bool(getattr(self, "vocab_parallel_loss", False)),
                                    max_rows_per_rank=int(self.batch_size) * int(self.context_len))

    def memory_note(self) -> str:
        """One line on how the run sits in 180 GB of HBM per GPU under the configured sharding, and what would fit if
        it does not (``parallel.memory``)."""
        from ..parallel import memory
        strategy = getattr(self.comm, "full_shard", False) and "zero3" or \
            ("fsdp" if getattr(self.comm, "shards_optimizer", False) else "ddp")
        tokens = int(self.batch_size) * int(self.context_len)
        kw = dict(topk=200, optimizer=self.optimizer_name)
        fp = memory.estimate(self.model.cfg, self.world, strategy, tokens, grad_checkpointing=bool(self.grad_checkpointing),
                             comm="p2p" if type(self.comm).__name__.startswith("P2P") else "nccl", **kw)
        note = (f"Estimated memory per GPU ({strategy}, {self.world} rank(s), up to {tokens} tokens per micro-batch): "
                f"{fp.total_gb:.0f} GB of {memory.HBM_GB:.0f} GB (weights {fp.weights_gb:.1f}, gradients "
                f"{fp.gradients_gb:.1f}, optimizer {fp.optimizer_gb:.1f}, activations {fp.activations_gb:.1f}).")
        if not fp.fits():
            pick, _ = memory.recommend(self.model.cfg, self.world, tokens, **kw)
            hint = {"none": "no built-in plan fits: use more GPUs, an 8-bit optimizer, a smaller batch_size or context_len",
                    "ddp": "it fits with replicated weights (shard_strategy ddp)"}.get(
                        pick, f"it fits with shard_strategy {pick.split('+')[0]}" +
                        (" and grad_checkpointing" if "checkpointing" in pick else ""))
            note += f" This does NOT fit; {hint}."
        return note

    def _unload_model(self) -> None:
        if self.comm is not None and hasattr(self.comm, "close"):
            self.comm.close()              # unit hooks of the full-shard engine leave with its model
        self.model = None
        self.engine = None
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    # ------------------------------------------------------------------ data order / batching
    def reorder_dataset(self) -> None:
        if self.dataset_sorted:
            return
        if self.data_order == "shuffle":
            self._rng.shuffle(self.dataset)
        elif self.data_order == "sorted":
            self.dataset.sort(key=lambda c: c.length, reverse=True)
            self.dataset_sorted = True
        elif self.data_order == "native":
            self.dataset_sorted = True

    def _construct_batches(self, dataset_chunk):
        n = math.ceil(len(dataset_chunk) / self.batch_size)
        convo_batches = [dataset_chunk[i * self.batch_size:(i + 1) * self.batch_size] for i in range(n)]
        return convo_batches, [[c.origin_convo_id for c in b] for b in convo_batches]

    def _my_share(self, convo_batches, id_batches):
        """Global step t trains batches t*world .. t*world+world-1, one per rank. Returns this rank's batches (None
        where the last global step has no batch for it) and the sample count of every global step."""
        w = self.world
        steps = math.ceil(len(convo_batches) / w)
        mine, mine_ids, sizes = [], [], []
        for t in range(steps):
            group = convo_batches[t * w:(t + 1) * w]
            sizes.append(sum(len(b) for b in group))
            mine.append(group[self.rank] if self.rank < len(group) else None)
            if self.rank < len(group):
                mine_ids.append(id_batches[t * w + self.rank])
        return mine, mine_ids, sizes

    def build_host_batch(self, convos, teacher: dict) -> HostBatch:
        """Assemble one micro-batch from tokenised conversations and their stored teacher rows."""
        L = max(c.length for c in convos)
        tokens = np.stack([c.tokenized[:L] for c in convos])
        rows, ids, logp, seg, labels, avoid = [], [], [], [], [], []
        need_ce = self.loss_kind == "reference"
        for b, c in enumerate(convos):
            ci = c.content_indices()
            ci = ci[ci < L]
            t_ids = teacher["indices"][b]
            n = min(len(ci), teacher["lengths"][b], len(t_ids) if t_ids is not None else len(ci))
            if n <= 0:
                continue
            rows.append(ci[:n] + b * L)
            vals = teacher["values"][b][:n]
            if t_ids is None:                      # full-distribution dataset: every id of the cropped vocabulary
                t_ids = np.broadcast_to(np.arange(vals.shape[1], dtype=np.int64), vals.shape)
            ids.append(np.asarray(t_ids[:n], dtype=np.int32))
            logp.append(vals.astype(np.float32))
            seg.append(np.full(n, b, dtype=np.int64))
            if need_ce:
                ce_idx, av = c.ce_indices(self.context_len)
                lab = np.full(n, -1, dtype=np.int64)
                m = min(n, len(ce_idx))
                ok = ce_idx[:m] < L
                lab[:m][ok] = c.tokenized[ce_idx[:m][ok]]
                labels.append(lab)
                a = np.zeros(n, dtype=bool)
                a[av[av < n]] = True
                avoid.append(a)
        cat = lambda xs, dt: torch.from_numpy(np.ascontiguousarray(np.concatenate(xs)).astype(dt, copy=False))  # noqa: E731
        hb = HostBatch(input_ids=torch.from_numpy(np.ascontiguousarray(tokens)), ids=cat(ids, np.int32),
                       logp=cat(logp, np.float32), seg=cat(seg, np.int64), n_seg=len(convos),
                       rows=cat(rows, np.int64), labels=cat(labels, np.int64) if need_ce else None,
                       avoid=cat(avoid, bool) if need_ce else None, n_tokens=int(tokens.size))
        return hb.pin() if torch.device(self.device).type == "cuda" else hb

    # ------------------------------------------------------------------ checkpoints
    def _save_model(self, step) -> None:
        folder = os.path.join(self.paths.student_trained, f"{self.model_name}_step_{step}")
        with self.engine.full_parameters():       # every rank: under full sharding the weights are gathered first
            # every rank holds the whole weights here: the shard files are written side by side, rank r taking shards
            # r, r + world, ...; rank 0 adds the config, the index and the tokenizer
            ckpt.save_hf_model(self.model, folder, tokenizer_src=self.tokenizer_dir, writer=(self.rank, self.world),
                               max_shard_bytes=int(getattr(self, "max_shard_bytes", 5 * 1024 ** 3)))

    _HASHED = ("model_name", "lr", "batch_size", "grad_accum", "loss_kind", "temperature", "alpha", "context_len",
               "crop_to_size", "optimizer_name", "lr_scheduler_name", "num_warmup_steps", "decay_start", "final_lr",
               "data_order", "freeze_layers", "seed")

    def _config_hash(self) -> str:
        """Fingerprint of what makes a resumed run the continuation of the saved one (not: paths, save / validation
        intervals, world size)."""
        import hashlib
        import json
        rec = {k: getattr(self, k, None) for k in self._HASHED}
        return hashlib.sha256(json.dumps(rec, sort_keys=True, default=str).encode()).hexdigest()[:16]

    def _counters(self) -> dict:
        return {"num_trained_steps": self.num_trained_steps, "next_save_step": self.next_save_step,
                "next_val_step": self.next_val_step, "next_accum_step": self.next_accum_step,
                "total_training_steps": self.total_training_steps, "seed": self.seed, "world": self.world,
                "tokens_trained": self.tokens_trained, "data_order": self.data_order,
                "rng_state": self._rng.bit_generator.state, "config_hash": self._config_hash()}

    def _save_state(self, collective: bool = True) -> None:
        """``collective=False``: emergency save after a peer failed - no barrier, files of this rank only."""
        if collective and self.num_trained_steps < self.total_training_steps and self.rank == 0:
            self.paths.empty_student_states()
        if collective and self.comm is not None:
            self.comm.barrier()
        mine = self.rank == 0 or (self.comm is not None and self.comm.shards_optimizer)
        # an emergency save happens after a step that failed half-way: its samples were counted but never applied
        counters = self._counters() if collective else (getattr(self, "_applied", None) or self._counters())
        if not collective and hasattr(self.comm, "unapplied_steps"):
            # the host may have issued one or two optimizer steps past the lost peer before it learnt of it; their
            # kernels did nothing (csrc/comm/p2p.cu), so the saved step count and sample counters go back with them
            lost = self.comm.unapplied_steps()
            if lost > 0:
                hist = self._applied_history
                self.engine.opt.step_count = max(0, self.engine.opt.step_count - lost)
                counters = hist[-1 - lost] if len(hist) > lost else (hist[0] if hist else counters)
        if not collective and getattr(self.comm, "full_shard", False):
            # no peer to gather the weights from: this rank's optimizer shard (with its fp32 master weights) only
            ckpt.save_trainer_state(self.paths.student_states, None, self.engine.opt, self.engine.schedule, counters)
            return
        with self.engine.full_parameters():
            if mine:
                ckpt.save_trainer_state(self.paths.student_states, self.model if (self.rank == 0 or not collective) else None,
                                        self.engine.opt, self.engine.schedule, counters)

    def _load_state(self) -> None:
        self._load_model()
        with self.engine.full_parameters(writeback=True):
            ckpt.load_model_state(self.paths.student_states, self.model)
        c = ckpt.load_trainer_state(self.paths.student_states, None, self.engine.opt, self.engine.schedule)
        if self.comm is not None and hasattr(self.comm, "shards_written"):
            self.comm.shards_written()      # the optimizer load rewrote this rank's weight pieces from its master copy
        for k in ("num_trained_steps", "next_save_step", "next_val_step", "next_accum_step", "tokens_trained"):
            if k in c:
                setattr(self, k, c[k])
        if "rng_state" in c:                 # the shuffle order of the epochs still to come continues where it stopped
            try:
                self._rng.bit_generator.state = c["rng_state"]
            except (TypeError, ValueError, KeyError):
                pass
        if c.get("config_hash") not in (None, self._config_hash()) and self.rank == 0:
            print("Note: the saved trainer state was written under different training settings "
                  f"(fingerprint {c['config_hash']} != {self._config_hash()}); counters and optimizer state are reused as they are.")

    # ------------------------------------------------------------------ training
    def _prefetch_dataset_chunk(self, data_manager, data_list, full_collect, trainable_ids):
        self.reorder_dataset()
        chunk = self.dataset if full_collect else [c for c in self.dataset if c.origin_convo_id in trainable_ids]
        convo_batches, id_batches = self._construct_batches(chunk)
        mine, mine_ids, sizes = self._my_share(convo_batches, id_batches)
        data_list.append((mine, sizes))
        data_manager.enqueue_get_batches(mine_ids, sort_ids=True)
        return data_list

    def train_chunk(self, data_manager, validation_data_manager, full_collect: bool) -> None:
        trainable_ids = set(data_manager.get_dataset_ids())
        if not self.validation_dataset_sorted:
            self.validation_dataset.sort(key=lambda c: c.length, reverse=True)
            self.validation_dataset_sorted = True
            self.validation_dataset_batched, self.val_batch_order_ids = self._construct_batches(self.validation_dataset)
            if self.val_batch_order_ids:
                validation_data_manager.read_only_mode(self.val_batch_order_ids, sort_ids=True)
        if self.logger is None and self.rank == 0:
            name = f"{self.wandb_comment} " if self.wandb_comment else ""
            short = self.model_name if len(self.model_name) <= 20 else f"{self.model_name[:20]}..."
            name += f"{short} lr({self.lr}) ({time.strftime('%d.%m.%Y / %H:%M:%S')})"
            cfg = {k: v for k, v in self.__dict__.items() if isinstance(v, (int, float, str, bool, list, dict))}
            self.logger = MetricsLogger(self.paths.cache, self.metrics_backend, run_name=name, config=cfg,
                                        group=self.model_name)
        resume = self.saved_state or (self.num_trained_steps == 0 and ckpt.has_trainer_state(self.paths.student_states)
                                      and os.environ.get("B200_RESUME", "1") == "1")
        self.progress_bar = progress(total=self.total_training_steps, initial=self.num_trained_steps, desc="Training",
                                     leave=False)
        if resume:
            with status(self.progress_bar, "Loading state..."):
                self._load_state()
            self.saved_state = False
            self.progress_bar.n = self.num_trained_steps      # the saved counters say where the run stands
            self.progress_bar.refresh()
        else:
            with status(self.progress_bar, "Loading model..."):
                self._load_model()
        self._applied = self._counters()
        self._applied_history = [self._applied]      # counters after each of the last few optimizer steps
        self.training_active = True
        if self.losses is None:
            self.losses = Losses(self.logger)
        if self.num_trained_steps == 0:
            self._validate_distillation(validation_data_manager)
        t0 = time.time()
        data_list = self._prefetch_dataset_chunk(data_manager, [], full_collect, trainable_ids)
        updated = True
        if full_collect:
            # a run taken up again in the middle of an epoch goes on where it stopped: the samples of that epoch that
            # the saved state already counts are passed over
            into_epoch = self.num_trained_steps % max(1, self.dataset_len) if resume else 0
            left = self.total_training_steps - self.num_trained_steps + into_epoch
            epochs_left = max(0, math.ceil(left / max(1, self.dataset_len)))
            for e in range(epochs_left):
                if e + 1 < epochs_left:
                    data_list = self._prefetch_dataset_chunk(data_manager, data_list, full_collect, trainable_ids)
                updated = self._run_distillation_cycle(data_list.pop(0), data_manager, validation_data_manager,
                                                       skip_samples=into_epoch if e == 0 else 0)
        else:
            updated = self._run_distillation_cycle(data_list.pop(0), data_manager, validation_data_manager)
        if not updated:
            self._optimizer_step()
        self.train_seconds += time.time() - t0
        if not full_collect:
            with status(self.progress_bar, "Saving state..."):
                self._save_state()
            self.saved_state = True
        if self.num_trained_steps >= self.total_training_steps:
            with status(self.progress_bar, "Saving model at step final..."):
                self._save_model("final")
            if self.save_final_state:
                with status(self.progress_bar, "Saving state..."):
                    self._save_state()
                self.saved_state = True
        with status(self.progress_bar, "Unloading model..."):
            self.training_active = False
            self._unload_model()
        self.progress_bar.close()

    def _stop_agreed(self) -> bool:
        """A stop request (``stop_requested``, set by the signal handler) reaches the ranks at different moments: they
        agree after an optimizer step - a tiny MAX all-reduce - so that all of them save and leave at the same step."""
        mine = bool(getattr(self, "stop_requested", False))
        if self.world <= 1:
            return mine
        import torch.distributed as dist
        if not dist.is_initialized():
            return mine
        dev = self.engine.device if dist.get_backend() == "nccl" else "cpu"
        t = torch.tensor([1.0 if mine else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return bool(t.item() > 0)

    def _phase_times(self) -> tuple[dict, dict]:
        """(this rank's device-timed phases since the last step, cross-rank figures). With tracing on, every rank
        takes part: the compute time (forward + loss + backward) of each rank is gathered, and the spread between the
        slowest and the fastest rank is the time the fast ones spend waiting inside the gradient reduction."""
        if not self.engine.timer.enabled:
            return {}, {}
        phases = self.engine.timer.summary()
        cross = {}
        if self.world > 1:
            import torch.distributed as dist
            if dist.is_initialized():
                dev = self.engine.device if dist.get_backend() == "nccl" else "cpu"
                mine = torch.tensor([phases.get("forward+loss", 0.0) + phases.get("backward", 0.0)],
                                    dtype=torch.float64, device=dev)
                parts = [torch.zeros_like(mine) for _ in range(self.world)]
                dist.all_gather(parts, mine)
                ts = [float(p.item()) for p in parts]
                cross = {"Perf/rank skew ms": max(ts) - min(ts), "Perf/slowest rank": float(ts.index(max(ts)))}
                step = sum(phases.values())
                if step > 0:        # share of the step that is not compute: reduction + optimizer + waiting for peers
                    cross["Perf/non-compute share"] = 1.0 - float(mine.item()) / step
        return phases, cross

    def _optimizer_step(self) -> None:
        lr = self.engine.lr
        self.engine.optimizer_step()
        phases, cross = self._phase_times()
        if self.logger is not None:
            perf = {"Learning Rate": lr}
            now = time.time()
            last_t, last_tok = getattr(self, "_perf_mark", (None, 0))
            if last_t is not None and now > last_t:
                perf["Perf/train tokens per s"] = (self.tokens_trained - last_tok) * self.world / (now - last_t)
                perf["Perf/step ms"] = 1e3 * (now - last_t)
            self._perf_mark = (now, self.tokens_trained)
            if self.engine.timer.enabled:
                for k, v in phases.items():
                    perf[f"Perf/{k} ms"] = v
                perf.update(cross)
                if torch.cuda.is_available():
                    perf["Perf/HBM high-water GB"] = torch.cuda.max_memory_allocated() / 2 ** 30
            self.logger.log(perf, self.num_trained_steps)
        self.losses.log(self.num_trained_steps)
        self.losses.empty()
        if self.comm is not None and hasattr(self.comm, "check"):
            self.comm.check()      # a bounded device-side wait that ran out (lost peer) surfaces here, not as a hang

    def _run_distillation_cycle(self, cycle, data_manager, validation_data_manager, skip_samples: int = 0) -> bool:
        batches, sizes = cycle
        updated = False
        for convos, n_samples in zip(batches, sizes):
            if skip_samples >= n_samples > 0:        # trained before the interruption
                skip_samples -= n_samples
                if convos is not None:
                    data_manager.read_next_batch()   # its rows were queued with the rest of the epoch: drop them
                continue
            skip_samples = 0
            updated = False
            hbt = getattr(self, "heartbeat", None)
            if hbt is not None:      # between steps, nothing in flight: learn about a lost peer BEFORE the next launch
                hbt.beat(self.num_trained_steps, "train")
                hbt.check()
            # known before the micro-batch runs: the optimizer step follows it (the sharded engines then fold the
            # update of each layer into that layer's gradient reduction)
            steps_after = self.num_trained_steps + n_samples >= self.next_accum_step
            if convos is not None:
                teacher = data_manager.read_next_batch()
                hb = self.build_host_batch(convos, teacher)
                mb = hb.to_device(self.engine.device)
                loss, logs = self.engine.micro_step(mb, last=steps_after)
                self.losses.add_losses(logs, count=len(convos))
                self.tokens_trained += hb.n_tokens
            else:
                self.engine.idle_micro_step(last=steps_after)
            self.progress_bar.update(n_samples)
            self.num_trained_steps += n_samples
            if self.num_trained_steps >= self.next_accum_step:
                self._optimizer_step()
                updated = True
                self.next_accum_step += self.eff_batch_size
                self._applied = self._counters()     # what an emergency save may claim: nothing beyond this step
                self._applied_history.append(self._applied)
                del self._applied_history[:-4]
                if self._stop_agreed() and self.num_trained_steps < self.total_training_steps:
                    print("Stop requested: saving the trainer state; the same command takes the run up again.", flush=True)
                    with status(self.progress_bar, "Saving state..."):
                        self._save_state()
                    self.training_active = False
                    raise StopRequested()
            if self.num_trained_steps >= self.next_save_step and self.num_trained_steps < self.total_training_steps:
                with status(self.progress_bar, f"Saving model at step {self.num_trained_steps}..."):
                    self._save_model(self.num_trained_steps)
                self.next_save_step += self.save_every_steps
            if self.num_trained_steps >= self.next_val_step:
                self._validate_distillation(validation_data_manager)
        return updated

    @torch.no_grad()
    def _validate_distillation(self, validation_data_manager) -> None:
        losses = Losses(self.logger, validation=True)
        for convos in self.validation_dataset_batched:
            teacher = validation_data_manager.read_next_batch()
            hb = self.build_host_batch(convos, teacher)
            _, logs = self.engine.eval_batch(hb)
            losses.add_losses(logs, count=len(convos))
        losses.log(self.num_trained_steps)
        self.last_validation = losses.averages()
        self.next_val_step += self.validation_every_steps if self.validation_every_steps > 0 else float("inf")

    def close(self) -> None:
        if self.logger is not None:
            self.logger.finish()
            self.logger = None
