"""The reference arm of ``bench.py``: the UNMODIFIED reference tree under ``baseline/_ref`` trains the benchmark's
student through its own ``StudentModel.train_chunk`` (classes/student/model.py:319-391) - its model loading,
optimizer and scheduler set-up, training loop (``_run_distillation_cycle``, :393-470), loss
(utils/finetuning_utils.py:47-124, ``calculate_divergence``), loss accumulation and backward (classes/losses.py) and
optimizer step. Nothing of this repository's models, kernels or engine is imported on this path.

What stands in for things the image does not have (none of it is reference code):

* ``bitsandbytes`` (not installed): a module whose ``optim`` classes are the ``torch.optim`` equivalents
  (``AdamW`` -> ``torch.optim.AdamW(fused=True)``, the fastest stock implementation).
* ``accelerate`` (not installed): ``transformers`` refuses ``device_map=...`` without it, and the reference always
  passes one. ``AutoModelForCausalLM.from_pretrained`` is wrapped so that the map is dropped, the whole model goes to
  this rank's GPU and ``hf_device_map`` reads ``{"": gpu_index}`` - what accelerate's ``device_map="auto"`` yields
  when one GPU is visible.
* ``wandb`` runs in offline mode (no network, no key); where it is not installed, a logger that turns every logged
  tensor into a Python number (as wandb does when it serialises a row) and drops it. ``h5py`` / ``exllamav2`` (not
  installed): empty modules; the training path never calls them.
* the HDF5 data-manager process: a feeder object with the manager's methods that hands out the same tuples
  (shared-memory name, shape, dtype, per-conversation index arrays, lengths: classes/data_manager.py:332-353) built
  from synthetic top-K targets BEFORE the timed region - the reference's manager prefetches in another process too.

The reference sets ``CUDA_LAUNCH_BLOCKING=1`` when its student module is imported (classes/student/model.py:20);
that is its stock behaviour and stays in force here (``B200_REF_ASYNC=1`` removes it for a side measurement).

The reference has no data parallelism. With N > 1 ranks every rank runs an independent replica on its own GPU with no
gradient exchange; the reported value is N x tokens per step over the slowest rank's time - an upper bound on what N
GPUs could give the reference.

Its only loss is its own weighted KL + reverse-KL + CE-difference loss; the benchmark's temperature (2.0) is applied
the way the reference applies it.
"""
from __future__ import annotations

import json
import os
import shutil
import sys
import time
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

TINYLLAMA = dict(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22,
                 num_attention_heads=32, num_key_value_heads=4, rms_norm_eps=1e-5, rope_theta=10000.0,
                 max_position_embeddings=2048, tie_word_embeddings=False)


def unavailable(why: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}))
    return 0


def _install_stand_ins(gpu_index: int | None):
    import torch

    def _has(name):
        try:
            __import__(name)
            return True
        except Exception:  # noqa: BLE001
            return False

    notes = []
    if not _has("bitsandbytes"):
        o = torch.optim

        def _fused(cls):
            def make(params, **kw):
                try:
                    return cls(params, fused=True, **kw)
                except (TypeError, RuntimeError):
                    return cls(params, **kw)
            return make
        optim = types.SimpleNamespace(
            Adam=_fused(o.Adam), AdamW=_fused(o.AdamW), AdamW8bit=_fused(o.AdamW), AdamW32bit=_fused(o.AdamW),
            PagedAdam=_fused(o.Adam), PagedAdamW8bit=_fused(o.AdamW), PagedAdamW32bit=_fused(o.AdamW), SGD=o.SGD,
            RMSprop=o.RMSprop, RMSprop8bit=o.RMSprop, RMSprop32bit=o.RMSprop, Adagrad=o.Adagrad)
        m = types.ModuleType("bitsandbytes")
        m.optim = optim
        sys.modules["bitsandbytes"] = m
        notes.append("bitsandbytes -> torch.optim (fused)")
    for name in ("h5py", "exllamav2", "nvidia_smi"):
        if not _has(name):
            stub = types.ModuleType(name)
            stub.File = object          # h5py.File appears in annotations of classes/data_manager.py
            sys.modules[name] = stub
            notes.append(f"{name} -> empty module (unused by the training path)")
    os.environ.setdefault("WANDB_MODE", "offline")       # no network, no API key: wandb itself, writing local files
    os.environ.setdefault("WANDB_SILENT", "true")
    if _has("wandb"):
        notes.append("wandb in offline mode")
    else:
        class _Run:
            def log(self, row, step=None):
                for v in row.values():
                    if hasattr(v, "item"):
                        v.item()            # wandb serialises the row: a device tensor is read back here

            def finish(self):
                pass
        w = types.ModuleType("wandb")
        w.init = lambda *a, **k: _Run()
        wr = types.ModuleType("wandb.wandb_run")
        wr.Run = _Run
        w.wandb_run = wr
        sys.modules["wandb"] = w
        sys.modules["wandb.wandb_run"] = wr
        notes.append("wandb -> logger that reads logged tensors back and drops them")
    if not _has("accelerate"):
        import transformers
        real = transformers.AutoModelForCausalLM.from_pretrained.__func__

        def from_pretrained(cls, path, *a, device_map=None, max_memory=None, **kw):
            model = real(cls, path, *a, **kw)
            where = "cpu" if gpu_index is None else f"cuda:{gpu_index}"
            model = model.to(where)
            model.hf_device_map = {"": where if gpu_index is None else gpu_index}
            return model
        transformers.AutoModelForCausalLM.from_pretrained = classmethod(from_pretrained)
        notes.append("accelerate device_map -> whole model on this rank's GPU")
    return notes


def _make_model_dir(folder: str, arch: dict, dtype, device: str) -> None:
    """Random-init checkpoint in HF layout with a small tokenizer and the two sidecar files the reference asks for
    interactively when they are missing (classes/base_model.py:164-176)."""
    import torch
    from tokenizers import Tokenizer, models
    from transformers import LlamaConfig, LlamaForCausalLM, PreTrainedTokenizerFast
    os.makedirs(folder, exist_ok=True)
    torch.manual_seed(1234)
    with torch.device(device):
        model = LlamaForCausalLM(LlamaConfig(**arch)).to(dtype)
    model.save_pretrained(folder, safe_serialization=True)
    del model
    vocab = {"<unk>": 0, "<s>": 1, "</s>": 2}
    vocab.update({f"t{i}": i for i in range(3, 64)})
    tok = PreTrainedTokenizerFast(tokenizer_object=Tokenizer(models.WordLevel(vocab, unk_token="<unk>")),
                                  bos_token="<s>", eos_token="</s>", unk_token="<unk>")
    tok.save_pretrained(folder)
    with open(os.path.join(folder, "prompt_format.json"), "w") as f:
        json.dump({"SYS_START": "#System:\n", "USER_START": "#User:\n", "ASSISTANT_START": "#AI:\n", "SYS_END": "\n\n",
                   "USER_END": "\n\n", "ASSISTANT_END": "\n\n"}, f)
    with open(os.path.join(folder, "pipeline_config.json"), "w") as f:
        json.dump({"batch_size": 1, "add_bos": False, "seq_chunk_len": 256, "completion": False}, f)


class Feeder:
    """Stands in for ``H5DataManager`` on the training side: same methods, same tuples, data prepared up front.
    Call number ``warmup`` of ``read_next_batch`` opens the timed region, call ``warmup + steps`` closes it."""

    def __init__(self, n_batches, B, L, K, vocab, seed, warmup, steps, sync, barrier):
        import numpy as np
        from multiprocessing import shared_memory
        rng = np.random.default_rng(seed)
        self.items = []
        self.h2d_bytes = 0
        for _ in range(n_batches):
            logits = (rng.standard_normal((B, L, K), dtype=np.float32) * 3.0)
            logp = logits - np.log(np.exp(logits - logits.max(-1, keepdims=True)).sum(-1, keepdims=True)) - logits.max(-1, keepdims=True)
            data = logp.astype(np.float16).astype(np.float32)       # stored fp16, handed out fp32 (data_manager.py:323)
            shm = shared_memory.SharedMemory(create=True, size=data.nbytes)
            np.copyto(np.ndarray(data.shape, dtype=data.dtype, buffer=shm.buf), data)
            # K distinct ids per position: a random start plus a stride walk stays distinct below the vocabulary size
            start = rng.integers(0, vocab, (B, L, 1))
            idx = ((start + np.arange(K)[None, None, :] * 157) % vocab).astype(np.int64)
            self.items.append((shm.name, data.shape, data.dtype, [idx[b] for b in range(B)], [L] * B))
            self.h2d_bytes = data.nbytes + idx.nbytes + B * L * 8
            shm.close()
        self.calls, self.warmup, self.steps = 0, warmup, steps
        self.sync, self.barrier = sync, barrier
        self.ev = None
        self.on_start = self.on_stop = None
        self.t0 = self.t1 = None
        self.ids = list(range(n_batches * B))

    # ---- what train_chunk and the training loop call
    def get_dataset_ids(self):
        return self.ids

    def enqueue_get_batches(self, id_batches):
        pass

    def read_only_mode(self, id_batches):
        pass

    def read_next_batch(self):
        import torch
        if self.calls == self.warmup:
            self.barrier()
            self.sync()
            if self.on_start:
                self.on_start()
            if torch.cuda.is_available():
                self.ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                self.ev[0].record()
            self.t0 = time.perf_counter()
        elif self.calls == self.warmup + self.steps:
            if self.ev is not None:
                self.ev[1].record()
            self.sync()
            self.t1 = time.perf_counter()
            if self.on_stop:
                self.on_stop()
            self.barrier()
        item = self.items[self.calls]
        self.calls += 1
        return item

    def leftover(self):
        from multiprocessing import shared_memory
        for name, *_ in self.items[self.calls:]:
            try:
                s = shared_memory.SharedMemory(name=name)
                s.close()
                s.unlink()
            except FileNotFoundError:
                pass


def run(args, sampler=None) -> int:
    if not os.path.exists(os.path.join(REF, "classes", "student", "model.py")):
        return unavailable("baseline/_ref holds no copy of the reference tree (pip cannot install it: it has neither "
                           "setup.py nor pyproject.toml; copy the tree there)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.model != "tinyllama-1.1b":
        return unavailable(f"the reference arm is set up for tinyllama-1.1b, not {args.model}")
    if os.environ.get("B200_REF_ASYNC") == "1":
        os.environ.pop("CUDA_LAUNCH_BLOCKING", None)
    import torch
    cuda = torch.cuda.is_available()
    arch = dict(TINYLLAMA)
    tiny = os.environ.get("B200_REF_TINY") == "1"           # CPU plumbing check of this file, not a benchmark
    if tiny:
        arch.update(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                    num_key_value_heads=2)
    try:
        notes = _install_stand_ins(local_rank if cuda else None)
        sys.path.insert(0, REF)
        for k in list(sys.modules):          # the reference's packages have generic names (utils, classes)
            if k.split(".")[0] in ("utils", "classes"):
                del sys.modules[k]
        blocking_before = os.environ.get("CUDA_LAUNCH_BLOCKING")
        from classes.student.model import StudentModel
        from classes.data_classes import ConvoTokenized
        from classes.paths import Paths
        if os.environ.get("B200_REF_ASYNC") == "1":
            os.environ.pop("CUDA_LAUNCH_BLOCKING", None)
        if cuda:
            torch.cuda.set_device(local_rank)
    except Exception as e:  # noqa: BLE001
        return unavailable(f"reference import failed: {type(e).__name__}: {e}")
    import numpy as np
    import torch.distributed as dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if cuda else "gloo")
    dev = f"cuda:{local_rank}" if cuda else "cpu"
    B, L, K, W, S = args.micro_batch, args.seq_len, args.topk, args.warmup, args.steps
    vocab = arch["vocab_size"]
    work = os.path.join(os.environ.get("TMPDIR", "/tmp"), f"b200_reference_arm_{os.getpid() if world == 1 else os.environ.get('MASTER_PORT', '0')}")
    model_dir = os.path.join(work, "student")
    clocks: dict = {}
    try:
        if rank == 0:
            _make_model_dir(model_dir, arch, torch.bfloat16 if cuda else torch.float32, dev)
        if world > 1:
            dist.barrier()

        def sync():
            if cuda:
                torch.cuda.synchronize()

        def barrier():
            if world > 1:
                dist.barrier()
        n_batches = W + S + 1
        feeder = Feeder(n_batches, B, L, K, vocab, 100 + rank, W, S, sync, barrier)
        if sampler is not None and rank == 0:
            feeder.on_start, feeder.on_stop = sampler.start, lambda: clocks.update(sampler.stop())
        val_feeder = Feeder(0, B, L, K, vocab, 0, 10 ** 9, 0, sync, barrier)
        paths = Paths(os.path.join(work, f"cache{rank}"), clean_start=True)
        student = StudentModel(model_dir, paths, False, {}, B)
        # ---- collect_and_finetune.set_params / set_training_params, for the benchmark's configuration
        student.crop_to_size, student.context_len, student.temperature, student.device = vocab, L, args.temperature, dev
        rng = np.random.default_rng(7 + rank)
        student.dataset = [ConvoTokenized(rng.integers(0, vocab, L).astype(np.int64), [(0, L)], 0, False, i)
                           for i in range(n_batches * B)]
        student.dataset_len = len(student.dataset)
        student.validation_dataset, student.validation_dataset_len = [], 0
        student.num_epochs = 1
        student.eff_batch_size = 1 * student.batch_size
        student.num_warmup_steps = 0
        student.total_training_steps = student.num_epochs * student.dataset_len
        # "wsd" (the reference's own scheduler class) passes `verbose` to LRScheduler.__init__, which this torch no
        # longer takes; any other name goes to transformers.get_scheduler (utils/finetuning_utils.py:158-170)
        student.lr, student.lr_scheduler_name, student.optimizer_name = 1e-5, "constant", "adamw"
        student.grad_accum = 1
        student.num_grad_accum_batches = -(-student.total_training_steps // student.eff_batch_size)
        student.training_precision_name = "bf16" if cuda else "fp32"
        student.decay_start, student.data_order = 0.9, "native"
        student.multi_gpu, student.device_map_name = True, "auto"          # the path on which accelerate places the model
        student.validation_every_steps = 10 * student.dataset_len
        student.next_val_step = student.validation_every_steps
        student.next_accum_step = student.eff_batch_size
        student.save_every_steps = student.next_save_step = 10 * student.dataset_len
        student.save_final_state, student.grad_checkpointing, student.freeze_layers = False, False, []
        student.use_fa2 = cuda and os.environ.get("B200_REF_ATTN", "fa2") == "fa2"
        student.wandb_comment, student.alpha, student.max_memory, student.num_gpu0_layers = "bench", 2, {}, 0
        student.num_trained_steps = 1           # 0 would start with a validation pass (there is no validation set here)
        if not cuda:
            student.input_device = "cpu"
        attn = "flash_attention_2" if student.use_fa2 else "sdpa"
        try:
            student.train_chunk(feeder, val_feeder, True)
        except Exception as e:  # noqa: BLE001
            if not student.use_fa2 or feeder.calls > 0:
                raise
            notes.append(f"flash_attention_2 refused ({type(e).__name__}: {str(e)[:120]}); ran with sdpa")
            student.use_fa2, attn = False, "sdpa"
            student.train_chunk(feeder, val_feeder, True)
        student.close()
    except Exception as e:  # noqa: BLE001
        import traceback
        traceback.print_exc()
        try:
            feeder.leftover()
        except Exception:  # noqa: BLE001
            pass
        shutil.rmtree(work, ignore_errors=True)
        return unavailable(f"reference run failed: {type(e).__name__}: {e}")
    feeder.leftover()
    if feeder.t1 is None:
        return unavailable("the reference's loop ended before the timed region closed")
    ms = feeder.ev[0].elapsed_time(feeder.ev[1]) if feeder.ev is not None else 1e3 * (feeder.t1 - feeder.t0)
    wall = feeder.t1 - feeder.t0
    if world > 1:
        t = torch.tensor([ms, wall], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, wall = float(t[0]), float(t[1])
    tokens = B * L * world
    if rank == 0:
        out = {
            "metric": "student train tokens/s", "value": tokens * S / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": S, "warmup": W, "ms_per_step": ms / S, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16" if cuda else "fp32",
            "data": "synthetic token ids + synthetic top-K teacher targets, random-init weights", "impl": "reference",
            "config": {"model": args.model if not tiny else "tiny", "global_batch": B * world, "micro_batch_per_gpu": B,
                       "seq_len": L, "topk": K, "attention": attn,
                       "parallelism": "none" if world == 1 else f"{world} independent replicas, no gradient exchange "
                                      "(the reference has no data parallelism): an upper bound",
                       "loss": f"the reference's weighted KL / reverse-KL loss, T={args.temperature}",
                       "optimizer": "adamw via the bitsandbytes stand-in (torch.optim.AdamW fused, bf16 params)",
                       "entry": "StudentModel.train_chunk of the unmodified tree in baseline/_ref",
                       "cuda_launch_blocking": os.environ.get("CUDA_LAUNCH_BLOCKING", "unset"),
                       "stand_ins": notes,
                       "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2) if cuda else None},
            "e2e": {"value": tokens * S / wall, "unit": "tokens/s", "ms_per_step": 1e3 * wall / S,
                    "h2d_bytes_per_step": feeder.h2d_bytes, "d2h_bytes_per_step": 4 * 9,
                    "note": "the reference's loop copies its inputs from host memory and logs its losses every step; "
                            "value and e2e time the same steps (CUDA events / wall clock)"},
            "gpu_launches": None, "clocks": clocks or None,
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        shutil.rmtree(work, ignore_errors=True)
    return 0
