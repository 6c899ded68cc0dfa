"""Configuration: ``config.json`` keys + CLI flags, merged as "CLI value if given, else config value".

Same 44 keys, short flags and grouping as the reference (collect_and_finetune.py:350-433, config.json:1-64).
Differences, all deliberate:
  * boolean flags parse their text (``--use_teachers false`` is False; the reference's ``type=bool`` turns any
    non-empty string into True, collect_and_finetune.py:373-375);
  * ``--reserve_vram 4 0.5`` and ``--max_memory '{"0": "24GB"}'`` work from the command line
    (``type=list`` / ``type=dict`` in the reference do not, :389, :409);
  * the config file path can be given (``--config``); default is ``config.json`` next to the entry script,
    then the packaged default;
  * extra keys for what the reference does not have: parallelism (``tp_size``, ``dp_size``, ``shard_strategy``),
    loss menu (``loss``), cross-tokenizer teachers (``cross_tokenizer``), ``comm_backend``, ``seed``,
    ``interactive``, ``metrics_backend``. Their defaults reproduce the reference's behaviour.
"""
from __future__ import annotations

import argparse
import json
import os
from dataclasses import dataclass, field, fields, asdict
from typing import Any

TRUE_WORDS = {"y", "ye", "yes", "1", "true", "t", "on"}
FALSE_WORDS = {"n", "no", "0", "false", "f", "off", ""}


def str2bool(v: Any) -> bool:
    if isinstance(v, bool):
        return v
    s = str(v).strip().lower()
    if s in TRUE_WORDS:
        return True
    if s in FALSE_WORDS:
        return False
    raise argparse.ArgumentTypeError(f"expected a boolean, got {v!r}")


DEFAULT_PROMPT_FORMAT = {
    "SYS_START": "### System:\n", "USER_START": "### User:\n", "ASSISTANT_START": "### Assistant:\n",
    "SYS_END": "\n", "USER_END": "\n", "ASSISTANT_END": "\n",
}

OPTIMIZERS = ("adam", "adamw", "adamw8bit", "adamw32bit", "paged_adamw", "paged_adamw8bit", "paged_adamw32bit",
              "sgd", "rmsprop", "rmsprop8bit", "rmsprop32bit", "adagrad")
LOSSES = ("reference", "kl", "rkl", "jsd")
PRECISIONS = ("fp32", "fp16", "bf16", "4bit", "8bit")
DATA_ORDERS = ("shuffle", "sorted", "native")


@dataclass
class DistillConfig:
    # ---- paths
    cache_folder: str = "cache"
    dataset_path: str = "train.jsonl"
    validation_dataset_path: str = "val.jsonl"
    teacher_models_folder: str = "teachers"
    student_path: str = "student"
    # ---- cache
    max_cache_size_gb: float = 320
    # ---- pipeline
    ignore_model_type: bool = True
    rebase_dataset: bool = False
    use_teachers: bool = True
    # ---- general model
    context_len: int = 2048
    save_sys_range: bool = True
    save_user_range: bool = True
    save_assistant_range: bool = True
    crop_distr_to_size: int = 32000
    enable_topK: bool = True
    save_topK: int = 400
    device: str = "cuda:0"
    # ---- collection
    num_inference_workers: int = 1
    reserve_vram: list = field(default_factory=lambda: [0.5, 0.5])
    # ---- training
    num_epochs: int = 2
    num_warmup_steps: int = 200
    batch_size: int = 4
    grad_accum_batches: int = 4
    grad_checkpointing: bool = False
    temperature: float = 1.0
    lr: float = 1e-6
    decay_start: float = 0.9
    alpha: float = 2.0
    lr_scheduler: str = "wsd"
    optimizer: str = "adamw8bit"
    data_order: str = "sorted"
    training_precision: str = "4bit"
    validate_every_n_epochs: float = 0.5
    save_student_every_n_epochs: float = 4
    num_gpu0_layers: int = 9
    device_map: str = "custom"
    max_memory: dict = field(default_factory=dict)
    multi_gpu: bool = False
    save_final_state: bool = False
    use_flash_attn_2: bool = True
    wandb_comment: str = "FFT"
    # ---- student
    freeze_layers: list = field(default_factory=lambda: [".block_sparse_moe.gate"])
    add_bos: bool = False
    prompt_format: dict = field(default_factory=lambda: dict(DEFAULT_PROMPT_FORMAT))
    # ---- new in this framework (defaults = reference behaviour)
    loss: str = "reference"            # reference | kl | rkl | jsd
    tp_size: int = 1                   # tensor-parallel width for teacher collection; 0 = the smallest width that fits one GPU
    dp_size: int = 0                   # 0 = world_size / tp_size
    shard_strategy: str = "ddp"        # ddp | fsdp (optimizer state sharded) | zero3 (weights and gradients too) | auto
    comm_backend: str = "p2p"          # p2p (in-kernel NVLink) | nccl
    cross_tokenizer: bool = False      # allow teachers of another vocab family (byte-trie alignment)
    chunked_prefill: str = "auto"      # teacher forward in chunks against a KV cache: true (chunks of the teacher's
                                       # seq_chunk_len, as the reference does) | false | auto (only batches of more
                                       # than prefill_max_tokens tokens, in chunks that keep a pass below that)
    prefill_max_tokens: int = 131072
    vocab_parallel_loss: bool = False  # training: LM head and loss split over the vocabulary across the ranks
    seed: int = 0
    interactive: bool = False          # ask before destructive HDF5 operations / for missing model sidecars
    metrics_backend: str = "jsonl"     # jsonl | wandb | both
    compat_reference_bugs: bool = False

    REFERENCE_KEYS = (
        "max_cache_size_gb", "cache_folder", "dataset_path", "validation_dataset_path", "teacher_models_folder",
        "student_path", "ignore_model_type", "rebase_dataset", "use_teachers", "context_len", "save_sys_range",
        "save_user_range", "save_assistant_range", "crop_distr_to_size", "enable_topK", "save_topK", "device",
        "num_inference_workers", "reserve_vram", "num_epochs", "num_warmup_steps", "batch_size",
        "grad_accum_batches", "grad_checkpointing", "temperature", "lr", "decay_start", "alpha", "lr_scheduler",
        "optimizer", "data_order", "training_precision", "validate_every_n_epochs", "save_student_every_n_epochs",
        "num_gpu0_layers", "device_map", "max_memory", "multi_gpu", "save_final_state", "use_flash_attn_2",
        "wandb_comment", "freeze_layers", "add_bos", "prompt_format")

    def validate(self) -> "DistillConfig":
        if self.optimizer.lower() not in OPTIMIZERS:
            raise ValueError(f"Invalid optimizer name: {self.optimizer}\nAvailable optimizers: {list(OPTIMIZERS)}")
        if self.loss.lower() not in LOSSES:
            raise ValueError(f"Invalid loss: {self.loss}; choose from {LOSSES}")
        if self.training_precision.lower() not in PRECISIONS:
            raise ValueError(f"Invalid training_precision: {self.training_precision}; choose from {PRECISIONS}")
        if self.data_order.lower() not in DATA_ORDERS:
            raise ValueError(f"Invalid data_order: {self.data_order}; choose from {DATA_ORDERS}")
        if self.shard_strategy not in ("ddp", "fsdp", "zero3", "auto"):
            raise ValueError("shard_strategy must be ddp, fsdp, zero3 or auto")
        self.chunked_prefill = str(self.chunked_prefill).lower()
        if self.chunked_prefill not in ("true", "false", "auto"):
            raise ValueError("chunked_prefill must be true, false or auto")
        if self.comm_backend not in ("p2p", "nccl"):
            raise ValueError("comm_backend must be p2p or nccl")
        if self.context_len <= 0 or self.batch_size <= 0 or self.grad_accum_batches <= 0:
            raise ValueError("context_len, batch_size and grad_accum_batches must be positive")
        if self.enable_topK and 0 < self.crop_distr_to_size < self.save_topK:
            print(f"save_topK ({self.save_topK}) exceeds crop_distr_to_size ({self.crop_distr_to_size}): keeping "
                  f"{self.crop_distr_to_size} values per token")
            self.save_topK = int(self.crop_distr_to_size)
        if self.enable_topK and self.save_topK <= 0:
            raise ValueError("save_topK must be positive when enable_topK is set")
        if self.temperature <= 0:
            raise ValueError("temperature must be positive")
        missing = [k for k in DEFAULT_PROMPT_FORMAT if k not in self.prompt_format]
        if missing:
            raise ValueError(f"prompt_format lacks {missing}")
        return self

    def to_dict(self) -> dict:
        return asdict(self)


def load_config(config_path: str) -> dict:
    """Same contract as the reference (collect_and_finetune.py:342-346): the file must exist."""
    if not os.path.exists(config_path):
        raise FileNotFoundError(
            f"Config file not found at {config_path}!\nPlease make sure the file exists, and has all the necessary parameters.")
    with open(config_path, "r", encoding="utf-8") as f:
        return json.load(f)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Offline logit distillation: collect teacher distributions, then finetune "
                                            "the student.", formatter_class=argparse.RawTextHelpFormatter)
    p.add_argument("--config", type=str, default=None, help="Path to config.json (default: next to the entry script).")
    g = p.add_argument_group("Path args")
    g.add_argument("--cache_folder", "-c", type=str, help="Directory for cache storage. {string}")
    g.add_argument("--dataset_path", "-d", type=str, help="Path to the training dataset (JSONL). {string}")
    g.add_argument("--validation_dataset_path", "-vd", type=str, help="Path to the validation dataset. {string}")
    g.add_argument("--teacher_models_folder", "-tm", type=str,
                   help="Directory containing teacher models, or a path to one teacher. {string}")
    g.add_argument("--student_path", "-s", type=str, help="Path to the student model. {string}")
    g = p.add_argument_group("Cache args")
    g.add_argument("--max_cache_size_gb", "-maxgb", type=float,
                   help="Maximum size of the main HDF5 dataset in GB; above it, collection and training alternate in chunks. {float}")
    g = p.add_argument_group("Pipeline args")
    g.add_argument("--ignore_model_type", type=str2bool, help="Let completion teachers collect instruct data and vice versa. {bool}")
    g.add_argument("--rebase_dataset", type=str2bool, help="Overwrite the HDF5 metadata from the current text dataset without checks. {bool}")
    g.add_argument("--use_teachers", type=str2bool, help="False: train from an existing HDF5 dataset without teacher models. {bool}")
    g = p.add_argument_group("General model args")
    g.add_argument("--context_len", "-ctx", type=int, help="Context length to collect and train on. {int}")
    g.add_argument("--save_sys_range", type=str2bool, help="Collect/train on system-prompt content tokens. {bool}")
    g.add_argument("--save_user_range", type=str2bool, help="Collect/train on user-turn content tokens. {bool}")
    g.add_argument("--save_assistant_range", type=str2bool, help="Collect/train on assistant-turn content tokens. {bool}")
    g.add_argument("--crop_distr_to_size", type=int, help="distributions[:, :crop_distr_to_size]; set to the base vocabulary size. {int}")
    g.add_argument("--enable_topK", type=str2bool, help="Store only the top-K teacher log-probs. {bool}")
    g.add_argument("--save_topK", "-topk", type=int, help="K for top-K storage (giving it enables top-K). {int}")
    g.add_argument("--device", type=str, help="Main device for single-device work (e.g. cuda:0). {string}")
    g = p.add_argument_group("Data collection args")
    g.add_argument("--num_inference_workers", "-niw", type=int, help="Teacher replicas collecting in parallel. {int}")
    g.add_argument("--reserve_vram", type=float, nargs="+", help="GB to keep free per GPU during collection. {float list}")
    g = p.add_argument_group("Training args")
    g.add_argument("--num_epochs", "-ne", type=int)
    g.add_argument("--num_warmup_steps", "-nws", type=int, help="Warm-up length in samples. {int}")
    g.add_argument("--batch_size", "-bs", type=int)
    g.add_argument("--grad_accum_batches", "-g", type=int)
    g.add_argument("--grad_checkpointing", type=str2bool)
    g.add_argument("--temperature", "-t", type=float)
    g.add_argument("--lr", "-lr", type=float)
    g.add_argument("--decay_start", type=float, help="wsd: fraction of optimizer steps before the linear decay. {float}")
    g.add_argument("--alpha", type=float, help="weights = ((kl / kl.max()) + 1) ** alpha in the reference loss. {float}")
    g.add_argument("--lr_scheduler", type=str, help="wsd, cosine, linear, constant, constant_with_warmup. {string}")
    g.add_argument("--optimizer", type=str, help="One of: " + ", ".join(OPTIMIZERS))
    g.add_argument("--data_order", type=str, help="shuffle | sorted | native")
    g.add_argument("--training_precision", type=str, help="fp32 | fp16 | bf16 | 4bit | 8bit")
    g.add_argument("--validate_every_n_epochs", type=float)
    g.add_argument("--save_student_every_n_epochs", type=float)
    g.add_argument("--num_gpu0_layers", type=int)
    g.add_argument("--device_map", type=str)
    g.add_argument("--max_memory", type=json.loads, help='JSON dict, e.g. \'{"0": "24GB", "cpu": "200GB"}\'')
    g.add_argument("--multi_gpu", type=str2bool)
    g.add_argument("--save_final_state", type=str2bool)
    g.add_argument("--wandb_comment", "-wdb", type=str)
    g.add_argument("--use_flash_attn_2", "-fa2", type=str2bool)
    g = p.add_argument_group("Student args")
    g.add_argument("--freeze_layers", "-fl", type=str, nargs="+")
    g.add_argument("--add_bos", type=str2bool)
    g.add_argument("--prompt_format", type=json.loads)
    g = p.add_argument_group("Parallelism / loss (new)")
    g.add_argument("--loss", type=str, help="reference | kl | rkl | jsd")
    g.add_argument("--tp_size", type=int, help="tensor-parallel width of the teachers; 0 = smallest width that fits 180 GB per GPU")
    g.add_argument("--dp_size", type=int, help="data-parallel replicas of the teacher; 0 = ranks / tp_size")
    g.add_argument("--shard_strategy", type=str, help="student sharding: ddp (replicated weights) | fsdp (optimizer state sharded) | "
                   "zero3 (weights, gradients and state sharded) | auto (first plan that fits 180 GB per GPU)")
    g.add_argument("--comm_backend", type=str, help="p2p (NVLink peer-access kernels) | nccl (library collectives)")
    g.add_argument("--cross_tokenizer", type=str2bool)
    g.add_argument("--chunked_prefill", type=str, help="true | false | auto")
    g.add_argument("--prefill_max_tokens", type=int)
    g.add_argument("--vocab_parallel_loss", type=str2bool)
    g.add_argument("--seed", type=int)
    g.add_argument("--interactive", type=str2bool)
    g.add_argument("--metrics_backend", type=str)
    g.add_argument("--compat_reference_bugs", type=str2bool)
    return p


def merge(config: dict, args: argparse.Namespace) -> DistillConfig:
    """CLI value if not None else config value (collect_and_finetune.py:426); unknown config keys are rejected."""
    known = {f.name for f in fields(DistillConfig)}
    unknown = [k for k in config if k not in known]
    if unknown:
        raise KeyError(f"Unknown config keys: {unknown}")
    params: dict[str, Any] = {}
    for name in known:
        cli = getattr(args, name, None)
        if cli is not None:
            params[name] = cli
        elif name in config:
            params[name] = config[name]
    if getattr(args, "save_topK", None) is not None:
        params["enable_topK"] = True  # collect_and_finetune.py:428-429
    mm = params.get("max_memory") or {}
    params["max_memory"] = {int(k): v for k, v in mm.items() if str(k).lower() != "cpu"}  # :431
    for key in ("ignore_model_type", "rebase_dataset", "use_teachers", "save_sys_range", "save_user_range",
                "save_assistant_range", "enable_topK", "grad_checkpointing", "multi_gpu", "save_final_state",
                "use_flash_attn_2", "add_bos"):
        if key in params:
            params[key] = str2bool(params[key])
    return DistillConfig(**params).validate()


def get_params(argv: list[str] | None = None, default_config_path: str | None = None) -> DistillConfig:
    args = build_parser().parse_args(argv)
    path = args.config or default_config_path or os.path.join(os.getcwd(), "config.json")
    return merge(load_config(path), args)
