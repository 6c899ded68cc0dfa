"""Entry point: collect teacher distributions, then finetune the student (reference: collect_and_finetune.py).

    python -m llm_distillery_b200.cli --config config.json [flags]
    torchrun --nproc-per-node 8 -m llm_distillery_b200.cli --config config.json      (data-parallel ranks)

Flow (same order as the reference's ``main``): parameters -> signal handlers -> cache tree -> teachers + student ->
two HDF5 stores (train / validation) -> vocabulary compatibility -> tokenisation -> hyper-parameter fan-out ->
data order -> chunk plan -> SHA sync of the stores -> validation collection -> one of: full collect then train;
chunked collect/train per epoch; train from the data on disk.
"""
from __future__ import annotations

import math
import os
import signal
import sys

from .config import DistillConfig, get_params
from .data import plan
from .data.h5store import H5Store
from .data.sync import sync_datasets
from .data.tokenize import tokenize_dataset
from .models.student import StudentModel
from .models.teacher import TeacherModel
from .obs.console import progress
from .paths import Paths

_STATE = {"data_manager": None, "validation_data_manager": None, "teachers": None, "student": None}


def get_teachers(models_folder: str, use_teachers: bool, interactive: bool = False) -> list[TeacherModel]:
    """One teacher if the folder itself holds model files, else one per sub-folder (collect_and_finetune.py:55-80)."""
    if not use_teachers:
        return []
    entries = sorted(os.listdir(models_folder))
    if any(f.endswith((".bin", ".json", ".safetensors")) for f in entries):
        return [TeacherModel(models_folder, interactive=interactive)]
    paths = [os.path.join(models_folder, n) for n in entries if os.path.isdir(os.path.join(models_folder, n))]
    if not paths:
        print("No models found in the teacher models folder!")
        raise SystemExit(0)
    return [TeacherModel(p, interactive=interactive) for p in paths]


def ensure_compatibility(teachers, student, use_teachers: bool, cross_tokenizer: bool = False) -> None:
    """All teachers and the student must share one vocabulary family (collect_and_finetune.py:83-101), unless
    cross-tokenizer alignment is enabled: then teachers of another family are mapped onto the student's
    vocabulary by the byte-trie aligner."""
    if not use_teachers or not teachers:
        return
    first = teachers[0]
    for t in teachers:
        t.needs_alignment = t.vocab_id != student.vocab_id
        if cross_tokenizer:
            continue
        if t.vocab_id != first.vocab_id:
            raise ValueError(f"Teacher {t.model_name} has vocab_family={t.vocab_family} while the first teacher has "
                             f"vocab_family={first.vocab_family}")
    if not cross_tokenizer and student.vocab_id != first.vocab_id:
        raise ValueError(f"Student has vocab_family = {student.vocab_family} while the teachers have "
                         f"vocab_family = {first.vocab_family}")


def prepare_datasets(cfg: DistillConfig, data_manager, validation_data_manager, teachers, student) -> None:
    print("Preparing datasets for the student...")
    all_not_add_bos = (not student.add_bos) and all(not t.add_bos for t in teachers)
    args = (cfg.context_len, cfg.save_sys_range, cfg.save_user_range, cfg.save_assistant_range)
    has_val = bool(cfg.validation_dataset_path)       # the reference requires a validation set; here "" = train without one

    def tokenize_val(model):
        if not has_val:
            return [], set()
        return tokenize_dataset(cfg.validation_dataset_path, *args, model, cfg.ignore_model_type, all_not_add_bos)
    student.dataset, ids = tokenize_dataset(cfg.dataset_path, *args, student, cfg.ignore_model_type, all_not_add_bos)
    student.validation_dataset, ids_val = tokenize_val(student)
    t_ids, t_ids_val = set(), set()
    for t in teachers:
        print(f"Preparing datasets for {t.model_name}...")
        t.dataset, a = tokenize_dataset(cfg.dataset_path, *args, t, cfg.ignore_model_type, all_not_add_bos)
        t.validation_dataset, b = tokenize_val(t)
        t_ids |= a
        t_ids_val |= b
    if cfg.use_teachers:
        common, common_val = ids & t_ids, ids_val & t_ids_val
    else:
        common, common_val = set(data_manager.get_dataset_ids()), set(validation_data_manager.get_dataset_ids())
    student.dataset = [c for c in student.dataset if c.origin_convo_id in common]
    student.dataset_len = len(student.dataset)
    print(f"Total tokens in dataset: {sum(c.length for c in student.dataset)}; "
          f"Content tokens: {sum(c.len_content for c in student.dataset)}")
    student.validation_dataset = [c for c in student.validation_dataset if c.origin_convo_id in common_val]
    student.validation_dataset_len = len(student.validation_dataset)
    print(f"Total tokens in validation dataset: {sum(c.length for c in student.validation_dataset)}; "
          f"Content tokens: {sum(c.len_content for c in student.validation_dataset)}")
    for t in teachers:
        t.dataset = [c for c in t.dataset if c.origin_convo_id in common]
        t.dataset_len = len(t.dataset)
        t.validation_dataset = [c for c in t.validation_dataset if c.origin_convo_id in common_val]
        t.validation_dataset_len = len(t.validation_dataset)


def set_params(teachers, student, cfg: DistillConfig) -> None:
    for t in teachers:
        t.crop_to_size, t.context_len, t.temperature = cfg.crop_distr_to_size, cfg.context_len, cfg.temperature
        t.device, t.topK, t.enable_topK = cfg.device, cfg.save_topK, cfg.enable_topK
        t.chunked_prefill, t.prefill_max_tokens = cfg.chunked_prefill, int(cfg.prefill_max_tokens)
    student.crop_to_size, student.context_len = cfg.crop_distr_to_size, cfg.context_len
    student.temperature, student.device = cfg.temperature, cfg.device


def set_training_params(student: StudentModel, cfg: DistillConfig) -> None:
    """All step counts are in samples; warm-up is converted to optimizer steps (collect_and_finetune.py:178-208).
    With W data-parallel ranks one optimizer step covers grad_accum * batch_size * W samples."""
    student.num_epochs = cfg.num_epochs
    student.eff_batch_size = cfg.grad_accum_batches * student.batch_size * student.world
    student.num_warmup_steps = math.ceil(cfg.num_warmup_steps / student.eff_batch_size)
    student.total_training_steps = cfg.num_epochs * student.dataset_len
    student.lr = cfg.lr
    student.lr_scheduler_name = cfg.lr_scheduler.lower()
    student.optimizer_name = cfg.optimizer.lower()
    student.grad_accum = cfg.grad_accum_batches
    student.num_grad_accum_batches = math.ceil(student.total_training_steps / student.eff_batch_size)
    student.training_precision_name = cfg.training_precision.lower()
    student.vocab_parallel_loss = bool(cfg.vocab_parallel_loss) and student.world > 1
    student.decay_start = cfg.decay_start
    student.multi_gpu = cfg.multi_gpu
    student.data_order = cfg.data_order.lower()
    student.validation_every_steps = cfg.validate_every_n_epochs * student.dataset_len
    student.next_accum_step = student.eff_batch_size
    student.save_every_steps = cfg.save_student_every_n_epochs * student.dataset_len
    student.next_save_step = cfg.save_student_every_n_epochs * student.dataset_len
    student.save_final_state = cfg.save_final_state
    student.grad_checkpointing = cfg.grad_checkpointing
    student.freeze_layers = cfg.freeze_layers
    student.use_fa2 = cfg.use_flash_attn_2
    student.wandb_comment = cfg.wandb_comment
    student.alpha = cfg.alpha
    student.device_map_name = cfg.device_map
    student.max_memory = cfg.max_memory
    student.num_gpu0_layers = cfg.num_gpu0_layers
    student.loss_kind = cfg.loss.lower()
    student.metrics_backend = cfg.metrics_backend
    student.seed = cfg.seed


def check_topk(data_manager, enable_topk: bool, save_topk: int, validation: bool = False, interactive: bool = False):
    """Reconcile the configured K with the K the file was collected with (collect_and_finetune.py:318-339). Without a
    terminal to ask, the file's K wins (collected data cannot change its K)."""
    if not enable_topk:
        return save_topk
    dataset_topk = data_manager.get_topk()
    if dataset_topk is None:
        data_manager.set_topk(save_topk)
        return save_topk
    if dataset_topk != save_topk:
        which = "validation" if validation else "main"
        print(f"\nTopK mismatch between the {which} h5 dataset, and your config!\n{which.upper()} dataset has "
              f"TopK={dataset_topk}, while you set TopK={save_topk}.")
        if interactive:
            ans = input("Do you wish to continue with the dataset's TopK?\nIf not, the program will exit to allow you "
                        "to change the config. (y/n): ")
            if ans.lower() not in ("y", "ye", "yes", "1", "true", "t"):
                handle_termination(None, None)
        return dataset_topk
    return save_topk


def handle_termination(signum, frame) -> None:
    student = _STATE.get("student")
    if (signum is not None and student is not None and getattr(student, "training_active", False)
            and not getattr(student, "stop_requested", False)):
        # in the middle of training: finish the step, save the trainer state (all ranks together), then leave; a
        # second signal ends the process at once
        student.stop_requested = True
        print("\nStop requested: the run ends after the current step with its state saved "
              "(signal again to end it at once).", flush=True)
        return
    print("\nTerminating the script...")
    for key in ("data_manager", "validation_data_manager"):
        dm = _STATE.get(key)
        if dm is not None:
            try:
                dm.close()
            except Exception as e:  # noqa: BLE001
                print(f"closing {key}: {e}")
    for t in _STATE.get("teachers") or []:
        t.close()
    if _STATE.get("student") is not None:
        _STATE["student"].close()
    if _STATE.get("heartbeat") is not None:
        _STATE["heartbeat"].close("done")
        _STATE["heartbeat"] = None
    if signum is not None:
        os._exit(0)


def resolve_shard_strategy(cfg: DistillConfig, world: int) -> str:
    """``shard_strategy = auto``: the first of replicated weights, full sharding, full sharding + gradient checkpointing
    whose estimated footprint fits one GPU (``parallel.memory``); the config is updated in place (also
    ``grad_checkpointing`` when the plan needs it). Other values pass through."""
    if cfg.shard_strategy != "auto":
        return cfg.shard_strategy
    from .models.llama import LlamaConfig
    from .parallel import memory
    try:
        mcfg = LlamaConfig.from_pretrained(cfg.student_path)
    except (OSError, ValueError, NotImplementedError, KeyError):
        cfg.shard_strategy = "ddp"
        return cfg.shard_strategy
    tokens = int(cfg.batch_size) * int(cfg.context_len)
    pick, table = memory.recommend(mcfg, world, tokens, topk=int(cfg.save_topK) if cfg.enable_topK else 200,
                                   optimizer=cfg.optimizer, grad_checkpointing=bool(cfg.grad_checkpointing))
    if pick == "none":
        pick = "zero3+checkpointing" if world > 1 else "ddp+checkpointing"
        print("shard_strategy auto: no plan is estimated to fit 180 GB per GPU; using the smallest one")
    cfg.shard_strategy = pick.split("+")[0]
    if "checkpointing" in pick:
        cfg.grad_checkpointing = True
    fp = table.get(pick) or next(iter(table.values()))
    print(f"shard_strategy auto -> {cfg.shard_strategy}" + (" with grad_checkpointing" if "checkpointing" in pick else "") +
          f" (estimated {fp.total_gb:.0f} GB per GPU)")
    return cfg.shard_strategy


def _init_distributed(cfg: DistillConfig):
    """(rank, world, communicator) - communicator is None for a single process."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    resolve_shard_strategy(cfg, world)
    if world == 1:
        return 0, 1, None
    import torch
    import torch.distributed as dist
    rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", "0"))
    cuda = cfg.device.startswith("cuda") and torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
        cfg.device = f"cuda:{local}"
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if cuda else "gloo")
    from .parallel.ddp import make_comm
    kind = cfg.comm_backend if cuda else "gloo"
    return rank, world, make_comm(kind, torch.device(cfg.device), shard_strategy=cfg.shard_strategy)


def refresh_stores(rank: int, world: int, *stores) -> None:
    """Rank 0 is the only writer of the HDF5 files: make its writes visible to the other ranks' handles."""
    if world == 1:
        return
    import torch.distributed as dist
    if rank == 0:
        for st in stores:
            st.wait()
            st.flush()
    dist.barrier()
    if rank != 0:
        for st in stores:
            st.reopen()
    dist.barrier()


_TP_GROUPS: dict = {}


def _tp_group(cfg, teacher, rank: int, world: int, tp: int):
    """The tensor-parallel group of this rank (consecutive ranks), with symmetric buffers sized for the teacher's
    largest batch. Process groups are created once (every rank takes part in every ``new_group`` call)."""
    import torch
    import torch.distributed as dist
    from .models.llama import LlamaConfig
    from .parallel.tp import TPGroup, padded_seq_len
    if "pg" not in _TP_GROUPS:
        if tp == world:
            _TP_GROUPS["pg"] = dist.group.WORLD
        else:
            mine = None
            for g0 in range(0, world, tp):
                pg = dist.new_group(list(range(g0, g0 + tp)))
                if g0 <= rank < g0 + tp:
                    mine = pg
            _TP_GROUPS["pg"] = mine
    mcfg = LlamaConfig.from_pretrained(teacher.model_path)
    B = max(1, teacher.batch_size)
    # a teacher with another tokenizer can spell the same text in more tokens than the student's context length
    longest = max([int(cfg.context_len)] + [int(c.length) for ds in (getattr(teacher, "dataset", None),
                                                                      getattr(teacher, "validation_dataset", None))
                                            for c in (ds or [])])
    # the last batch of a share can hold fewer conversations, and an odd count pads each of them further
    tokens = max(b * padded_seq_len(b, longest, tp) for b in range(1, B + 1))
    key = (mcfg.hidden_size, tokens, int(teacher.topK))
    if key not in _TP_GROUPS:
        _TP_GROUPS[key] = TPGroup(torch.device(cfg.device), tokens, mcfg.hidden_size, topk=int(teacher.topK),
                                  group=_TP_GROUPS["pg"], dtype=torch.float32)
    return _TP_GROUPS[key]


def resolve_tp_size(cfg, teachers, world: int) -> int:
    """``tp_size`` > 0 is taken as given (capped at the number of ranks); 0 = the smallest width at which every teacher
    fits one GPU (``parallel.memory.recommend_tp``) - the remaining ranks become data-parallel replicas."""
    if int(cfg.tp_size) > 0 or world <= 1:
        return max(1, min(int(cfg.tp_size), world))
    cached = getattr(cfg, "_tp_auto", None)
    if cached:
        return cached
    from .models.llama import LlamaConfig
    from .parallel import memory
    cfgs = []
    for t in teachers:
        try:
            cfgs.append(LlamaConfig.from_pretrained(t.model_path))
        except (OSError, ValueError, NotImplementedError, KeyError):
            pass
    tokens = int(cfg.context_len) * max([int(getattr(t, "batch_size", 1) or 1) for t in teachers] or [1])
    tp = memory.recommend_tp(cfgs, world, tokens, int(cfg.save_topK) if cfg.enable_topK else 200,
                             int(cfg.crop_distr_to_size) or None) if cfgs else 1
    print(f"tp_size auto -> {tp} ({world // tp} data-parallel replica(s) of a {tp}-way tensor-parallel teacher)")
    cfg._tp_auto = tp
    return tp


def collect(teachers, cfg, store, ids, validation, rank, world, student=None) -> None:
    """Every teacher in turn collects ``ids`` into ``store`` (teachers after the first merge into the same
    conversations). With several ranks each rank collects a strided share into its own shard file and rank 0
    folds the shards into the main file."""
    if not ids:
        return
    target = store
    shas = None
    if student is not None:
        shas = {c.origin_convo_id: c.content_sha for c in (student.validation_dataset if validation else student.dataset)}
    tp = resolve_tp_size(cfg, teachers, world)
    if world % tp:
        raise ValueError(f"tp_size={tp} must divide the number of ranks ({world})")
    dp_rank, dp_world = rank // tp, world // tp
    if int(getattr(cfg, "dp_size", 0) or 0) not in (0, dp_world):
        raise ValueError(f"dp_size={cfg.dp_size} x tp_size={tp} does not match the {world} ranks of this run")
    if world > 1:
        shard_path = store.file_path.replace(".hdf5", f".rank{rank}.hdf5")
        if os.path.exists(shard_path):       # left behind by a run that was killed mid-collection: its rows are not
            os.remove(shard_path)            # this run's, and folding them again would count their teachers twice
        target = H5Store(shard_path)
    from .data.convo import PARTIAL_SHA_PREFIX
    for k, t in enumerate(progress(teachers, desc="Teachers", leave=False, disable=len(teachers) == 1)):
        tp_group = _tp_group(cfg, t, rank, world, tp) if tp > 1 else None
        t.process_chunk(cfg.reserve_vram, cfg.num_inference_workers, ids_to_collect=ids, data_manager=target,
                        validation=validation, rank=dp_rank, world=dp_world, sha_by_id=shas, tp_group=tp_group,
                        last_teacher=(k + 1 == len(teachers)))
        t.unload()

    def finalize(st) -> None:
        """Every teacher is through: a conversation the last teacher had no rows for still carries the mark."""
        marked = {cid: sha[len(PARTIAL_SHA_PREFIX):] for cid, sha in st.get_available_shas().items()
                  if sha.startswith(PARTIAL_SHA_PREFIX)}
        if marked:
            st.update_shas(marked)
            st.flush()
    if world == 1:
        finalize(store)
    if world > 1:
        import torch.distributed as dist
        target.close()
        dist.barrier()
        if rank == 0:
            from .data.convo import TeacherRows
            seen: set[int] = set()
            for r in range(world):
                shard_path = store.file_path.replace(".hdf5", f".rank{r}.hdf5")
                shard = H5Store(shard_path)
                for cid in shard.get_dataset_ids():
                    v, ix = shard.load_id(cid)
                    sha = shard.get_sha(cid) or ""
                    if sha.startswith(PARTIAL_SHA_PREFIX):     # all teachers are through by now: the mark comes off
                        sha = sha[len(PARTIAL_SHA_PREFIX):]
                    rows = [TeacherRows(cid, v, ix, sha, shard._attr(cid, "sample") or "")]
                    # teachers batch the conversations differently, so one conversation can sit in several ranks' files,
                    # each holding other teachers' rows: the first one replaces what the main file had, the others merge
                    (store.write_batch if cid in seen else store.update_batch)(rows)
                    seen.add(cid)
                shard.close()
                os.remove(shard_path)
                store.wait()            # a replace must have landed before a later shard merges into it
        dist.barrier()


def _leave_after_rank_failure(e) -> None:
    """Emergency exit of a surviving rank: trainer state of this rank without any collective, stores closed, status 3."""
    print(f"[watchdog] {e}: saving state and leaving", flush=True)
    student, hb = _STATE.get("student"), _STATE.get("heartbeat")
    if student is not None and getattr(student, "engine", None) is not None:
        try:
            student._save_state(collective=False)
        except Exception as ex:  # noqa: BLE001
            print(f"[watchdog] emergency save failed: {ex}", flush=True)
    if hb is not None:
        hb.close("failed")
    for key in ("data_manager", "validation_data_manager"):
        if _STATE.get(key) is not None:
            try:
                _STATE[key].close()
            except Exception:  # noqa: BLE001
                pass
    os._exit(3)


def main(argv=None, default_config_path: str | None = None) -> dict:
    """Run the pipeline. With several ranks a heartbeat / watchdog pair runs beside it: when a peer stops beating,
    the surviving ranks find out between two steps, save their trainer state without any collective and exit with
    status 3; running the same command again resumes (SHA sync for collection, trainer state for training).

    A peer that leaves just before a collective is usually noticed the other way round: the collective ends with an
    error before the heartbeat record is old enough. A RuntimeError / OSError under several ranks (what collectives and
    device-side waits raise) is therefore followed by a look at the heartbeats (for as long as a record takes to go stale): if a peer is gone, the exception is its
    consequence and the rank leaves the same way; if every peer is alive, the exception is this rank's own."""
    import time
    from .obs import watchdog
    from .models.student import StopRequested
    try:
        return _main(argv, default_config_path)
    except StopRequested:
        student = _STATE.get("student")
        summary = {"stopped": True, "trained_samples": getattr(student, "num_trained_steps", 0)}
        handle_termination(None, None)
        return summary
    except watchdog.RankFailure as e:
        _leave_after_rank_failure(e)
    except (RuntimeError, OSError, TimeoutError) as ex:       # what a collective or a device-side wait raises
        hb = _STATE.get("heartbeat")
        if hb is None:
            raise
        deadline = time.time() + hb.timeout + 3 * hb.interval + 1.0
        failed = hb.scan()
        while not failed and time.time() < deadline:
            time.sleep(hb.interval)
            failed = hb.scan()
        if not failed:
            raise
        ranks = sorted(failed)
        _leave_after_rank_failure(watchdog.RankFailure(
            ranks, "; ".join(f"rank {k}: {failed[k]}" for k in ranks) + f" (seen as {type(ex).__name__}: {str(ex)[:200]})"))


def _main(argv=None, default_config_path: str | None = None) -> dict:
    from .obs import watchdog
    cfg = get_params(argv, default_config_path)
    rank, world, comm = _init_distributed(cfg)
    def _escalate(failed):      # watchdog thread: the main thread is stuck (e.g. inside a collective with a dead peer)
        print(f"[watchdog] {failed}; the main thread did not return from its step: leaving without a state save "
              f"(the last checkpoint and the HDF5 cache stay valid)", flush=True)
        os._exit(3)

    stall = os.environ.get("B200_STALL_TIMEOUT")
    heartbeat = watchdog.from_env(rank, world, timeout=float(os.environ.get("B200_HEARTBEAT_TIMEOUT", "60")),
                                  stall_timeout=float(stall) if stall else None, on_failure=_escalate)
    _STATE["heartbeat"] = heartbeat

    signal.signal(signal.SIGTERM, handle_termination)
    signal.signal(signal.SIGINT, handle_termination)

    paths = Paths(cfg.cache_folder)
    teachers = get_teachers(cfg.teacher_models_folder, cfg.use_teachers, cfg.interactive)
    student = StudentModel(cfg.student_path, paths, cfg.add_bos, cfg.prompt_format, cfg.batch_size, cfg.interactive)
    student.comm, student.rank, student.world = comm, rank, world
    student.heartbeat = heartbeat
    for t in teachers:
        t.heartbeat = heartbeat
    print("Opening data stores...")
    def open_stores():
        return (H5Store(paths.dataset, cfg.device, manager_name="main", interactive=cfg.interactive),
                H5Store(paths.dataset_validation, cfg.device, manager_name="validation", interactive=cfg.interactive))
    if world > 1:       # rank 0 creates missing files; the others open them only once they are complete
        import torch.distributed as dist
        if rank == 0:
            data_manager, validation_data_manager = open_stores()
        dist.barrier()
        if rank != 0:
            data_manager, validation_data_manager = open_stores()
    else:
        data_manager, validation_data_manager = open_stores()
    _STATE.update(data_manager=data_manager, validation_data_manager=validation_data_manager, teachers=teachers,
                  student=student)

    ensure_compatibility(teachers, student, cfg.use_teachers, cfg.cross_tokenizer)
    prepare_datasets(cfg, data_manager, validation_data_manager, teachers, student)
    set_params(teachers, student, cfg)
    set_training_params(student, cfg)
    if cfg.cross_tokenizer:
        from .align.aligner import attach_aligners
        attach_aligners(teachers, student)
    student.reorder_dataset()
    loop_ids, full_collect = plan.calculate_loop_ids(student.dataset, cfg.max_cache_size_gb, cfg.enable_topK,
                                                     cfg.save_topK, cfg.crop_distr_to_size)
    if rank == 0:
        ids_collect, ids_collect_val = sync_datasets(validation_data_manager, data_manager, cfg.rebase_dataset, student,
                                                     cfg.use_teachers)
    else:
        ids_collect, ids_collect_val = [], []
    if world > 1:
        import torch.distributed as dist
        box = [ids_collect, ids_collect_val]
        dist.broadcast_object_list(box, src=0)
        ids_collect, ids_collect_val = box

    if ids_collect_val and not cfg.rebase_dataset:
        print(f"Collecting validation data for {len(ids_collect_val)} samples...")
        k = check_topk(validation_data_manager, cfg.enable_topK, cfg.save_topK, validation=True, interactive=cfg.interactive)
        for t in teachers:
            t.topK = k
        if rank == 0:
            validation_data_manager.set_vocab_family(student.vocab_family)
        collect(teachers, cfg, validation_data_manager, ids_collect_val, True, rank, world, student)
    else:
        print("Using data on disk for validation...")

    if ids_collect and not cfg.rebase_dataset:
        if rank == 0:
            data_manager.set_vocab_family(student.vocab_family)
        if full_collect:
            print(f"Collecting data for {len(ids_collect)} samples...")
            k = check_topk(data_manager, cfg.enable_topK, cfg.save_topK, interactive=cfg.interactive)
            for t in teachers:
                t.topK = k
            collect(teachers, cfg, data_manager, ids_collect, False, rank, world, student)
            refresh_stores(rank, world, data_manager, validation_data_manager)
            student.train_chunk(data_manager, validation_data_manager, full_collect)
        else:
            print(f"WARNING: The calculated size of the h5 dataset is too large for the specified cache size "
                  f"({cfg.max_cache_size_gb}GB).\nThe data will be collected and trained on in chunks.")
            if data_manager.has_data() and cfg.interactive:
                print("This will erase all previous data in the main h5 dataset!")
                if input("Do you wish to continue? (y/n): ").lower() not in ("y", "ye", "yes", "1", "true", "t"):
                    handle_termination(None, None)
                    return {}
            if rank == 0:
                data_manager.set_topk(cfg.save_topK)
            for _ in progress(range(cfg.num_epochs), desc="Epochs"):
                for chunk_ids in progress(loop_ids, desc="Chunks", leave=False):
                    if rank == 0:
                        data_manager.purge_dataset(ask_confirmation=False)
                        data_manager.set_topk(cfg.save_topK)
                        data_manager.set_vocab_family(student.vocab_family)
                    collect(teachers, cfg, data_manager, chunk_ids, False, rank, world, student)
                    refresh_stores(rank, world, data_manager, validation_data_manager)
                    student.train_chunk(data_manager, validation_data_manager, full_collect)
    else:
        print("Using data on disk for training...")
        refresh_stores(rank, world, data_manager, validation_data_manager)
        student.train_chunk(data_manager, validation_data_manager, True)

    print("Done!")
    summary = {"trained_samples": student.num_trained_steps, "tokens_trained": student.tokens_trained,
               "train_seconds": student.train_seconds,
               "tokens_collected": sum(t.tokens_collected for t in teachers),
               "collect_seconds": sum(t.collect_seconds for t in teachers),
               "last_validation": getattr(student, "last_validation", None)}
    handle_termination(None, None)
    return summary


if __name__ == "__main__":
    main(default_config_path=os.path.join(os.path.dirname(os.path.abspath(sys.argv[0])), "config.json"))
