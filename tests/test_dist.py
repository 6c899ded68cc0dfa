"""Multi-rank paths: gloo ranks on CPU (always), NCCL + NVLink P2P ranks when two or more GPUs are visible."""
import os
import socket
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(mode, nproc, timeout=600, env=None, extra=()):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "dist_worker.py"), mode, *extra]
    e = dict(os.environ, B200_NO_PROGRESS="1", OMP_NUM_THREADS="2", **(env or {}))
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e)
    assert r.returncode == 0 and "WORKER_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])


def test_cpu_ranks_ddp_and_fsdp_match_single_process():
    _launch("cpu_engine", 2)


@pytest.mark.parametrize("world", [2, 3])
def test_cpu_ranks_training_through_the_vocabulary_parallel_head_matches_replicated_heads(world):
    _launch("cpu_vp_training", world)


@pytest.mark.parametrize("world", [2, 3])
def test_cpu_ranks_full_parameter_sharding_matches_single_process(world):
    _launch("cpu_zero3", world)


def test_cpu_ranks_full_parameter_sharding_of_a_mixture_of_experts_student():
    """The expert half of a Mixtral-style layer is a second autograd node: the unit hooks of the full-shard engine (gather
    before a layer's backward, reduction after it) must still see the layer as one unit."""
    _launch("cpu_zero3", 2, env={"Z3_MOE": "1"})


@pytest.mark.parametrize("family", ["olmo2", "glm4"])
def test_cpu_ranks_full_sharding_with_layers_that_have_output_norms(family):
    """The general layer node (models/sandwich.py) calls the engines' per-layer hooks like the fused layer does."""
    _launch("cpu_zero3", 2, env={"Z3_FAMILY": family})


def test_cpu_ranks_pipeline_with_fully_sharded_student(tmp_path):
    _launch("cpu_cli_zero3", 2, extra=(str(tmp_path),))


def test_cpu_ranks_chunked_pipeline_replicated_and_fully_sharded(tmp_path):
    """Cache smaller than the data: collect / train / save state / load state per chunk, on two ranks."""
    _launch("cpu_cli_zero3_chunked", 2, extra=(str(tmp_path),))


def test_cpu_three_ranks_pipeline_with_a_rank_short_of_a_batch(tmp_path):
    _launch("cpu_cli_zero3_three", 3, extra=(str(tmp_path),))


def test_cpu_ranks_pipeline_with_accumulation_that_straddles_epochs(tmp_path):
    _launch("cpu_cli_zero3_accum", 2, extra=(str(tmp_path),))


@pytest.mark.parametrize("optimizer", ["adamw"])
def test_cpu_ranks_pipeline_variants_replicated_and_fully_sharded(tmp_path, optimizer):
    """Gradient checkpointing, shuffled order, the reference's weighted loss, a frozen layer."""
    _launch("cpu_cli_zero3_variants", 2, extra=(str(tmp_path),), env={"Z3_OPT": optimizer})


@pytest.mark.parametrize("strategy", ["ddp", "zero3"])
def test_cpu_ranks_lost_peer_in_the_command_line_run(tmp_path, strategy):
    """The survivor meets the loss as a failed collective, learns from the heartbeats that a peer is gone, writes its
    trainer state without any collective (under full sharding: its optimizer pieces with their master weights) and
    exits with status 3. Replicated case, peer lost in the middle of the second epoch: the same command again takes
    the state up, passes over the samples it already counts and completes the run (that a run taken up in the middle of
    an epoch ends with the weights of an undisturbed one is checked in tests/test_e2e_cpu.py)."""
    at = "3" if strategy == "ddp" else "2"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(HERE, "dist_worker.py"), "cpu_cli_rank_loss", str(tmp_path)]
    env = dict(os.environ, B200_NO_PROGRESS="1", OMP_NUM_THREADS="2", B200_HEARTBEAT_TIMEOUT="2", RL_STRATEGY=strategy,
               RL_AT=at)
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    log = r.stdout + r.stderr
    assert "RANK 1 LEAVES" in log and "finished the run although" not in log, log[-3000:]
    assert "[watchdog] rank(s) [1]" in log and "saving state and leaving" in log, log[-3000:]
    assert "exitcode  : 3" in log or "exitcode: 3" in log, log[-3000:]
    states_dir = os.path.join(str(tmp_path), "cache", "student", "states")
    states = os.listdir(states_dir)
    assert "trainer_state.json" in states
    assert ("optimizer_state.rank0.pt" if strategy == "zero3" else "optimizer_state.pt") in states, states
    assert ("model_state.pt" in states) == (strategy != "zero3")
    import json
    with open(os.path.join(states_dir, "trainer_state.json")) as f:
        counted = json.load(f)["num_trained_steps"]
    assert counted == 4 * int(at)            # four samples per step; the step that failed is not claimed
    if strategy != "ddp":
        return
    _launch("cpu_cli_rank_loss", 2, extra=(str(tmp_path),), env={"RL_LEAVE": "0", "RL_STRATEGY": strategy})


def test_cpu_ranks_stop_request_at_one_rank_stops_all_and_the_run_resumes(tmp_path):
    """SIGTERM reaches rank 1 during its third step of a fully sharded run: after the next step both ranks agree, save
    the state together (weights through the gathered view) and return; the rerun completes the run (that a resumed run
    equals an undisturbed one is checked in the single-process test and in the lost-peer test)."""
    env = {"RL_STRATEGY": "zero3", "RL_MODE": "stop", "RL_AT": "3"}
    _launch("cpu_cli_rank_loss", 2, extra=(str(tmp_path),), env=env)
    _launch("cpu_cli_rank_loss", 2, extra=(str(tmp_path),), env=dict(env, RL_LEAVE="0"))


def test_cpu_ranks_changed_dataset_is_synced_not_recollected(tmp_path):
    _launch("cpu_cli_sync", 2, extra=(str(tmp_path),))


def test_cpu_ranks_fully_sharded_run_resumes_where_it_stopped(tmp_path):
    _launch("cpu_cli_resume", 2, extra=(str(tmp_path),))


@pytest.mark.parametrize("tp", ["0", "2"])
def test_cpu_ranks_multi_teacher_cross_tokenizer_pipeline_fully_sharded(tmp_path, tp):
    """tp 0: the planner picks the width (1: two replicas); tp 2: both teachers run as one two-way group."""
    _launch("cpu_cli_config3", 2, extra=(str(tmp_path),), env={"C3_TP": tp})


@pytest.mark.gpu
def test_gpu_pipeline_with_replicated_and_fully_sharded_student(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    _launch("gpu_cli_zero3", 2, env={"NCCL_NVLS_ENABLE": "0"}, extra=(str(tmp_path),))


@pytest.mark.gpu
def test_full_parameter_sharding_matches_replicated_training():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    _launch("gpu_zero3", min(4, torch.cuda.device_count()), env={"NCCL_NVLS_ENABLE": "0"})


@pytest.mark.gpu
@pytest.mark.parametrize("overlap", ["0", "1"])
def test_p2p_collectives_and_training_match_nccl(overlap):
    """overlap = 1: the gradient reduction runs behind backward on a side stream (off by default)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    _launch("gpu_p2p", min(4, torch.cuda.device_count()), env={"NCCL_NVLS_ENABLE": "0", "B200_OVERLAP": overlap})


def test_cpu_ranks_tensor_parallel_teacher_matches_unsharded():
    _launch("cpu_tp", 2)


def test_cpu_ranks_tensor_parallel_teacher_with_per_head_qk_norms():
    _launch("cpu_tp", 2, env={"TP_QKNORM": "1"})


def test_cpu_ranks_tensor_parallel_teacher_with_partial_rotation_and_a_layer_without():
    _launch("cpu_tp", 2, env={"TP_VARIANT": "partial_nope"})


def test_cpu_ranks_vocabulary_parallel_head_matches_unsharded():
    _launch("cpu_vp_head", 2)


def test_cpu_ranks_pipeline_with_tensor_parallel_teacher(tmp_path):
    _launch("cpu_cli_tp", 2, extra=(str(tmp_path),))


@pytest.mark.gpu
def test_fused_tp_gemms_and_tp_teacher_match_references():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    _launch("gpu_tp", min(4, torch.cuda.device_count()), env={"NCCL_NVLS_ENABLE": "0"})


@pytest.mark.gpu
def test_fused_tp_gemms_on_cta_pairs_match_references():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    _launch("gpu_tp", min(4, torch.cuda.device_count()), env={"NCCL_NVLS_ENABLE": "0", "B200_TP_PAIR": "1"})
