"""A device-side wait that nothing satisfies runs out of its time budget, reports through the error word and returns;
the context stays usable. (The wait is on a flag word that no one writes: nothing faults, traps or spins forever.)"""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_flag_wait_times_out_with_a_status_and_the_gpu_keeps_working():
    from llm_distillery_b200.ops import _lib
    from llm_distillery_b200.parallel import p2p  # noqa: F401  (registers the barrier entry point)
    dev = torch.device("cuda", 0)
    assert _lib.take_device_error() == 0
    # a two-rank barrier whose second rank does not exist: both flag arrays live on this GPU, nobody plays rank 1
    flags0 = torch.zeros(64, dtype=torch.int32, device=dev)
    flags1 = torch.zeros(64, dtype=torch.int32, device=dev)
    ptrs = (ctypes.c_void_p * 2)(flags0.data_ptr(), flags1.data_ptr())
    t0 = time.time()
    _lib.check(_lib.kernels().b200_p2p_barrier(ptrs, 0, 2, 1, _lib.stream()), "b200_p2p_barrier")
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 1.0 < waited < 10.0, waited                  # the 2 s budget, not forever
    assert _lib.take_device_error() == 5                # ERR_WAIT_PEER
    assert _lib.take_device_error() == 0                # reading clears it
    assert flags1[0].item() == 1                        # rank 0's own announcement was made
    # the failed barrier left this GPU's peer collectives switched off until the host acknowledges the error
    _lib.check(_lib.kernels().b200_p2p_clear_poison(_lib.stream()), "b200_p2p_clear_poison")
    # the context is intact: run a tensor-core kernel and check it
    from llm_distillery_b200.ops import basic
    a = torch.randn((256, 128), device=dev).to(torch.bfloat16)
    b = torch.randn((256, 128), device=dev).to(torch.bfloat16)
    c = basic.gemm(a, b)
    assert torch.allclose(c.float(), a.float() @ b.float().t(), atol=0.5, rtol=2e-2)
    assert _lib.take_device_error() == 0


def test_kernels_queued_behind_a_failed_barrier_change_nothing():
    """The reduce + AdamW + all-gather kernel, the wire copy and the step counter launched after a barrier that ran
    out must leave weights, master weights, moments and the counter as they were; after the host has cleared the
    condition the same launches do their work (checked against AdamW in PyTorch)."""
    from llm_distillery_b200.ops import _lib
    from llm_distillery_b200.parallel import p2p  # noqa: F401
    dev = torch.device("cuda", 0)
    lib = _lib.kernels()
    assert _lib.take_device_error() == 0
    n, world, rank = 8192, 2, 0
    torch.manual_seed(3)
    grads = [torch.randn(n, device=dev) for _ in range(world)]          # rank 1's memory is played by this GPU too
    wires = [torch.zeros(n, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    wires[1].copy_(grads[1])                                            # what rank 1 would have published
    models = [torch.randn(n, device=dev).bfloat16() for _ in range(world)]
    shard_lo, shard_n = 0, n // 2
    master = models[0][:shard_n].float().clone()
    m, v = torch.zeros(shard_n, device=dev), torch.zeros(shard_n, device=dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    before = [t.clone() for t in (master, m, v, models[0], models[1], wires[0])]
    arr = lambda ts: (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])  # noqa: E731
    lr, b1, b2, eps, wd, gs = 1e-2, 0.9, 0.99, 1e-8, 0.0, 0.5

    def launches():
        _lib.check(lib.b200_p2p_cast_wire(_lib.ptr(grads[0]), _lib.ptr(wires[0]), shard_n, n - shard_n, _lib.stream()), "cast")
        _lib.check(lib.b200_p2p_rs_adamw_ag(arr(wires), _lib.ptr(grads[0]), 1, arr(models), _lib.ptr(master), _lib.ptr(m),
                                            _lib.ptr(v), shard_lo, shard_n, 0, rank, world, lr, b1, b2, eps, wd, 1, gs, 1,
                                            0, _lib.stream()), "rs_adamw_ag")
        _lib.check(lib.b200_p2p_mark_step(_lib.ptr(counter), _lib.stream()), "mark")

    flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(world)]
    _lib.check(lib.b200_p2p_barrier(arr(flags), rank, world, 1, _lib.stream()), "b200_p2p_barrier")   # nobody answers
    launches()
    torch.cuda.synchronize()
    assert _lib.take_device_error() == 5
    for t, ref in zip((master, m, v, models[0], models[1], wires[0]), before):
        assert torch.equal(t, ref)
    assert counter.item() == 0
    _lib.check(lib.b200_p2p_clear_poison(_lib.stream()), "b200_p2p_clear_poison")
    launches()
    torch.cuda.synchronize()
    assert counter.item() == 1
    assert torch.equal(wires[0][shard_n:], grads[0][shard_n:].bfloat16())
    g = (grads[0][:shard_n] + wires[1][:shard_n].float()) * gs
    m_ref = (1 - b1) * g
    v_ref = (1 - b2) * g * g
    p_ref = before[0] - (lr / (1 - b1)) * m_ref / ((v_ref / (1 - b2)).sqrt() + eps)
    assert torch.allclose(master, p_ref, atol=1e-5, rtol=1e-5)
    assert torch.allclose(m, m_ref, atol=1e-6) and torch.allclose(v, v_ref, atol=1e-6)
    for mod in models:
        assert torch.equal(mod[:shard_n], master.bfloat16()) and torch.equal(mod[shard_n:], before[3 if mod is models[0] else 4][shard_n:])
    assert _lib.take_device_error() == 0
