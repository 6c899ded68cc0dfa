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
    # the context is intact: run a tensor-core kernel and check it
    from llm_distillery_b200.ops import basic
    a = torch.randn((256, 128), device=dev).to(torch.bfloat16)
    b = torch.randn((256, 128), device=dev).to(torch.bfloat16)
    c = basic.gemm(a, b)
    assert torch.allclose(c.float(), a.float() @ b.float().t(), atol=0.5, rtol=2e-2)
    assert _lib.take_device_error() == 0
