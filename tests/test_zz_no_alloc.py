"""The allocation-free RMSNorm backward (csrc/ops/rmsnorm_noalloc.h) called through its exported C symbol.

Why it exists: some users of the shared library cannot allocate device memory at call time - another runtime owns
the whole device arena, cudaMalloc is banned inside their latency-critical loop because it synchronises the
device, or they are plain C programs with no tensor library. For them the weight-gradient workspace lives in a
fixed __device__ array inside the library. This test loads the .so with ctypes (no Python binding layer), calls the
symbol twice in a row with different inputs and checks both results against the regular entry point, which takes
its workspace from the caller. It is collected last so that a run stopping at the first failure has already run
every other test, and it does not depend on anything the other tests leave behind.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "llm_distillery_b200", "_C",
                   "libb200_kernels.so")
VP, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _lib():
    lib = ctypes.CDLL(LIB)
    lib.b200_rmsnorm_bwd_noalloc.argtypes = [VP, VP, VP, VP, VP, VP, VP, I, I, I, VP]
    lib.b200_rmsnorm_bwd_noalloc.restype = I
    lib.b200_rmsnorm_bwd.argtypes = [VP, VP, VP, VP, VP, VP, VP, VP, I, I, I, VP]
    lib.b200_rmsnorm_bwd.restype = I
    lib.b200_rmsnorm_bwd_blocks.argtypes = [I]
    lib.b200_rmsnorm_bwd_blocks.restype = I
    lib.b200_last_cuda_error.restype = ctypes.c_char_p
    return lib


def _p(t):
    return VP(0 if t is None else t.data_ptr())


def _case(rows, h, seed, with_res):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g)  # noqa: E731
    x, dy = mk(rows, h).bfloat16(), mk(rows, h).bfloat16()
    w = (1 + 0.1 * mk(h)).bfloat16()
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    dres = mk(rows, h).bfloat16() if with_res else None
    return dy, x, w, rstd, dres


def test_noalloc_matches_regular_entry_point_twice():
    lib = _lib()
    stream = VP(torch.cuda.current_stream().cuda_stream)
    for call, (rows, h, with_res, acc) in enumerate([(700, 2048, True, False), (300, 4096, False, True)]):
        dy, x, w, rstd, dres = _case(rows, h, 10 + call, with_res)
        dx_a, dx_b = torch.empty_like(x), torch.empty_like(x)
        dw_a = torch.full((h,), 0.5, device="cuda")
        dw_b = dw_a.clone()
        rc = lib.b200_rmsnorm_bwd_noalloc(_p(dy), _p(x), _p(w), _p(rstd), _p(dres), _p(dx_a), _p(dw_a), int(acc), rows, h,
                                          stream)
        assert rc == 0, lib.b200_last_cuda_error()
        partial = torch.empty((lib.b200_rmsnorm_bwd_blocks(rows), h), device="cuda")
        rc = lib.b200_rmsnorm_bwd(_p(dy), _p(x), _p(w), _p(rstd), _p(dres), _p(dx_b), _p(partial), _p(dw_b), int(acc), rows,
                                  h, stream)
        assert rc == 0, lib.b200_last_cuda_error()
        torch.cuda.synchronize()
        # same math per row (the regular entry point may use another kernel: sums in another order, bf16 rounding)
        assert torch.allclose(dx_a.float(), dx_b.float(), atol=2e-2, rtol=2e-2), (dx_a.float() - dx_b.float()).abs().max()
        assert torch.allclose(dw_a, dw_b, atol=5e-2 * rows ** 0.5, rtol=2e-2), (dw_a - dw_b).abs().max()
        # and both agree with the fp32 PyTorch restatement
        xh = x.float() * rstd[:, None]
        ref_dw = (dy.float() * xh).sum(0) + (0.5 if acc else 0.0)
        assert torch.allclose(dw_a, ref_dw, atol=5e-2 * rows ** 0.5, rtol=2e-2)


def test_noalloc_rejects_rows_wider_than_its_workspace():
    lib = _lib()
    dy, x, w, rstd, _ = _case(4, 8192, 3, False)
    dx, dw = torch.empty_like(x), torch.zeros(8192, device="cuda")
    rc = lib.b200_rmsnorm_bwd_noalloc(_p(dy), _p(x), _p(w), _p(rstd), None, _p(dx), _p(dw), 0, 4, 8192,
                                      VP(torch.cuda.current_stream().cuda_stream))
    assert rc == -4 and b"B200_RMSNORM_NOALLOC_MAX_H" in lib.b200_last_cuda_error()
