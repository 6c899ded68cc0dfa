"""ctypes loader for the in-tree native libraries.

``kernels()`` returns ``_C/libb200_kernels.so`` (sm_100a CUDA kernels, C ABI, raw pointers + stream);
``host()`` returns ``_C/libb200_host.so`` (C++ HDF5 store and other host-side runtime).
Loading fails loudly: on a GPU box a missing library is an error, never a silent PyTorch fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_void_p, c_int, c_longlong, c_float, c_char_p, c_uint, POINTER
from pathlib import Path

import torch

_C_DIR = Path(__file__).resolve().parent.parent / "_C"
_KERNELS = None
_HOST = None


class NativeError(RuntimeError):
    pass


def _load(name: str) -> ctypes.CDLL:
    path = _C_DIR / name
    if not path.exists():
        if os.environ.get("B200_AUTO_BUILD", "1") == "1":
            from .. import build as _build
            _build.build()
        if not path.exists():
            raise NativeError(f"{path} is missing: run `python -m llm_distillery_b200.build`")
    return ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)


_VP, _I, _LL, _F = c_void_p, c_int, c_longlong, c_float

_SIGS = {
    # name: argtypes
    "b200_gemm": [_VP, _VP, _VP, _I, _I, _I, _LL, _LL, _LL, _I, _I, _I, _I, _I, _F, _VP, _LL, _VP, _VP],
    "b200_rmsnorm_fwd": [_VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _F, _VP],
    "b200_rmsnorm_bwd": [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _VP],
    "b200_rmsnorm_bwd_blocks": [_I],
    "b200_rope": [_VP, _VP, _VP, _VP, _LL, _I, _I, _LL, _I, _VP],
    "b200_rope_partial": [_VP, _VP, _VP, _VP, _LL, _I, _I, _I, _LL, _I, _VP],
    "b200_swiglu_fwd": [_VP, _VP, _LL, _I, _VP],
    "b200_swiglu_bwd": [_VP, _VP, _VP, _LL, _I, _VP],
    "b200_embed_fwd": [_VP, _VP, _VP, _LL, _I, _I, _VP],
    "b200_embed_bwd": [_VP, _VP, _VP, _LL, _I, _I, _VP],
    "b200_scatter_rows": [_VP, _VP, _VP, _LL, _I, _LL, _VP],
    "b200_cast_f32_to_bf16": [_VP, _VP, _LL, _F, _VP],
    "b200_cast_bf16_to_f32": [_VP, _VP, _LL, _F, _I, _VP],
    "b200_adam_step": [_VP, _VP, _VP, _VP, _VP, _LL, _F, _F, _F, _F, _F, _I, _F, _I, _VP],
    "b200_adam8_step": [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _LL, _F, _F, _F, _F, _F, _I, _F, _I, _VP],
    "b200_simple_opt_step": [_VP, _VP, _VP, _VP, _VP, _LL, _I, _F, _F, _F, _F, _F, _I, _I, _F, _VP],
    "b200_sumsq": [_VP, _LL, _F, _VP, _VP],
    "b200_sm_count": [],
    "b200_segment_reduce": [_VP, _VP, _VP, _LL, _I, _I, _VP],
    "b200_gemm_reset_split_sync": [_VP],
    "b200_gemm_swiglu": [_VP, _VP, _VP, _VP, _I, _I, _I, _LL, _LL, _LL, _LL, _VP],
    "b200_gemm_rope": [_VP, _VP, _VP, _VP, _VP, _VP, _I, _I, _I, _I, _I, _LL, _LL, _LL, _VP],
    "b200_gemm_swiglu_bwd": [_VP, _VP, _VP, _VP, _I, _I, _I, _LL, _LL, _LL, _LL, _VP],
    "b200_headnorm_fwd": [_VP, _VP, _VP, _VP, _VP, _LL, _I, _I, _I, _LL, _F, _VP],
    "b200_headnorm_bwd_blocks": [_LL, _I, _I],
    "b200_headnorm_bwd": [_VP, _VP, _VP, _VP, _VP, _VP, _VP, _I, _LL, _I, _I, _I, _LL, _VP],
}


# device kernels launched by one call of each exported launcher (default 1); used to count launches
KERNELS_PER_CALL = {"b200_rmsnorm_bwd": 2, "b200_flash_attn_bwd": 3, "b200_flash_attn_bwd_rope": 3, "b200_head_num_tiles": 0, "b200_sm_count": 0,
                    "b200_rmsnorm_bwd_blocks": 0, "b200_last_cuda_error": 0, "b200_take_device_error": 0,
                    "b200_gemm_reset_split_sync": 0, "b200_headnorm_bwd_blocks": 0, "b200_headnorm_bwd": 2}
LAUNCH_COUNT = [0]


class _CountingLib:
    """Attribute proxy over the CDLL that counts kernel launches (``LAUNCH_COUNT[0]``)."""

    def __init__(self, lib):
        object.__setattr__(self, "_lib", lib)
        object.__setattr__(self, "_cache", {})

    def __getattr__(self, name):
        cache = object.__getattribute__(self, "_cache")
        fn = cache.get(name)
        if fn is None:
            raw = getattr(object.__getattribute__(self, "_lib"), name)
            n = KERNELS_PER_CALL.get(name, 1)
            if n == 0:
                fn = raw
            else:
                def fn(*a, _raw=raw, _n=n):
                    LAUNCH_COUNT[0] += _n
                    return _raw(*a)
            cache[name] = fn
        return fn


def kernels():
    global _KERNELS
    if _KERNELS is None:
        lib = _load("libb200_kernels.so")
        lib.b200_last_cuda_error.restype = c_char_p
        lib.b200_last_cuda_error.argtypes = []
        lib.b200_take_device_error.restype = c_uint
        lib.b200_take_device_error.argtypes = []
        for name, args in _SIGS.items():
            try:
                fn = getattr(lib, name)
            except AttributeError:
                continue
            fn.argtypes = args
            fn.restype = c_int
        _KERNELS = _CountingLib(lib)
    return _KERNELS


def register(name: str, argtypes: list) -> None:
    """Declare the signature of one more exported launcher (used by ops modules that own their kernels)."""
    _SIGS[name] = argtypes
    if _KERNELS is not None:
        try:
            fn = getattr(object.__getattribute__(_KERNELS, "_lib"), name)
        except AttributeError:  # declared by Python but not built into the library yet: calling it will raise
            return
        fn.argtypes = argtypes
        fn.restype = c_int


def host() -> ctypes.CDLL:
    global _HOST
    if _HOST is None:
        # B200_HOST_LIB: another build of the same library, e.g. the AddressSanitizer one of `build --sanitize`
        override = os.environ.get("B200_HOST_LIB")
        _HOST = ctypes.CDLL(override, mode=ctypes.RTLD_GLOBAL) if override else _load("libb200_host.so")
    return _HOST


def available() -> bool:
    """True when the CUDA kernels can run here (a GPU is visible and the library loads)."""
    if not torch.cuda.is_available():
        return False
    kernels()
    return True


_RC = {-1: "bad argument (shape / alignment / null pointer)", -2: "CUDA runtime error", -3: "tensor-map encode failed",
       -4: "size exceeds compiled maximum"}


def check(rc: int, what: str) -> None:
    if rc != 0:
        detail = kernels().b200_last_cuda_error().decode() if rc in (-2, -3) else ""
        raise NativeError(f"{what} failed: {_RC.get(rc, rc)} {detail}")


def _after_error(err: int) -> int:
    """A kernel that gave up on a wait may have left the split-K turn counters of the GEMM library non-zero."""
    if err:
        kernels().b200_gemm_reset_split_sync(stream())
    return err


def take_device_error() -> int:
    """Synchronise and return (then clear) the in-kernel wait error word of the current device (0 = none)."""
    torch.cuda.synchronize()
    return _after_error(int(kernels().b200_take_device_error()))


def peek_device_error() -> int:
    """The error word as it stands (pinned host memory), read and cleared WITHOUT synchronising the device."""
    return _after_error(int(kernels().b200_take_device_error()))


def stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())
