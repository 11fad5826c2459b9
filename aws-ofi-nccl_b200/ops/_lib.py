"""Loader for libb200ops.so (the sm_100a kernel library) and its C signatures.

The library is loaded with ctypes from ``aws-ofi-nccl_b200/lib``.  If it is missing the import
fails loudly — there is no PyTorch fallback path for the ops it provides.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent.parent / "lib"
_lib = None

_vp, _i, _ll, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_float

_SIGNATURES = {
    "b200_gemm_bf16": ([_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _i, _i, _i, _vp], _i),
    "b200_read_status": ([_i], _i),
    "b200_rmsnorm_fwd": ([_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp], _i),
    "b200_rmsnorm_bwd_partial_rows": ([], _i),
    "b200_rmsnorm_bwd": ([_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp], _i),
    "b200_gemm_fp8": ([_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _vp], _i),
    "b200_quant_rows_fp8": ([_vp, _vp, _vp, _i, _i, _ll, _ll, _vp], _i),
    "b200_swiglu_fwd": ([_vp, _vp, _ll, _i, _vp], _i),
    "b200_swiglu_bwd": ([_vp, _vp, _vp, _ll, _i, _vp], _i),
    "b200_swiglu_bwd_interleaved": ([_vp, _vp, _vp, _ll, _i, _vp], _i),
    "b200_rope": ([_vp, _vp, _vp, _ll, _i, _i, _ll, _i, _i, _vp], _i),
    "b200_cross_entropy": ([_vp, _vp, _vp, _i, _i, _ll, _f, _vp], _i),
    "b200_embedding_fwd": ([_vp, _vp, _vp, _ll, _i, _vp], _i),
    "b200_embedding_bwd": ([_vp, _vp, _vp, _ll, _i, _vp], _i),
    "b200_adamw": ([_vp, _vp, _vp, _vp, _vp, _ll, _f, _f, _f, _f, _f, _i, _f, _i, _vp], _i),
    "b200_sumsq": ([_vp, _ll, _vp, _vp], _i),
}


def lib_path() -> Path:
    return _LIB_DIR / "libb200ops.so"


def register(name: str, argtypes, restype=_i) -> None:
    """Let other modules declare the signature of an entry point they use."""
    _SIGNATURES[name] = (argtypes, restype)
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.argtypes, fn.restype = argtypes, restype


# kernels launched per library call (default 1); used for the launch counter
_KERNELS_PER_CALL = {"b200_rmsnorm_bwd": 2, "b200_read_status": 0, "b200_rmsnorm_bwd_partial_rows": 0}
launch_count = 0


class _CountingLib:
    """Proxy of the CDLL that counts the kernels this library launches."""

    def __init__(self, cdll):
        object.__setattr__(self, "_cdll", cdll)
        object.__setattr__(self, "_cache", {})

    def __getattr__(self, name):
        cache = object.__getattribute__(self, "_cache")
        w = cache.get(name)
        if w is None:
            fn = getattr(object.__getattribute__(self, "_cdll"), name)
            k = _KERNELS_PER_CALL.get(name, 1)

            def w(*args, _fn=fn, _k=k):
                global launch_count
                launch_count += _k
                return _fn(*args)

            cache[name] = w
        return w


_proxy = None


def load():
    global _proxy
    if _proxy is None:
        _proxy = _CountingLib(_load_cdll())
    return _proxy


def set_kernels_per_call(name: str, k: int) -> None:
    _KERNELS_PER_CALL[name] = k


def _load_cdll() -> C.CDLL:
    global _lib
    if _lib is None:
        p = lib_path()
        if not p.exists():
            raise RuntimeError(
                f"{p} is missing: run `python -m aws_ofi_nccl_b200.build` (needs nvcc); "
                "the CUDA ops have no fallback implementation")
        _lib = C.CDLL(os.fspath(p), mode=C.RTLD_GLOBAL)
        for name, (argtypes, restype) in _SIGNATURES.items():
            if hasattr(_lib, name):
                fn = getattr(_lib, name)
                fn.argtypes, fn.restype = argtypes, restype
    return _lib


class B200OpsError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise B200OpsError(f"{what} failed with code {rc}")


def stream_ptr() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


def read_status(clear: bool = True) -> int:
    """Device status word: 0, or the code of the first bounded wait that gave up (synchronises)."""
    return load().b200_read_status(1 if clear else 0)
