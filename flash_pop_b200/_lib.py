"""Loader and ctypes bindings for ``libflash_pop_b200.so`` (the C ABI in include/flash_pop_b200.h).

The shared library is the only implementation of the operators in this package: if it is missing
or the device is not a B200, every operator call raises.  There is no CPU or PyTorch path.
"""
from __future__ import annotations

import ctypes
import glob
import os
import shutil
import subprocess
from typing import Optional, Sequence

import torch

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC_DIR = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libflash_pop_b200.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-shared", "-Xcompiler", "-fPIC",
    "--threads", "0",
]

FPB_BF16, FPB_F32 = 0, 1
PATH_NONE, PATH_SIMT, PATH_TCGEN05 = 0, 1, 2
FLAG_FORCE_SIMT, FLAG_SKIP_DQ, FLAG_SKIP_DKDV = 1, 2, 4


class _Seq(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("stride_b", ctypes.c_int64), ("stride_t", ctypes.c_int64),
                ("stride_h", ctypes.c_int64)]


class _State(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("stride_b", ctypes.c_int64), ("stride_h", ctypes.c_int64)]


class _Dims(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int32), ("B", ctypes.c_int32), ("T", ctypes.c_int32), ("H", ctypes.c_int32),
                ("dk", ctypes.c_int32), ("dv", ctypes.c_int32), ("block_size", ctypes.c_int32),
                ("flags", ctypes.c_int32), ("head_decays", ctypes.POINTER(ctypes.c_double))]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC_DIR, "*.cu")))


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = sources() + glob.glob(os.path.join(CSRC_DIR, "*.cuh")) + glob.glob(os.path.join(CSRC_DIR, "*.h")) + \
        glob.glob(os.path.join(PKG_DIR, "..", "include", "*.h"))
    return any(os.path.getmtime(p) > built for p in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source of the package for sm_100a into one shared library, in-tree."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [nvcc, *NVCC_FLAGS, "-o", LIB_PATH, *sources()]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


_lib: Optional[ctypes.CDLL] = None

_SEQ_P, _STATE_P, _DIMS_P = ctypes.POINTER(_Seq), ctypes.POINTER(_State), ctypes.POINTER(_Dims)
_SIGNATURES = {
    "fpb_retention_fwd": [_DIMS_P, _SEQ_P, _SEQ_P, _SEQ_P, _STATE_P, _SEQ_P, _STATE_P, ctypes.c_void_p],
    "fpb_retention_bwd": [_DIMS_P, _SEQ_P, _SEQ_P, _SEQ_P, _STATE_P, _SEQ_P, _STATE_P, _SEQ_P, _SEQ_P, _SEQ_P,
                          _STATE_P, ctypes.c_void_p],
    "fpb_pop_retention_fwd": [_DIMS_P, _SEQ_P, _SEQ_P, _SEQ_P, _STATE_P, _SEQ_P, ctypes.c_void_p, ctypes.c_void_p],
    "fpb_pop_retention_bwd": [_DIMS_P, _SEQ_P, _SEQ_P, _SEQ_P, _STATE_P, _SEQ_P, ctypes.c_void_p, _SEQ_P, _SEQ_P,
                              _SEQ_P, _STATE_P, ctypes.c_void_p],
    "fpb_pop_suffix_fwd": [_DIMS_P, ctypes.c_int32, ctypes.c_int32, _SEQ_P, _SEQ_P, _SEQ_P, _STATE_P,
                           ctypes.c_void_p, _SEQ_P, ctypes.c_void_p],
    "fpb_pop_suffix_bwd": [_DIMS_P, ctypes.c_int32, ctypes.c_int32, _SEQ_P, _SEQ_P, _SEQ_P, _STATE_P,
                           ctypes.c_void_p, _SEQ_P, _SEQ_P, _SEQ_P, _SEQ_P, _STATE_P, ctypes.c_void_p,
                           ctypes.c_void_p],
    "fpb_retention_step": [_DIMS_P, ctypes.c_int32, _SEQ_P, _SEQ_P, _SEQ_P, _STATE_P, _SEQ_P, _STATE_P, ctypes.c_void_p],
    "fpb_rotary": [ctypes.c_int32] * 7 + [ctypes.c_void_p, ctypes.c_int64, _SEQ_P, _SEQ_P, _SEQ_P, _SEQ_P, ctypes.c_void_p],
    "fpb_groupnorm_gate_fwd": [ctypes.c_int32] * 5 + [ctypes.c_float, ctypes.c_int32, _SEQ_P, _SEQ_P, _SEQ_P, ctypes.c_void_p],
    "fpb_groupnorm_gate_bwd": [ctypes.c_int32] * 5 + [ctypes.c_float, ctypes.c_int32, _SEQ_P, _SEQ_P, _SEQ_P, _SEQ_P, _SEQ_P,
                               ctypes.c_void_p],
    "fpb_layernorm_fwd": [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_float, ctypes.c_void_p, ctypes.c_int64,
                          ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p],
    "fpb_layernorm_bwd": [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_float, ctypes.c_void_p, ctypes.c_int64,
                          ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                          ctypes.c_void_p],
    "fpb_cross_entropy_fwd": [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                              ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p],
    "fpb_cross_entropy_bwd": [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                              ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p],
    "fpb_device_status": [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)],
}


def exported_symbols() -> list[str]:
    """Every entry point include/flash_pop_b200.h declares."""
    return list(_SIGNATURES) + ["fpb_strerror", "fpb_version", "fpb_last_path", "fpb_last_cuda_error",
                                "fpb_launch_count"]


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -c 'import flash_pop_b200; flash_pop_b200.build()'` "
                "(needs nvcc).  flash_pop_b200 has no other implementation to fall back to.")
        _lib = ctypes.CDLL(LIB_PATH)
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.argtypes = argtypes
            fn.restype = ctypes.c_int
        _lib.fpb_strerror.argtypes = [ctypes.c_int]
        _lib.fpb_strerror.restype = ctypes.c_char_p
        _lib.fpb_version.restype = ctypes.c_int
        _lib.fpb_last_path.restype = ctypes.c_int
        _lib.fpb_last_cuda_error.restype = ctypes.c_int
        _lib.fpb_launch_count.restype = ctypes.c_int64
    return _lib


def check(status: int) -> None:
    if status == 0:
        return
    msg = lib().fpb_strerror(status).decode()
    if status == 8:
        msg += f" [cudaError {lib().fpb_last_cuda_error()}]"
    if status in (1, 2, 3, 4, 5, 6, 11):
        raise ValueError(f"flash_pop_b200: {msg}")
    raise RuntimeError(f"flash_pop_b200: {msg}")


def last_path() -> int:
    return lib().fpb_last_path()


def launch_count() -> int:
    return lib().fpb_launch_count()


def device_status(device=None) -> int:
    """Synchronise the current stream of `device` and raise if a kernel reported a timed-out wait."""
    stream = torch.cuda.current_stream(device).cuda_stream
    detail = ctypes.c_int32(0)
    status = lib().fpb_device_status(ctypes.c_void_p(stream), ctypes.byref(detail))
    if status != 0:
        raise RuntimeError(f"flash_pop_b200: {lib().fpb_strerror(status).decode()} (status word {detail.value:#x})")
    return 0


# ---- tensor marshalling ---------------------------------------------------------------------------
_DTYPES = {torch.bfloat16: FPB_BF16, torch.float32: FPB_F32}


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("flash_pop_b200 operators run on CUDA (B200) tensors only; there is no CPU path")


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise ValueError(f"flash_pop_b200: unsupported dtype {t.dtype} (bfloat16 and float32 only)") from None


def unit_inner(t: torch.Tensor) -> torch.Tensor:
    """(B,T,H,d) view with unit inner stride; copies only if the inner stride is not 1."""
    return t if t.stride(-1) == 1 or t.size(-1) == 1 and t.is_contiguous() else t.contiguous()


def seq(t: Optional[torch.Tensor]) -> _Seq:
    if t is None:
        return _Seq(None, 0, 0, 0)
    assert t.dim() == 4
    return _Seq(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def state(t: Optional[torch.Tensor]) -> _State:
    if t is None:
        return _State(None, 0, 0)
    assert t.dim() == 4 and t[0, 0].is_contiguous()
    return _State(t.data_ptr(), t.stride(0), t.stride(1))


def state_tensor(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    """(B,H,dk,dv) with a contiguous inner (dk,dv) block."""
    if t is None:
        return None
    return t if t.numel() == 0 or t[0, 0].is_contiguous() else t.contiguous()


def dims(t_like: torch.Tensor, dv: int, head_decays: Sequence[float], block_size: int = 0, flags: int = 0,
         batch: Optional[int] = None):
    B, T, H, dk = t_like.shape
    arr = (ctypes.c_double * max(H, 1))(*[float(g) for g in head_decays])
    d = _Dims(dtype_code(t_like), B if batch is None else batch, T, H, dk, dv, block_size, flags,
              ctypes.cast(arr, ctypes.POINTER(ctypes.c_double)))
    d._keepalive = arr
    return d


def stream_ptr(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
