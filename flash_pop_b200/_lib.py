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
# the same sources with -DFPB_DIAGNOSTICS: adds the fpb_debug_* hooks (schedule choices, wait limit, time stamps) that
# some tests use; the operators never load it on their own
DIAG_LIB_PATH = os.path.join(LIB_DIR, "libflash_pop_b200_diag.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-shared", "-Xcompiler", "-fPIC",
    "--threads", "0",
]

FPB_BF16, FPB_F32 = 0, 1
STATIC_SCRATCH_BYTES = 16 << 20      # FPB_STATIC_SCRATCH_BYTES of the header
PATH_NONE, PATH_SIMT, PATH_TCGEN05 = 0, 1, 2
FLAG_FORCE_SIMT, FLAG_SKIP_DQ, FLAG_SKIP_DKDV, FLAG_STATE_F32 = 1, 2, 4, 8


class _Seq(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("stride_b", ctypes.c_int64), ("stride_t", ctypes.c_int64),
                ("stride_h", ctypes.c_int64)]


class _State(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("stride_b", ctypes.c_int64), ("stride_h", ctypes.c_int64)]


class _Dims(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int32), ("B", ctypes.c_int32), ("T", ctypes.c_int32), ("H", ctypes.c_int32),
                ("dk", ctypes.c_int32), ("dv", ctypes.c_int32), ("block_size", ctypes.c_int32),
                ("flags", ctypes.c_int32), ("head_decays", ctypes.POINTER(ctypes.c_double)),
                ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_int64)]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC_DIR, "*.cu")))


def _stale(path: str = LIB_PATH) -> bool:
    if not os.path.exists(path):
        return True
    built = os.path.getmtime(path)
    deps = sources() + glob.glob(os.path.join(CSRC_DIR, "*.cuh")) + glob.glob(os.path.join(CSRC_DIR, "*.h")) + \
        glob.glob(os.path.join(PKG_DIR, "..", "include", "*.h"))
    return any(os.path.getmtime(p) > built for p in deps)


def build(force: bool = False, verbose: bool = False, diagnostics: bool = True) -> str:
    """Compile every CUDA source of the package for sm_100a into one shared library, in-tree; with `diagnostics`
    also the diagnostics build of the same sources.  Returns the path of the release library."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(LIB_DIR, exist_ok=True)
    jobs = [(LIB_PATH, [])] + ([(DIAG_LIB_PATH, ["-DFPB_DIAGNOSTICS"])] if diagnostics else [])
    procs = []
    for path, extra in jobs:
        if not force and not _stale(path):
            continue
        tmp = path + ".partial"                 # built beside the target and renamed: a reader never sees half a library
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-o", tmp, *sources()]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd))
        procs.append((path, tmp, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
    for path, tmp, proc in procs:
        out, err = proc.communicate()
        if proc.returncode != 0:
            if os.path.exists(tmp):
                os.remove(tmp)
            raise RuntimeError("nvcc failed:\n" + out + err)
        os.replace(tmp, path)
        if verbose:
            print(err)
    return LIB_PATH


_lib: Optional[ctypes.CDLL] = None

_SEQ_P, _STATE_P, _DIMS_P = ctypes.POINTER(_Seq), ctypes.POINTER(_State), ctypes.POINTER(_Dims)
_SIGNATURES = {
    "fpb_retention_fwd": [_DIMS_P, _SEQ_P, _SEQ_P, _SEQ_P, _STATE_P, _SEQ_P, _STATE_P, ctypes.c_void_p],
    "fpb_retention_fwd_static": [_DIMS_P, _SEQ_P, _SEQ_P, _SEQ_P, _STATE_P, _SEQ_P, _STATE_P, ctypes.c_void_p],
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
    "fpb_copy_rows_async": [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
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
    "fpb_adaln_fwd": [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_float, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                      ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p],
    "fpb_adaln_bwd": [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_float, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                      ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                      ctypes.c_void_p],
    "fpb_gate_residual_fwd": [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                              ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64,
                              ctypes.c_void_p],
    "fpb_gate_residual_bwd": [ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                              ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p,
                              ctypes.c_void_p],
    "fpb_device_status": [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)],
}
# hooks of the diagnostics build only
_DIAG_SIGNATURES = {
    "fpb_debug_trace": [ctypes.c_void_p],
    "fpb_debug_tile_pref": [ctypes.c_int],
    "fpb_debug_suffix_group": [ctypes.c_int, ctypes.c_int],
    "fpb_debug_pop_emit": [ctypes.c_int],
    "fpb_debug_fused_bwd": [ctypes.c_int],
    "fpb_debug_segments": [ctypes.c_int],
    "fpb_debug_col_split": [ctypes.c_int],
    "fpb_debug_deep": [ctypes.c_int],
    "fpb_debug_ablate": [ctypes.c_int],
    "fpb_debug_tuning": [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int],
}


def exported_symbols() -> list[str]:
    """Every entry point include/flash_pop_b200.h declares."""
    return list(_SIGNATURES) + ["fpb_strerror", "fpb_version", "fpb_last_path", "fpb_last_cuda_error",
                                "fpb_launch_count", "fpb_workspace_bytes"]


def _load(path: str) -> ctypes.CDLL:
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -c 'import flash_pop_b200; flash_pop_b200.build()'` "
            "(needs nvcc).  flash_pop_b200 has no other implementation to fall back to.")
    handle = ctypes.CDLL(path)
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(handle, name)
        fn.argtypes = argtypes
        fn.restype = ctypes.c_int
    handle.fpb_strerror.argtypes = [ctypes.c_int]
    handle.fpb_strerror.restype = ctypes.c_char_p
    handle.fpb_version.restype = ctypes.c_int
    handle.fpb_last_path.restype = ctypes.c_int
    handle.fpb_last_cuda_error.restype = ctypes.c_int
    handle.fpb_launch_count.restype = ctypes.c_int64
    handle.fpb_workspace_bytes.argtypes = [_DIMS_P]
    handle.fpb_workspace_bytes.restype = ctypes.c_int64
    return handle


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = _load(LIB_PATH)
    return _lib


_diag: Optional[ctypes.CDLL] = None


def diag_lib() -> ctypes.CDLL:
    """The diagnostics build (release sources + the fpb_debug_* hooks)."""
    global _diag
    if _diag is None:
        _diag = _load(DIAG_LIB_PATH)
        for name, argtypes in _DIAG_SIGNATURES.items():
            fn = getattr(_diag, name)
            fn.argtypes = argtypes
            fn.restype = None
    return _diag


class diagnostics_build:
    """Context manager: inside it every operator of the package runs on the diagnostics build, whose handle it
    yields (for the fpb_debug_* hooks).  Tests only."""

    def __enter__(self) -> ctypes.CDLL:
        global _lib
        self.saved = lib()
        _lib = diag_lib()
        return _lib

    def __exit__(self, *exc):
        global _lib
        _lib = self.saved
        return False


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
    """(B,T,H,d) tensor the C ABI accepts: unit inner stride and, over every dimension longer than 1, a positive
    stride that does not fold rows onto each other.  Views that already are (head-split slices of a packed
    projection, batch slices) pass through; anything else - a transposed layout, or an ``expand()``-ed tensor such
    as the gradient autograd hands over for ``o.sum(dim=1)`` - is copied."""
    if t.dim() == 0 or t.numel() == 0:
        return t.contiguous()
    ok = t.stride(-1) == 1 or t.size(-1) == 1
    if ok:
        # sort the outer dimensions by stride and require each to step over the whole extent of the next smaller one
        span = t.size(-1)
        for size, stride in sorted(((t.size(i), t.stride(i)) for i in range(t.dim() - 1) if t.size(i) > 1), key=lambda p: p[1]):
            if stride < span:
                ok = False
                break
            span = stride * size
    return t if ok else t.contiguous()


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
         batch: Optional[int] = None, workspace: bool = False):
    """The call's `fpb_dims`.  With `workspace`, scratch memory for T-segments is allocated through torch's caching
    allocator when the shape can use it (fpb_workspace_bytes) and kept alive with the returned object; the allocator
    hands the block to later work on the same stream only, which is the order the kernels run in."""
    B, T, H, dk = t_like.shape
    arr = (ctypes.c_double * max(H, 1))(*[float(g) for g in head_decays])
    d = _Dims(dtype_code(t_like), B if batch is None else batch, T, H, dk, dv, block_size, flags,
              ctypes.cast(arr, ctypes.POINTER(ctypes.c_double)), None, 0)
    d._keepalive = arr
    if workspace and t_like.is_cuda:
        need = lib().fpb_workspace_bytes(ctypes.byref(d))
        if need > 0:
            d._scratch = torch.empty(need, dtype=torch.uint8, device=t_like.device)
            d.workspace, d.workspace_bytes = d._scratch.data_ptr(), need
    return d


def state_flags(q: torch.Tensor, *states) -> int:
    """FLAG_STATE_F32 when the call's states are fp32 under bf16 activations; raises on any other mix."""
    kinds = {s.dtype for s in states if s is not None}
    if not kinds or kinds == {q.dtype}:
        return 0
    if kinds == {torch.float32} and q.dtype == torch.bfloat16:
        return FLAG_STATE_F32
    raise ValueError(f"states must share the activations' dtype ({q.dtype}) or all be float32; got {sorted(map(str, kinds))}")


def stream_ptr(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
