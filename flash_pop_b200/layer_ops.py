"""The elementwise passes of a retention layer either side of the operator, fused: the rotary rotation of q and k
(flash_pop/xpos_emb.py:32-40,120-126) and GroupNorm-per-head times the swish gate (flash_pop/retnet.py:294-309).
Each is one streaming CUDA kernel forward and one backward, over the C ABI (fpb_rotary, fpb_groupnorm_gate_*)."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
from torch import Tensor

from flash_pop_b200 import _lib

_OK_DTYPES = (torch.bfloat16, torch.float32)


def _aligned(t: Tensor, nbytes: int) -> Tensor:
    """`t` (B,T,H,d) with unit inner stride and pointer/strides that allow `nbytes`-wide accesses, copied if not."""
    vec = nbytes // t.element_size()
    ok = t.stride(-1) == 1 and t.data_ptr() % nbytes == 0 and all(s % vec == 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


def rotary_supported(q: Tensor) -> bool:
    return q.is_cuda and q.dim() == 4 and q.dtype in _OK_DTYPES and q.size(-1) % 8 == 0


def _rotate(q: Tensor, k: Optional[Tensor], phasors: Tensor, conjugate: bool, out_dtype: torch.dtype):
    B, T, H, d = q.shape
    rows = phasors.shape[0]
    assert phasors.dtype == torch.float32 and phasors.is_contiguous() and tuple(phasors.shape[1:]) == (T, d // 2, 2)
    assert rows in (1, B), "one phasor table for all rows, or one per batch row"
    q = _aligned(q, 16)
    k = None if k is None else _aligned(k.to(q.dtype), 16)
    q_out = torch.empty((B, T, H, d), device=q.device, dtype=out_dtype)
    k_out = None if k is None else torch.empty((B, T, H, d), device=q.device, dtype=out_dtype)
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib().fpb_rotary(B, T, H, d, _lib.dtype_code(q), _lib.dtype_code(q_out), int(conjugate),
                                         ctypes.c_void_p(phasors.data_ptr()), 0 if rows == 1 else T * (d // 2),
                                         _lib.seq(q), _lib.seq(k), _lib.seq(q_out), _lib.seq(k_out),
                                         _lib.stream_ptr(q.device)))
    return q_out, k_out


class RotaryQK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, phasors, out_dtype):
        ctx.save_for_backward(phasors)
        ctx.in_dtype = q.dtype
        return _rotate(q, k, phasors, False, out_dtype or q.dtype)

    @staticmethod
    def backward(ctx, dq, dk):
        (phasors,) = ctx.saved_tensors
        if dq is None and dk is None:
            return None, None, None, None
        ref = dq if dq is not None else dk
        dq = torch.zeros_like(ref) if dq is None else dq
        dk = torch.zeros_like(ref) if dk is None else dk
        gq, gk = _rotate(dq, dk, phasors, True, ctx.in_dtype)      # the rotation is orthogonal: backward = inverse
        return gq, gk, None, None


def rotary_qk(q: Tensor, k: Tensor, phasors: Tensor, out_dtype: Optional[torch.dtype] = None) -> Tuple[Tensor, Tensor]:
    """Rotate the channel pairs of q and k (B,T,H,d) by `phasors` (1 or B, T, d/2, 2) = (cos, sin), fp32."""
    return RotaryQK.apply(q, k, phasors, out_dtype)


def groupnorm_gate_supported(o: Tensor, z: Tensor) -> bool:
    return (o.is_cuda and o.dim() == 4 and o.dtype in _OK_DTYPES and z.dtype == o.dtype and o.size(-1) % 2 == 0
            and o.size(-1) <= 256 and o.shape == z.shape)


class GroupNormGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o, z, eps: float, swish: bool):
        nb = 4 if o.dtype == torch.bfloat16 else 8
        o, z = _aligned(o, nb), _aligned(z, nb)
        B, T, H, dv = o.shape
        y = torch.empty((B, T, H, dv), device=o.device, dtype=o.dtype)
        with torch.cuda.device(o.device):
            _lib.check(_lib.lib().fpb_groupnorm_gate_fwd(B, T, H, dv, _lib.dtype_code(o), float(eps), int(swish),
                                                         _lib.seq(o), _lib.seq(z), _lib.seq(y), _lib.stream_ptr(o.device)))
        ctx.save_for_backward(o, z)
        ctx.eps, ctx.swish = float(eps), bool(swish)
        return y

    @staticmethod
    def backward(ctx, dy):
        o, z = ctx.saved_tensors
        B, T, H, dv = o.shape
        dy = _aligned(dy.to(o.dtype), 4 if o.dtype == torch.bfloat16 else 8)
        d_o, d_z = torch.empty_like(o, memory_format=torch.contiguous_format), torch.empty_like(z, memory_format=torch.contiguous_format)
        with torch.cuda.device(o.device):
            _lib.check(_lib.lib().fpb_groupnorm_gate_bwd(B, T, H, dv, _lib.dtype_code(o), ctx.eps, int(ctx.swish),
                                                         _lib.seq(o), _lib.seq(z), _lib.seq(dy), _lib.seq(d_o),
                                                         _lib.seq(d_z), _lib.stream_ptr(o.device)))
        return d_o, d_z, None, None


def groupnorm_gate(o: Tensor, z: Tensor, eps: float, swish: bool = True) -> Tensor:
    """GroupNorm over the last dimension of o (B,T,H,dv) (no affine parameters) times the gate: z * sigmoid(z) when
    `swish`, else z as given."""
    return GroupNormGate.apply(o, z, eps, swish)
