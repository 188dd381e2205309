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
    t = _lib.unit_inner(t)      # also copies expanded / overlapping views, which the C ABI refuses
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


# ---- LayerNorm with fp32 arithmetic on bf16 rows ------------------------------------------------------------------
def layer_norm_supported(x: Tensor, d: int) -> bool:
    if not (x.is_cuda and x.dtype in _OK_DTYPES and x.dim() >= 1 and x.size(-1) == d):
        return False
    vec = 8 if x.dtype == torch.bfloat16 else 4
    return d % vec == 0 and d <= 128 * vec


def _rows(t: Tensor) -> Tensor:
    """(rows, d) view with unit inner stride and a 16-byte aligned row pitch, copied if that is not what `t` is."""
    t2 = t.reshape(-1, t.size(-1))
    vec = 16 // t2.element_size()
    ok = t2.stride(1) == 1 and t2.data_ptr() % 16 == 0 and (t2.size(0) <= 1 or t2.stride(0) % vec == 0)
    return t2 if ok else t2.contiguous()


def _ptr(t: Optional[Tensor]):
    return ctypes.c_void_p(None if t is None else t.data_ptr())


class FusedLayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps: float):
        x2 = _rows(x)
        rows, d = x2.shape
        w = None if weight is None else weight.detach().float().contiguous()
        b = None if bias is None else bias.detach().float().contiguous()
        y = torch.empty((rows, d), device=x.device, dtype=x.dtype)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().fpb_layernorm_fwd(rows, d, _lib.dtype_code(x2), float(eps), _ptr(x2), x2.stride(0) if rows > 1 else d,
                                                    _ptr(w), _ptr(b), _ptr(y), d, _lib.stream_ptr(x.device)))
        ctx.save_for_backward(x2, w)
        ctx.eps, ctx.shape = float(eps), x.shape
        ctx.w_dtype = None if weight is None else weight.dtype
        ctx.b_dtype = None if bias is None else bias.dtype
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        rows, d = x2.shape
        dy2 = _rows(dy.to(x2.dtype))
        dx = torch.empty((rows, d), device=x2.device, dtype=x2.dtype)
        need_w = ctx.w_dtype is not None and ctx.needs_input_grad[1]
        need_b = ctx.b_dtype is not None and ctx.needs_input_grad[2]
        dw = torch.empty(d, device=x2.device, dtype=torch.float32) if need_w else None
        db = torch.empty(d, device=x2.device, dtype=torch.float32) if need_b else None
        x_in = x2 if (rows <= 1 or x2.stride(0) == d) else x2.contiguous()      # d_x is written with x's row pitch
        with torch.cuda.device(x2.device):
            _lib.check(_lib.lib().fpb_layernorm_bwd(rows, d, _lib.dtype_code(x2), ctx.eps, _ptr(x_in), d, _ptr(w), _ptr(dy2),
                                                    dy2.stride(0) if rows > 1 else d, _ptr(dx), _ptr(dw), _ptr(db),
                                                    _lib.stream_ptr(x2.device)))
        return (dx.view(ctx.shape), None if dw is None else dw.to(ctx.w_dtype), None if db is None else db.to(ctx.b_dtype), None)


def layer_norm(x: Tensor, weight: Optional[Tensor], bias: Optional[Tensor], eps: float) -> Tensor:
    """LayerNorm over the last dimension, fp32 arithmetic, result in x's dtype; weight / bias may be None."""
    return FusedLayerNorm.apply(x, weight, bias, eps)


def norm_in_fp32(module: torch.nn.LayerNorm, x: Tensor) -> Tensor:
    """``module(x.float()).to(x.dtype)`` — as one kernel when the rows qualify, else literally that."""
    if len(module.normalized_shape) == 1 and layer_norm_supported(x, module.normalized_shape[0]):
        return layer_norm(x, module.weight, module.bias, module.eps)
    return module(x.float()).to(dtype=x.dtype)


# ---- softmax cross entropy for the language-model head --------------------------------------------------------------
def cross_entropy_supported(logits: Tensor, targets: Tensor) -> bool:
    vec = 16 // max(logits.element_size(), 1)
    return (logits.is_cuda and logits.dim() == 2 and logits.dtype in _OK_DTYPES and targets.dtype == torch.int64 and
            targets.shape == logits.shape[:1] and logits.stride(1) == 1 and logits.data_ptr() % 16 == 0 and
            (logits.size(0) <= 1 or logits.stride(0) % vec == 0))


class FusedCrossEntropy(torch.autograd.Function):
    """Mean softmax cross entropy of (rows, V) logits; fp32 arithmetic, one read of the logits forward, one read and
    one write backward, gradient in the logits' own dtype."""

    @staticmethod
    def forward(ctx, logits, targets):
        rows, V = logits.shape
        targets = targets.contiguous()
        loss = torch.empty(rows, device=logits.device, dtype=torch.float32)
        lse = torch.empty(rows, device=logits.device, dtype=torch.float32)
        with torch.cuda.device(logits.device):
            _lib.check(_lib.lib().fpb_cross_entropy_fwd(rows, V, _lib.dtype_code(logits), _ptr(logits), logits.stride(0) if rows > 1 else V,
                                                        _ptr(targets), _ptr(loss), _ptr(lse), _lib.stream_ptr(logits.device)))
        ctx.save_for_backward(logits, targets, lse)
        return loss.mean()

    @staticmethod
    def backward(ctx, g):
        logits, targets, lse = ctx.saved_tensors
        rows, V = logits.shape
        vec = 16 // logits.element_size()
        pitch = (V + vec - 1) // vec * vec                       # rows of the gradient start on 16-byte boundaries too
        d_logits = torch.empty((rows, pitch), device=logits.device, dtype=logits.dtype)[:, :V]
        scale = g.detach().to(torch.float32).reshape(1).contiguous()
        with torch.cuda.device(logits.device):
            _lib.check(_lib.lib().fpb_cross_entropy_bwd(rows, V, _lib.dtype_code(logits), _ptr(logits), logits.stride(0) if rows > 1 else V,
                                                        _ptr(targets), _ptr(lse), _ptr(scale), 1.0 / max(rows, 1), _ptr(d_logits), pitch,
                                                        _lib.stream_ptr(logits.device)))
        return d_logits, None


def cross_entropy(logits: Tensor, targets: Tensor) -> Tensor:
    """Mean cross entropy of (rows, V) logits against int64 targets, as ``F.cross_entropy(logits.float(), targets)``."""
    if cross_entropy_supported(logits, targets):
        return FusedCrossEntropy.apply(logits, targets)
    return torch.nn.functional.cross_entropy(logits.float(), targets)
