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
    ok = t2.stride(1) == 1 and t2.data_ptr() % 16 == 0 and (t2.size(0) <= 1 or (t2.stride(0) >= t2.size(1) and t2.stride(0) % vec == 0))
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


# ---- adaptive LayerNorm modulation and gated residual (diffusion RetNet) ---------------------------------------------------
def row_broadcast_supported(x: Tensor, *mods: Tensor) -> bool:
    """x: (B, T, D) activations; mods: (B, Tm, D) operands each shared by T / Tm consecutive tokens (views into the
    modulation MLP's output are fine)."""
    if not (x.is_cuda and x.dim() == 3 and layer_norm_supported(x, x.shape[-1])):
        return False
    B, T, D = x.shape
    for m in mods:
        if not (m.is_cuda and m.dim() == 3 and m.dtype == x.dtype and m.shape[0] == B and m.shape[2] == D and m.shape[1] > 0
                and T % m.shape[1] == 0 and m.shape[1] == mods[0].shape[1]):
            return False
    return True


def _mod_rows(m: Tensor):
    """A (B, Tm, D) modulation operand as the C ABI reads it: pointer to its first row and the row pitch.  A chunk of the
    MLP's (B, Tm, n D) output qualifies in place when its rows are evenly spaced; anything else is copied."""
    B, Tm, D = m.shape
    vec = 16 // m.element_size()
    even = m.stride(2) == 1 and (B == 1 or Tm == 1 or m.stride(0) == Tm * m.stride(1))
    pitch = m.stride(1) if Tm > 1 else (m.stride(0) if B > 1 else D)
    if not (even and m.data_ptr() % 16 == 0 and pitch % vec == 0 and pitch >= D):
        m = m.contiguous()
        pitch = D
    return m, pitch


class AdaLNModulate(torch.autograd.Function):
    """y = LayerNorm(x) * (1 + scale) + shift with (B, Tm, D) shift / scale broadcast over T / Tm tokens each: one
    kernel forward, one backward (which also sums the gradients of shift and scale over the tokens that share them)."""

    @staticmethod
    def forward(ctx, x, shift, scale, eps):
        B, T, D = x.shape
        Tm = shift.shape[1]
        x2 = _rows(x)
        shift_r, pitch_a = _mod_rows(shift)
        scale_r, pitch_b = _mod_rows(scale)
        if pitch_a != pitch_b:                                   # one pitch serves both operands
            shift_r, scale_r, pitch_a = shift_r.contiguous(), scale_r.contiguous(), D
        rows = x2.shape[0]
        y = torch.empty((rows, D), device=x.device, dtype=x.dtype)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().fpb_adaln_fwd(rows, D, _lib.dtype_code(x2), eps, _ptr(x2), x2.stride(0) if rows > 1 else D,
                                                _ptr(shift_r), _ptr(scale_r), pitch_a, T // Tm, _ptr(y), D,
                                                _lib.stream_ptr(x.device)))
        ctx.save_for_backward(x2, scale_r)
        ctx.eps, ctx.shape, ctx.pitch, ctx.Tm = eps, x.shape, pitch_a, Tm
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, scale_r = ctx.saved_tensors
        B, T, D = ctx.shape
        rows = x2.shape[0]
        dy2 = _rows(dy.to(x2.dtype))
        x_in = x2 if (rows <= 1 or x2.stride(0) == D) else x2.contiguous()     # d_x is written with x's row pitch
        dx = torch.empty((rows, D), device=x2.device, dtype=x2.dtype)
        d_shift = torch.empty((B * ctx.Tm, D), device=x2.device, dtype=torch.float32)
        d_scale = torch.empty_like(d_shift)
        with torch.cuda.device(x2.device):
            _lib.check(_lib.lib().fpb_adaln_bwd(rows, D, _lib.dtype_code(x2), ctx.eps, _ptr(x_in), D, _ptr(scale_r), ctx.pitch,
                                                T // ctx.Tm, _ptr(dy2), dy2.stride(0) if rows > 1 else D, _ptr(dx), _ptr(d_shift),
                                                _ptr(d_scale), _lib.stream_ptr(x2.device)))
        as_mod = lambda t: t.view(B, ctx.Tm, D).to(x2.dtype)
        return dx.view(ctx.shape), as_mod(d_shift), as_mod(d_scale), None


class GateResidual(torch.autograd.Function):
    """out = x + gate * branch with a (B, Tm, D) gate broadcast over T / Tm tokens each."""

    @staticmethod
    def forward(ctx, x, branch, gate):
        B, T, D = x.shape
        Tm = gate.shape[1]
        x2, b2 = _rows(x), _rows(branch.to(x.dtype))
        gate_r, pitch = _mod_rows(gate)
        rows = x2.shape[0]
        out = torch.empty((rows, D), device=x.device, dtype=x.dtype)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().fpb_gate_residual_fwd(rows, D, _lib.dtype_code(x2), _ptr(x2), x2.stride(0) if rows > 1 else D, _ptr(b2),
                                                        b2.stride(0) if rows > 1 else D, _ptr(gate_r), pitch, T // Tm, _ptr(out), D,
                                                        _lib.stream_ptr(x.device)))
        ctx.save_for_backward(b2, gate_r)
        ctx.shape, ctx.pitch, ctx.Tm = x.shape, pitch, Tm
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, d_out):
        b2, gate_r = ctx.saved_tensors
        B, T, D = ctx.shape
        rows = b2.shape[0]
        d2 = _rows(d_out.to(b2.dtype))
        b_in = b2 if (rows <= 1 or b2.stride(0) == D) else b2.contiguous()
        d_branch = torch.empty((rows, D), device=b2.device, dtype=b2.dtype)
        d_gate = torch.empty((B * ctx.Tm, D), device=b2.device, dtype=torch.float32)
        with torch.cuda.device(b2.device):
            _lib.check(_lib.lib().fpb_gate_residual_bwd(rows, D, _lib.dtype_code(b2), _ptr(b_in), D, _ptr(gate_r), ctx.pitch,
                                                        T // ctx.Tm, _ptr(d2), d2.stride(0) if rows > 1 else D, _ptr(d_branch),
                                                        _ptr(d_gate), _lib.stream_ptr(b2.device)))
        return d_out, d_branch.view(ctx.shape), d_gate.view(B, ctx.Tm, D).to(b2.dtype)


def adaln_modulate(x: Tensor, shift: Tensor, scale: Tensor, eps: float) -> Tensor:
    """``LayerNorm(x.float()).to(x.dtype) * (1 + scale) + shift`` for (B, T, D) x and (B, Tm, D) shift / scale (T % Tm == 0,
    each modulation row shared by T / Tm consecutive tokens).  One kernel each way where the shapes qualify."""
    if row_broadcast_supported(x, shift, scale):
        return AdaLNModulate.apply(x, shift, scale, eps)
    rep = x.shape[1] // shift.shape[1]
    xn = torch.nn.functional.layer_norm(x.float(), x.shape[-1:], None, None, eps).to(x.dtype)
    return xn * (1 + scale.repeat_interleave(rep, dim=1)) + shift.repeat_interleave(rep, dim=1)


def gate_residual(x: Tensor, branch: Tensor, gate: Tensor) -> Tensor:
    """``x + branch * gate`` for (B, T, D) x / branch and a (B, Tm, D) gate shared by T / Tm consecutive tokens."""
    if row_broadcast_supported(x, gate) and branch.shape == x.shape and branch.is_cuda:
        return GateResidual.apply(x, branch, gate)
    return x + branch * gate.repeat_interleave(x.shape[1] // gate.shape[1], dim=1)


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
    """Softmax cross entropy of (rows, V) logits against int64 targets, fp32 arithmetic, averaged over ALL rows: a row
    whose target lies outside [0, V) (PyTorch's ignore_index -100 among them) adds zero loss and gets a zero gradient
    but still counts in the denominator.  With every target in range this is ``F.cross_entropy(logits.float(), targets)``.
    Both paths below follow this one rule; which one runs depends only on the logits' alignment."""
    if cross_entropy_supported(logits, targets):
        return FusedCrossEntropy.apply(logits, targets)
    valid = (targets >= 0) & (targets < logits.size(-1))
    safe = torch.where(valid, targets, torch.zeros_like(targets))
    per_row = torch.nn.functional.cross_entropy(logits.float(), safe, reduction="none")
    return (per_row * valid.to(per_row.dtype)).sum() / max(logits.size(0), 1)
