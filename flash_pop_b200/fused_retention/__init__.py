"""Fused chunked retention as a ``torch.autograd.Function`` over the C ABI.

Same call as the reference operator (flash_pop/fused_retention/__init__.py:10-67):

    o, s_out = fused_chunk_retention(q, k, v, s, head_decays)

q, k: (B, T, H, dk); v: (B, T, H, dv); s: (B, H, dk, dv) or None; head_decays: H Python floats.
Returns o (B, T, H, dv) and the state after the last token.  K is scaled by 1/sqrt(dk) inside the
operator.  Gradients flow to q, k, v and s; ``head_decays`` is not differentiable.

One addition to the reference's call: under bf16 activations the state may be float32 - pass an fp32 ``s``, or
``state_dtype=torch.float32`` as a sixth argument when there is no ``s`` yet - and ``s_out`` then is fp32 too.  A long
sequence fed in pieces (flash_pop/retnet.py:548-558) so carries its state from call to call without a bf16 rounding
at every hand-off.
"""
from __future__ import annotations

import contextlib
from typing import Optional, Sequence

import torch

from flash_pop_b200 import _lib

_force_simt = False


@contextlib.contextmanager
def cuda_core_kernels():
    """Within this context the operators take the fp32-arithmetic CUDA-core kernels even for shapes the
    tensor-core kernels handle (this is what ``use_fused_version=False`` selects in the layers)."""
    global _force_simt
    old, _force_simt = _force_simt, True
    try:
        yield
    finally:
        _force_simt = old


def _flags() -> int:
    return _lib.FLAG_FORCE_SIMT if _force_simt else 0


def _prepare(q, k, v, s, head_decays):
    _lib.require_cuda(q, k, v, s)
    if q.dim() != 4 or k.shape != q.shape or v.dim() != 4 or v.shape[:3] != q.shape[:3]:
        raise ValueError(f"expected q,k (B,T,H,dk) and v (B,T,H,dv); got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    assert len(head_decays) == H, f"got {len(head_decays)} decays for {H} heads"
    if not (q.dtype == k.dtype == v.dtype):
        raise ValueError("q, k and v must share one dtype")
    if s is not None and s.dtype != q.dtype and not (s.dtype == torch.float32 and q.dtype == torch.bfloat16):
        raise ValueError("the state must have the dtype of q, k, v, or be float32 under bfloat16 activations")
    if s is not None and tuple(s.shape) != (B, H, dk, dv):
        raise ValueError(f"state must be (B,H,dk,dv)={(B, H, dk, dv)}, got {tuple(s.shape)}")
    return _lib.unit_inner(q), _lib.unit_inner(k), _lib.unit_inner(v), _lib.state_tensor(s)


def _state_dtype(q, s, state_dtype):
    """Element type of the call's states: the one asked for, else that of the given state, else that of q."""
    sdt = state_dtype or (s.dtype if s is not None else q.dtype)
    if sdt != q.dtype and not (sdt == torch.float32 and q.dtype == torch.bfloat16):
        raise ValueError(f"state dtype {sdt} is not available with {q.dtype} activations")
    return sdt


class FusedChunkRetention(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, s, head_decays: Sequence[float], state_dtype: Optional[torch.dtype] = None):
        head_decays = tuple(float(g) for g in head_decays)
        q, k, v, s = _prepare(q, k, v, s, head_decays)
        B, T, H, dk = q.shape
        dv = v.shape[-1]
        sdt = _state_dtype(q, s, state_dtype)
        if s is not None and s.dtype != sdt:
            s = s.to(sdt)
        o = torch.empty((B, T, H, dv), device=q.device, dtype=q.dtype)
        s_out = torch.empty((B, H, dk, dv), device=q.device, dtype=sdt)
        flags = _flags() | (_lib.FLAG_STATE_F32 if sdt != q.dtype else 0)
        with torch.cuda.device(q.device):
            d = _lib.dims(q, dv, head_decays, flags=flags, workspace=True)
            _lib.check(_lib.lib().fpb_retention_fwd(d, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(s),
                                                    _lib.seq(o), _lib.state(s_out), _lib.stream_ptr(q.device)))
        ctx.save_for_backward(q, k, v, s)
        ctx.head_decays = head_decays
        ctx.flags = flags
        ctx.state_dtype = sdt
        ctx.set_materialize_grads(False)
        return o, s_out

    @staticmethod
    def backward(ctx, dO, dS_new):
        q, k, v, s = ctx.saved_tensors
        B, T, H, dk = q.shape
        dv = v.shape[-1]
        if dO is None:
            dO = torch.zeros((B, T, H, dv), device=q.device, dtype=q.dtype)
        dO = _lib.unit_inner(dO.to(q.dtype))
        sdt = ctx.state_dtype
        dS_new = _lib.state_tensor(None if dS_new is None else dS_new.to(sdt))
        # leave out the walk nobody needs: dQ is one launch, dK/dV/dS_0 the other
        need_q = ctx.needs_input_grad[0]
        need_s = s is not None and ctx.needs_input_grad[3]
        need_kv = ctx.needs_input_grad[1] or ctx.needs_input_grad[2] or need_s
        flags = ctx.flags | (0 if need_q else _lib.FLAG_SKIP_DQ) | (0 if need_kv else _lib.FLAG_SKIP_DKDV)
        dQ = torch.empty_like(q) if need_q else None
        dK = torch.empty_like(k) if need_kv else None
        dV = torch.empty_like(v) if need_kv else None
        dS = torch.empty((B, H, dk, dv), device=q.device, dtype=sdt) if need_s else None
        if need_q or need_kv:
            with torch.cuda.device(q.device):
                d = _lib.dims(q, dv, ctx.head_decays, flags=flags, workspace=True)
                _lib.check(_lib.lib().fpb_retention_bwd(d, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(s),
                                                        _lib.seq(dO), _lib.state(dS_new), _lib.seq(dQ), _lib.seq(dK),
                                                        _lib.seq(dV), _lib.state(dS), _lib.stream_ptr(q.device)))
        return dQ, dK, dV, dS, None, None


fused_chunk_retention = FusedChunkRetention.apply


def retention_forward_backward_into(q, k, v, dO, head_decays: Sequence[float], o, dQ, dK, dV) -> None:
    """Forward and backward of the operator (zero start state, no state gradient) written straight into tensors the
    caller provides - views of a staging buffer, say - instead of freshly allocated ones: two calls of the C ABI, no
    autograd graph, no copies.  All tensors (B,T,H,d) on one CUDA device, unit inner stride."""
    _lib.require_cuda(q, k, v, dO, o, dQ, dK, dV)
    head_decays = tuple(float(g) for g in head_decays)
    dv = v.shape[-1]
    for t in (q, k, v, dO, o, dQ, dK, dV):
        if t.stride(-1) != 1:
            raise ValueError("retention_forward_backward_into takes tensors with unit inner stride")
    with torch.cuda.device(q.device):
        stream = _lib.stream_ptr(q.device)
        d = _lib.dims(q, dv, head_decays, flags=_flags(), workspace=True)
        _lib.check(_lib.lib().fpb_retention_fwd(d, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(None), _lib.seq(o),
                                                _lib.state(None), stream))
        _lib.check(_lib.lib().fpb_retention_bwd(d, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(None), _lib.seq(dO),
                                                _lib.state(None), _lib.seq(dQ), _lib.seq(dK), _lib.seq(dV), _lib.state(None),
                                                stream))


def retention_step(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, head_decays: Sequence[float],
                   prev_state: Optional[torch.Tensor] = None, *, state_dtype: Optional[torch.dtype] = None,
                   in_place: bool = False):
    """One recurrent decoding step, S = gamma S_prev + k^T v / sqrt(dk), o = q S, as one streaming kernel over the
    state (the reference's ``retention_recurrent``, flash_pop/retnet.py:79-101).

    q, k: (B, H, dk); v: (B, H, dv); prev_state: (B, H, dk, dv) or None (zeros).  Returns (o (B, H, dv), state).
    The state's element type is ``state_dtype``, else that of ``prev_state``, else that of q; with ``in_place`` the
    new state overwrites ``prev_state``.  Inference only: no gradient is recorded."""
    _lib.require_cuda(q, k, v, prev_state)
    if q.dim() != 3 or k.shape != q.shape or v.dim() != 3 or v.shape[:2] != q.shape[:2]:
        raise ValueError(f"expected q,k (B,H,dk) and v (B,H,dv); got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    B, H, dk = q.shape
    dv = v.shape[-1]
    head_decays = tuple(float(g) for g in head_decays)
    assert len(head_decays) == H, f"got {len(head_decays)} decays for {H} heads"
    if not (q.dtype == k.dtype == v.dtype):
        raise ValueError("q, k and v must share one dtype")
    if prev_state is not None and tuple(prev_state.shape) != (B, H, dk, dv):
        raise ValueError(f"state must be (B,H,dk,dv)={(B, H, dk, dv)}, got {tuple(prev_state.shape)}")
    sdt = state_dtype or (prev_state.dtype if prev_state is not None else q.dtype)
    if prev_state is not None and prev_state.dtype != sdt:
        prev_state, in_place = prev_state.to(sdt), False
    prev_state = _lib.state_tensor(prev_state)
    q4, k4, v4 = (_lib.unit_inner(t.detach()).unsqueeze(1) for t in (q, k, v))
    o = torch.empty((B, 1, H, dv), device=q.device, dtype=q.dtype)
    state = prev_state if (in_place and prev_state is not None) else torch.empty((B, H, dk, dv), device=q.device, dtype=sdt)
    with torch.cuda.device(q.device):
        d = _lib.dims(q4, dv, head_decays)
        _lib.check(_lib.lib().fpb_retention_step(d, _lib.dtype_code(state), _lib.seq(q4), _lib.seq(k4), _lib.seq(v4),
                                                 _lib.state(None if prev_state is None else prev_state.detach()),
                                                 _lib.seq(o), _lib.state(state), _lib.stream_ptr(q.device)))
    return o.squeeze(1), state
