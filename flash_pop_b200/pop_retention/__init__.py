"""POP (parallel observation prediction) retention over the C ABI.

``flash_pop_retention(q, k, v, s, head_decays, block_size) -> (o, block_states)`` is the reference
operator (flash_pop/pop_retention/__init__.py:11-52): retention over the observation stream that
also returns the state after every full block, ``block_states`` (B, T // block_size, H, dk, dv).

``pop_suffix_retention(sq, sk, sv, s, block_states, head_decays)`` runs the prediction-token suffixes
(flash_pop/pop_retnet.py:152-171): suffix m of row b starts from the state at the start of block m,
read in place from ``s`` / ``block_states`` (no concatenated copy), and never writes a state.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from flash_pop_b200 import _lib
from flash_pop_b200.fused_retention import _flags, _prepare, _state_dtype


class FlashPOPRetention(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, s, head_decays: Sequence[float], block_size: int, state_dtype: Optional[torch.dtype] = None):
        head_decays = tuple(float(g) for g in head_decays)
        block_size = int(block_size)
        q, k, v, s = _prepare(q, k, v, s, head_decays)
        B, T, H, dk = q.shape
        dv = v.shape[-1]
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        sdt = _state_dtype(q, s, state_dtype)
        if s is not None and s.dtype != sdt:
            s = s.to(sdt)
        o = torch.empty((B, T, H, dv), device=q.device, dtype=q.dtype)
        block_states = torch.empty((B, T // block_size, H, dk, dv), device=q.device, dtype=sdt)
        flags = _flags() | (_lib.FLAG_STATE_F32 if sdt != q.dtype else 0)
        with torch.cuda.device(q.device):
            d = _lib.dims(q, dv, head_decays, block_size=block_size, flags=flags, workspace=True)
            _lib.check(_lib.lib().fpb_pop_retention_fwd(d, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(s),
                                                        _lib.seq(o), block_states.data_ptr(),
                                                        _lib.stream_ptr(q.device)))
        ctx.save_for_backward(q, k, v, s)
        ctx.head_decays, ctx.block_size, ctx.flags, ctx.state_dtype = head_decays, block_size, flags, sdt
        ctx.set_materialize_grads(False)
        return o, block_states

    @staticmethod
    def backward(ctx, dO, d_block_states):
        q, k, v, s = ctx.saved_tensors
        B, T, H, dk = q.shape
        dv = v.shape[-1]
        if dO is None:
            dO = torch.zeros((B, T, H, dv), device=q.device, dtype=q.dtype)
        dO = _lib.unit_inner(dO.to(q.dtype))
        sdt = ctx.state_dtype
        if d_block_states is not None:
            d_block_states = d_block_states.to(sdt).contiguous()
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
                d = _lib.dims(q, dv, ctx.head_decays, block_size=ctx.block_size, flags=flags, workspace=True)
                _lib.check(_lib.lib().fpb_pop_retention_bwd(
                    d, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(s), _lib.seq(dO),
                    None if d_block_states is None else d_block_states.data_ptr(),
                    _lib.seq(dQ), _lib.seq(dK), _lib.seq(dV), _lib.state(dS), _lib.stream_ptr(q.device)))
        return dQ, dK, dV, dS, None, None, None


flash_pop_retention = FlashPOPRetention.apply


def pop_retention_forward_backward_into(q, k, v, dO, head_decays: Sequence[float], block_size: int, o, block_states, dQ, dK, dV) -> None:
    """Forward and backward of POP retention (zero start state, no gradient into the block states) written straight
    into tensors the caller provides - views of a staging buffer, say: two calls of the C ABI, no autograd graph, no
    copies.  q ... dV (B,T,H,d) with unit inner stride; block_states (B, T // block_size, H, dk, dv) contiguous, of q's
    dtype."""
    _lib.require_cuda(q, k, v, dO, o, block_states, dQ, dK, dV)
    head_decays = tuple(float(g) for g in head_decays)
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    for t in (q, k, v, dO, o, dQ, dK, dV):
        if t.stride(-1) != 1:
            raise ValueError("pop_retention_forward_backward_into takes tensors with unit inner stride")
    if tuple(block_states.shape) != (B, T // int(block_size), H, dk, dv) or not block_states.is_contiguous() or block_states.dtype != q.dtype:
        raise ValueError("block_states must be a contiguous (B, T // block_size, H, dk, dv) tensor of q's dtype")
    with torch.cuda.device(q.device):
        stream = _lib.stream_ptr(q.device)
        d = _lib.dims(q, dv, head_decays, block_size=int(block_size), flags=_flags(), workspace=True)
        _lib.check(_lib.lib().fpb_pop_retention_fwd(d, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(None), _lib.seq(o),
                                                    block_states.data_ptr(), stream))
        _lib.check(_lib.lib().fpb_pop_retention_bwd(d, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(None), _lib.seq(dO), None,
                                                    _lib.seq(dQ), _lib.seq(dK), _lib.seq(dV), _lib.state(None), stream))


class POPSuffixRetention(torch.autograd.Function):

    @staticmethod
    def forward(ctx, sq, sk, sv, s, block_states, head_decays: Sequence[float]):
        head_decays = tuple(float(g) for g in head_decays)
        _lib.require_cuda(sq, sk, sv, s, block_states)
        if sq.dim() != 5:
            raise ValueError("suffix tensors must be (B, M, P, H, d)")
        B, M, P, H, dk = sq.shape
        dv = sv.shape[-1]
        N = block_states.shape[1]
        assert len(head_decays) == H
        if M > N + 1:
            raise ValueError(f"{M} suffixes per row need at least {M - 1} block states, got {N}")
        fq, fk, fv = (_lib.unit_inner(t.flatten(0, 1)) for t in (sq, sk, sv))
        sdt = block_states.dtype
        if sdt != sq.dtype and not (sdt == torch.float32 and sq.dtype == torch.bfloat16):
            raise ValueError("block_states must have the dtype of the suffix tensors, or be float32 under bfloat16 activations")
        s = _lib.state_tensor(None if s is None else s.to(sdt))
        block_states = block_states.contiguous()
        o = torch.empty((B * M, P, H, dv), device=sq.device, dtype=sq.dtype)
        flags = _flags() | (_lib.FLAG_STATE_F32 if sdt != sq.dtype else 0)
        with torch.cuda.device(sq.device):
            d = _lib.dims(fq, dv, head_decays, flags=flags, batch=B)
            _lib.check(_lib.lib().fpb_pop_suffix_fwd(d, M, N, _lib.seq(fq), _lib.seq(fk), _lib.seq(fv), _lib.state(s),
                                                     block_states.data_ptr(), _lib.seq(o), _lib.stream_ptr(sq.device)))
        ctx.save_for_backward(fq, fk, fv, s, block_states)
        ctx.head_decays, ctx.flags, ctx.shape = head_decays, flags, (B, M, N)
        return o.unflatten(0, (B, M))

    @staticmethod
    def backward(ctx, dO):
        fq, fk, fv, s, block_states = ctx.saved_tensors
        B, M, N = ctx.shape
        _, P, H, dk = fq.shape
        dv = fv.shape[-1]
        dO = _lib.unit_inner(dO.to(fq.dtype).flatten(0, 1))
        dQ, dK, dV = torch.empty_like(fq), torch.empty_like(fk), torch.empty_like(fv)
        dS = torch.empty((B, H, dk, dv), device=fq.device, dtype=block_states.dtype) if s is not None else None
        dBS = torch.empty_like(block_states)
        with torch.cuda.device(fq.device):
            d = _lib.dims(fq, dv, ctx.head_decays, flags=ctx.flags, batch=B)
            _lib.check(_lib.lib().fpb_pop_suffix_bwd(
                d, M, N, _lib.seq(fq), _lib.seq(fk), _lib.seq(fv), _lib.state(s), block_states.data_ptr(),
                _lib.seq(dO), _lib.seq(dQ), _lib.seq(dK), _lib.seq(dV), _lib.state(dS), dBS.data_ptr(),
                _lib.stream_ptr(fq.device)))
        unf = lambda t: t.unflatten(0, (B, M))
        return unf(dQ), unf(dK), unf(dV), dS, dBS, None


def pop_suffix_retention(sq, sk, sv, s: Optional[torch.Tensor], block_states, head_decays):
    """sq, sk: (B, M, P, H, dk); sv: (B, M, P, H, dv); s: (B,H,dk,dv) or None; block_states (B,N,H,dk,dv),
    M <= N + 1.  Returns (B, M, P, H, dv)."""
    return POPSuffixRetention.apply(sq, sk, sv, s, block_states, head_decays)
