"""CPU oracle for the retention / POP-retention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the algorithm that the reference
project (leor-c/flash-pop) implements in its own PyTorch retention code.  It is the
checker for the CUDA kernels: only the test-suite, the smoke entry and the CPU-baseline /
reference legs of the benchmark may import it.  Nothing in the shipped package imports it,
and the shipped package has no CPU path at all.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the reference's own
functions (``chunkwise_retention``, ``reference_grads``, ``retention_recurrent`` and the
test helper ``ref_pop``) and stores their outputs on seeded inputs as fixtures; the
CPU tests check every function below against those fixtures.

Conventions (identical to the reference):
  q, k : (B, T, H, dk)      v, o : (B, T, H, dv)      state : (B, H, dk, dv)
  the operator scales K by 1/sqrt(dk) itself      (fused_retention/reference.py:57)
  decay of head h is a Python float gamma_h in (0, 1)

All functions compute in the dtype of ``q`` (pass ``.double()`` tensors for a float64
oracle).  Decay powers follow the reference exactly: gamma is first rounded to float32
and the powers are taken in float32 (fused_retention/__init__.py:73-102,
fused_retention/reference.py:15,31-36), then cast to the compute dtype.
"""
from __future__ import annotations

from math import ceil
from typing import Optional, Sequence, Tuple

import numpy as np
import torch
from torch import Tensor


# --------------------------------------------------------------------------------------
# decays
# --------------------------------------------------------------------------------------
def head_decays(num_heads: int, decay_range: Optional[Tuple[float, float]] = None) -> Tuple[float, ...]:
    """gamma_h = 1 - 2^(-5-h), or 1 - 2^(-linspace(lo, hi, H)).  (flash_pop/retnet.py:70-76)"""
    if decay_range is None:
        expo = -5.0 - np.arange(num_heads)
    else:
        expo = -np.linspace(decay_range[0], decay_range[1], num_heads)
    return tuple((1.0 - np.exp2(expo)).tolist())


def _gamma32(decays: Sequence[float]) -> Tensor:
    return torch.tensor(tuple(decays), dtype=torch.float32)


def _pow32(decays: Sequence[float], exponents: Tensor, dtype) -> Tensor:
    """gamma_h ** e for every head and exponent, float32 like the reference. -> (H, len(e))"""
    g = _gamma32(decays).view(-1, 1)
    return (g ** exponents.to(torch.float32).view(1, -1)).to(dtype)


def decay_mask(decays: Sequence[float], length: int, dtype=torch.float32) -> Tensor:
    """D[h, i, j] = gamma_h^(i-j) for i >= j, else 0.  (fused_retention/__init__.py:73-102)"""
    pos = torch.arange(length, dtype=torch.float32)
    dist = pos.view(-1, 1) - pos.view(1, -1)
    g = _gamma32(decays).view(-1, 1, 1)
    return (g ** dist.unsqueeze(0)).tril().to(dtype)


# --------------------------------------------------------------------------------------
# forward forms
# --------------------------------------------------------------------------------------
def _one_chunk(q: Tensor, k_scaled: Tensor, v: Tensor, state: Optional[Tensor], decays) -> Tuple[Tensor, Tensor]:
    """Parallel form over one chunk given the state at its start; K already scaled.
    (fused_retention/reference.py:10-50)"""
    dtype = q.dtype
    L = q.size(1)
    D = decay_mask(decays, L, dtype)                                   # (H, L, L)
    scores = torch.einsum("bihd,bjhd->bhij", q, k_scaled) * D.unsqueeze(0)
    out = torch.einsum("bhij,bjhe->bihe", scores, v)

    pos = torch.arange(L)
    eta = _pow32(decays, (L - 1 - pos), dtype)                         # (H, L): gamma^(L-1-j)
    new_state = torch.einsum("bjhd,hj,bjhe->bhde", k_scaled, eta, v)
    if state is not None:
        zeta = _pow32(decays, pos + 1, dtype)                          # (H, L): gamma^(i+1)
        gL = _pow32(decays, torch.tensor([L]), dtype).view(1, -1, 1, 1)
        new_state = new_state + state.to(dtype) * gL
        out = out + torch.einsum("bihd,bhde->bihe", q, state.to(dtype)) * zeta.t().view(1, L, -1, 1)
    return out, new_state


def retention_chunkwise(q, k, v, state, decays, chunk_size: int = 512) -> Tuple[Tensor, Tensor]:
    """Chunk-by-chunk retention; equals the parallel form for chunk_size >= T.
    (fused_retention/reference.py:53-69)"""
    T = q.size(1)
    ks = k / (k.size(3) ** 0.5)
    outs = []
    for c in range(ceil(T / chunk_size)):
        sl = slice(c * chunk_size, (c + 1) * chunk_size)
        o_c, state = _one_chunk(q[:, sl], ks[:, sl], v[:, sl], state, decays)
        outs.append(o_c)
    return torch.cat(outs, dim=1), state


def retention_parallel(q, k, v, state, decays) -> Tuple[Tensor, Tensor]:
    """Whole sequence as a single chunk (O(T^2) memory)."""
    return retention_chunkwise(q, k, v, state, decays, chunk_size=q.size(1))


def retention_recurrent(q, k, v, state, decays) -> Tuple[Tensor, Tensor]:
    """Token-by-token form: S_t = gamma S_{t-1} + k_t^T v_t / sqrt(dk); o_t = q_t S_t.
    (flash_pop/retnet.py:79-101, applied T times)"""
    B, T, H, dk = q.shape
    dtype = q.dtype
    g = _gamma32(decays).to(dtype).view(1, H, 1, 1)
    S = torch.zeros(B, H, dk, v.size(3), dtype=dtype) if state is None else state.to(dtype).clone()
    ks = k / (dk ** 0.5)
    outs = []
    for t in range(T):
        S = S * g + torch.einsum("bhd,bhe->bhde", ks[:, t], v[:, t])
        outs.append(torch.einsum("bhd,bhde->bhe", q[:, t], S))
    return torch.stack(outs, dim=1), S


def pop_retention(q, k, v, state, decays, block_size: int) -> Tuple[Tensor, Tensor]:
    """Retention that also returns the state after every FULL block of ``block_size`` tokens:
    block_states[:, n] = state after token (n+1)*block_size - 1, n < T // block_size.
    (tests/test_pop_retention.py:13-32; pop_retention/pop_fwd.py:9,41-43)"""
    T = q.size(1)
    ks = k / (k.size(3) ** 0.5)
    outs, states = [], []
    for n in range(ceil(T / block_size)):
        sl = slice(n * block_size, (n + 1) * block_size)
        o_n, state = _one_chunk(q[:, sl], ks[:, sl], v[:, sl], state, decays)
        outs.append(o_n)
        if (n + 1) * block_size <= T:
            states.append(state)
    B, _, H, dk = q.shape
    if states:
        bs = torch.stack(states, dim=1)
    else:
        bs = torch.zeros(B, 0, H, dk, v.size(3), dtype=q.dtype)
    return torch.cat(outs, dim=1), bs


def pop_suffix_retention(sq, sk, sv, state0, block_states, decays) -> Tensor:
    """Prediction-token suffixes: suffix n of batch row b is ordinary retention started from
    the state at the START of block n, i.e. [S_0, block_states[:,0], ..., block_states[:,N-1]];
    its own end state is dropped, so the stream state is never written.
    (flash_pop/pop_retnet.py:152-171)

    sq, sk : (B, M, P, H, dk)   sv : (B, M, P, H, dv)   with M <= N + 1 suffixes per row.
    returns (B, M, P, H, dv)."""
    B, M = sq.shape[:2]
    if state0 is None:
        state0 = torch.zeros_like(block_states[:, 0]) if block_states.size(1) else None
    starts = torch.cat((state0.unsqueeze(1), block_states), dim=1)[:, :M]
    o, _ = retention_chunkwise(sq.flatten(0, 1), sk.flatten(0, 1), sv.flatten(0, 1),
                               starts.flatten(0, 1), decays, chunk_size=sq.size(2))
    return o.unflatten(0, (B, M))


# --------------------------------------------------------------------------------------
# gradients
# --------------------------------------------------------------------------------------
def retention_grads(q, k, v, state, decays, dO, dS_new):
    """Closed-form gradients of the parallel form (O(T^2) memory), in terms of UNSCALED k.
    (fused_retention/reference.py:72-111)   returns dQ, dK, dV, dS_0"""
    dtype = q.dtype
    B, T, H, dk = q.shape
    rs = 1.0 / (dk ** 0.5)
    D = decay_mask(decays, T, dtype)
    pos = torch.arange(T)
    zeta = _pow32(decays, pos + 1, dtype)            # (H, T)
    eta = _pow32(decays, T - 1 - pos, dtype)         # (H, T)
    gT = _pow32(decays, torch.tensor([T]), dtype).view(1, H, 1, 1)
    if state is None:
        state = torch.zeros(B, H, dk, v.size(3), dtype=dtype)
    if dS_new is None:
        dS_new = torch.zeros_like(state)

    P = torch.einsum("bihe,bjhe->bhij", dO, v) * rs * D.unsqueeze(0)
    dOz = dO * zeta.t().view(1, T, H, 1)
    dQ = torch.einsum("bhij,bjhd->bihd", P, k) + torch.einsum("bihe,bhde->bihd", dOz, state)
    dK = torch.einsum("bhij,bihd->bjhd", P, q) + torch.einsum("bjhe,bhde,hj->bjhd", v, dS_new, eta) * rs
    A = torch.einsum("bihd,bjhd->bhij", q, k) * rs * D.unsqueeze(0)
    dV = torch.einsum("bhij,bihe->bjhe", A, dO) + torch.einsum("bjhd,hj,bhde->bjhe", k * rs, eta, dS_new)
    dS0 = torch.einsum("bihd,bihe->bhde", q, dOz) + gT * dS_new
    return dQ, dK, dV, dS0


def pop_retention_grads(q, k, v, state, decays, block_size, dO, d_block_states, chunk_size: int = 64):
    """Gradients of ``pop_retention`` by a forward walk (dQ) and a reverse walk carrying the
    gradient of the running state (dK, dV, dS_0), cutting chunks at block ends and adding
    ``d_block_states[:, n]`` to the carried gradient where block n ends.
    (walk structure: fused_retention/fused_chunk_bwd.py:286-342,405-446;
     block-end injection: pop_retention/pop_bwd.py:137-159)

    With ``d_block_states`` empty and ``block_size`` >= T this is the plain chunked backward
    with dS_new = 0."""
    dtype = q.dtype
    B, T, H, dk = q.shape
    dv = v.size(3)
    bounds = chunk_schedule(T, block_size, chunk_size)
    if state is None:
        state = torch.zeros(B, H, dk, dv, dtype=dtype)
    ks = k / (dk ** 0.5)

    dQ = torch.zeros_like(q)
    dK = torch.zeros_like(k)
    dV = torch.zeros_like(v)
    S = state.to(dtype)
    for (a, b) in bounds:                                       # forward walk: dQ needs start states
        zero = torch.zeros_like(S)
        dq_c, _, _, _ = retention_grads(q[:, a:b], k[:, a:b], v[:, a:b], S, decays, dO[:, a:b], zero)
        dQ[:, a:b] = dq_c
        _, S = _one_chunk(q[:, a:b], ks[:, a:b], v[:, a:b], S, decays)
    G = torch.zeros(B, H, dk, dv, dtype=dtype)                  # gradient of the state after the chunk
    for (a, b) in reversed(bounds):
        if b % block_size == 0 and b // block_size - 1 < d_block_states.size(1):
            G = G + d_block_states[:, b // block_size - 1].to(dtype)
        _, dk_c, dv_c, G = retention_grads(q[:, a:b], k[:, a:b], v[:, a:b], None, decays, dO[:, a:b], G)
        dK[:, a:b] = dk_c
        dV[:, a:b] = dv_c
    return dQ, dK, dV, G


def retention_grads_chunked(q, k, v, state, decays, dO, dS_new, chunk_size: int = 64):
    """Chunked (O(T*chunk) memory) version of ``retention_grads``."""
    dtype = q.dtype
    B, T, H, dk = q.shape
    dv = v.size(3)
    bounds = chunk_schedule(T, T + 1, chunk_size)
    if state is None:
        state = torch.zeros(B, H, dk, dv, dtype=dtype)
    ks = k / (dk ** 0.5)
    dQ, dK, dV = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    S = state.to(dtype)
    for (a, b) in bounds:
        dQ[:, a:b] = retention_grads(q[:, a:b], k[:, a:b], v[:, a:b], S, decays, dO[:, a:b],
                                     torch.zeros_like(S))[0]
        _, S = _one_chunk(q[:, a:b], ks[:, a:b], v[:, a:b], S, decays)
    G = torch.zeros(B, H, dk, dv, dtype=dtype) if dS_new is None else dS_new.to(dtype)
    for (a, b) in reversed(bounds):
        _, dK[:, a:b], dV[:, a:b], G = retention_grads(q[:, a:b], k[:, a:b], v[:, a:b], None, decays,
                                                       dO[:, a:b], G)
    return dQ, dK, dV, G


def chunk_schedule(T: int, block_size: int, chunk_size: int):
    """Token ranges [a, b) walked by the chunked kernels: every block of ``block_size`` tokens is
    cut into chunks of at most ``chunk_size`` starting at the block start, so that every block end
    is also a chunk end."""
    out = []
    a = 0
    while a < T:
        block_end = (a // block_size + 1) * block_size
        b = min(a + chunk_size, block_end, T)
        out.append((a, b))
        a = b
    return out


# --------------------------------------------------------------------------------------
# error metrics used by the reference's own checks
# --------------------------------------------------------------------------------------
def rel_rms(approx: Tensor, ref: Tensor) -> float:
    """||a - r||_2 / ||r||_2   (tests/test_fused_retention.py:36-39)"""
    a, r = approx.double().flatten(), ref.double().flatten()
    return ((a - r).square().mean().sqrt() / r.square().mean().sqrt().clamp_min(1e-300)).item()
