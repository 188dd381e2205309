"""Helpers shared by the parity tests: seeded inputs with the configured laws and the three
acceptance checks (allclose, relative RMS, scale-aware elementwise bound)."""
from __future__ import annotations

import torch

from oracle import retention_oracle as orc


def make_inputs(seed, B, T, H, dk, dv, dtype, scale=None, state=True, device="cpu"):
    """q, k, v ~ N(0,1) * scale (default dk^-0.5, the configured input law), optional start state."""
    g = torch.Generator().manual_seed(seed)
    scale = dk ** -0.5 if scale is None else scale
    q = (torch.randn(B, T, H, dk, generator=g) * scale).to(dtype)
    k = (torch.randn(B, T, H, dk, generator=g) * scale).to(dtype)
    v = (torch.randn(B, T, H, dv, generator=g) * scale).to(dtype)
    s = (torch.randn(B, H, dk, dv, generator=g) * scale).to(dtype) if state else None
    return q, k, v, s, g


def rel_rms(a, r):
    return orc.rel_rms(a.detach().cpu(), r.detach().cpu())


def check(name, got, ref, dtype, rms_limit=None, max_outside=0.0, plain=True):
    """north-star tolerance (rtol=atol=2e-2 bf16, 1e-4 fp32) + the reference's own rel-RMS < 0.005
    + a bound that scales with the data so that tiny-magnitude tensors are still pinned.  `max_outside` is the
    fraction of elements allowed outside that last bound (0 for the small cases; the full-size cases compare
    10^7-10^8 bf16 elements, where the far tail of the rounding-error distribution crosses any fixed multiple).
    `plain=False` leaves out the fixed-tolerance allclose: for tensors whose magnitude is far above 1 (a state gradient
    summed over thousands of unit-variance tokens) no bf16-operand kernel can meet an absolute 2e-2, and the two
    scale-aware criteria are the ones that bind."""
    got = got.detach().float().cpu().double()
    ref = ref.detach().cpu().double()
    assert got.shape == ref.shape, f"{name}: shape {tuple(got.shape)} != {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{name}: non-finite values"
    if ref.numel() == 0:
        return
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    err = (got - ref).abs()
    rms_ref = ref.square().mean().sqrt().item()
    if plain:
        assert (err <= tol + tol * ref.abs()).all(), f"{name}: allclose({tol}) failed, max err {err.max().item():.3e}"
    bound = tol * rms_ref + tol * ref.abs()
    frac_out = (err > bound).double().mean().item()
    assert frac_out <= max_outside, f"{name}: {frac_out:.2%} outside scale-aware bound; max err {err.max().item():.3e}, rms(ref) {rms_ref:.3e}"
    rr = rel_rms(got, ref)
    limit = rms_limit if rms_limit is not None else (5e-3 if dtype == torch.bfloat16 else 2e-5)
    assert rr < limit, f"{name}: rel-RMS {rr:.3e} >= {limit}"
