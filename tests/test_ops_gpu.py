"""Parity of the CUDA operators (called through the C ABI) with the CPU oracle on identical seeded
inputs: outputs, states, block states and all gradients."""
import os

import numpy as np
import pytest
import torch

from oracle import retention_oracle as orc
from tests.util import check, make_inputs

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def ops():
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib, fused_retention
    return fp, _lib, fused_retention


def run_fwd_bwd(q, k, v, s, decays, dO, dS, simt):
    fp, _lib, fr = ops()
    dev = "cuda"
    leaves = [None if t is None else t.to(dev).requires_grad_(True) for t in (q, k, v, s)]
    ctx = fr.cuda_core_kernels() if simt else _null()
    with ctx:
        o, s_out = fp.fused_chunk_retention(*leaves, decays)
        path = _lib.last_path()
        loss = (o.float() * dO.to(dev).float()).sum()
        if dS is not None:
            loss = loss + (s_out.float() * dS.to(dev).float()).sum()
        loss.backward()
    _lib.device_status()
    grads = [None if t is None else t.grad for t in leaves]
    return o, s_out, grads, path


class _null:
    def __enter__(self): return self
    def __exit__(self, *a): return False


def oracle_fwd_bwd(q, k, v, s, decays, dO, dS, chunk=64):
    qd, kd, vd = q.double(), k.double(), v.double()
    sd = None if s is None else s.double()
    o, s_out = orc.retention_chunkwise(qd, kd, vd, sd, decays, chunk_size=chunk)
    g = orc.retention_grads_chunked(qd, kd, vd, sd, decays, dO.double(), None if dS is None else dS.double(), chunk)
    return o, s_out, g


# ---- the CPU-runnable reference case: fp32, B=2,H=4,T=256,d=64, default decays, compared with the parallel form ----
def test_config1_fp32_against_parallel_form():
    B, T, H, d = 2, 256, 4, 64
    decays = orc.head_decays(H)
    q, k, v, _, g = make_inputs(0, B, T, H, d, d, torch.float32, state=False)
    G = torch.randn(B, T, H, d, generator=g)
    o, s_out, grads, path = run_fwd_bwd(q, k, v, None, decays, G, None, simt=False)
    o_ref, s_ref = orc.retention_parallel(q.double(), k.double(), v.double(), None, decays)
    dQ, dK, dV, _ = orc.retention_grads(q.double(), k.double(), v.double(), None, decays, G.double(), None)
    check("O", o, o_ref, torch.float32), check("S", s_out, s_ref, torch.float32)
    check("dQ", grads[0], dQ, torch.float32), check("dK", grads[1], dK, torch.float32), check("dV", grads[2], dV, torch.float32)


SIMT_CASES = [
    # B, T, H, dk, dv, dtype, state, dS
    (2, 70, 3, 16, 24, torch.float32, True, True),       # ragged, dk != dv, odd dims
    (1, 1, 2, 8, 8, torch.float32, True, True),          # single token
    (2, 130, 2, 64, 128, torch.bfloat16, True, True),
    (1, 33, 2, 200, 256, torch.float32, False, False),   # largest dims the CUDA-core path takes
    (3, 47, 5, 40, 72, torch.bfloat16, True, False),
]


@pytest.mark.parametrize("B,T,H,dk,dv,dtype,state,with_dS", SIMT_CASES)
def test_cuda_core_path(B, T, H, dk, dv, dtype, state, with_dS):
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s, g = make_inputs(7, B, T, H, dk, dv, dtype, scale=1.0 if dtype == torch.float32 else None, state=state)
    dO = torch.randn(B, T, H, dv, generator=g).to(dtype)
    dS = torch.randn(B, H, dk, dv, generator=g).to(dtype) if with_dS else None
    o, s_out, grads, path = run_fwd_bwd(q, k, v, s, decays, dO, dS, simt=True)
    _, _lib, _ = ops()
    assert path == _lib.PATH_SIMT
    o_ref, s_ref, (dQ, dK, dV, dS0) = oracle_fwd_bwd(q, k, v, s, decays, dO, dS)
    check("O", o, o_ref, dtype), check("S", s_out, s_ref, dtype)
    check("dQ", grads[0], dQ, dtype), check("dK", grads[1], dK, dtype), check("dV", grads[2], dV, dtype)
    if state:
        check("dS0", grads[3], dS0, dtype)


def test_golden_fixture_forward_and_grads_fp32():
    z = np.load(os.path.join(GOLD, "grads.npz"))
    t = {n: torch.from_numpy(z[n]) for n in z.files}
    decays = tuple(z["decays"].tolist())
    o, s_out, grads, _ = run_fwd_bwd(t["q"], t["k"], t["v"], t["s"], decays, t["dO"], t["dS"], simt=False)
    check("O", o, t["o"], torch.float32), check("S", s_out, t["s_out"], torch.float32)
    for got, name in zip(grads, ("dQ", "dK", "dV", "dS0")):
        check(name, got, t[name], torch.float32)


def test_zero_length_sequence_returns_start_state():
    fp, _lib, _ = ops()
    s = torch.randn(2, 3, 16, 16, device="cuda")
    q = torch.empty(2, 0, 3, 16, device="cuda")
    o, s_out = fp.fused_chunk_retention(q, q, q, s, orc.head_decays(3))
    assert o.shape == (2, 0, 3, 16)
    assert torch.equal(s_out, s)


def test_strided_head_views_are_taken_in_place():
    fp, _lib, _ = ops()
    B, T, H, d = 2, 40, 3, 16
    decays = orc.head_decays(H)
    g = torch.Generator().manual_seed(5)
    packed = torch.randn(B, T, 3 * H * d, generator=g).cuda()
    q, k, v = (packed[..., i * H * d:(i + 1) * H * d].unflatten(-1, (H, d)) for i in range(3))
    assert not q.is_contiguous()
    o, s_out = fp.fused_chunk_retention(q, k, v, None, decays)
    o_ref, s_ref = orc.retention_chunkwise(q.cpu().double(), k.cpu().double(), v.cpu().double(), None, decays, 64)
    check("O", o, o_ref, torch.float32), check("S", s_out, s_ref, torch.float32)


def test_bad_arguments_raise():
    fp, _lib, _ = ops()
    q = torch.randn(1, 8, 2, 16, device="cuda")
    with pytest.raises(AssertionError):
        fp.fused_chunk_retention(q, q, q, None, (0.9,))
    with pytest.raises(ValueError):
        fp.fused_chunk_retention(q, q, q, None, (0.9, 1.5))
    with pytest.raises(ValueError):
        fp.fused_chunk_retention(q.half(), q.half(), q.half(), None, (0.9, 0.9))
    with pytest.raises(RuntimeError):
        fp.fused_chunk_retention(q.cpu(), q.cpu(), q.cpu(), None, (0.9, 0.9))
    with pytest.raises(ValueError):
        fp.flash_pop_retention(q, q, q, None, (0.9, 0.9), 0)


def test_expanded_upstream_gradients_are_accepted():
    """A loss that sums the output over tokens or heads hands the backward an expand()-ed dO (stride 0 along that
    dimension), and q, k, v may themselves be expanded views: both are valid graphs for the reference operator and
    must be here too (they are made contiguous before they reach the C ABI)."""
    import flash_pop_b200 as fp
    B, T, H, d = 2, 150, 3, 64
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s, g = make_inputs(55, B, T, H, d, d, torch.bfloat16)
    w_t = torch.randn(B, H, d, generator=g)
    w_h = torch.randn(B, T, d, generator=g)
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, s)]
    o, _ = fp.fused_chunk_retention(*leaves, decays)
    ((o.float().sum(1) * w_t.cuda()).sum() + (o.float().sum(2) * w_h.cuda()).sum()).backward()
    ref = [t.double().requires_grad_(True) for t in (q, k, v, s)]
    o_ref, _ = orc.retention_chunkwise(*ref, decays, 64)
    ((o_ref.sum(1) * w_t.double()).sum() + (o_ref.sum(2) * w_h.double()).sum()).backward()
    for name, got, want in zip(("dQ", "dK", "dV", "dS0"), leaves, ref):
        check(name, got.grad, want.grad, torch.bfloat16, max_outside=1e-4, plain=name != "dS0")
    # the same with dO itself an expanded tensor, and with an expanded v
    dO = torch.randn(B, 1, H, d, generator=g).to(torch.bfloat16).cuda().expand(B, T, H, d)
    v1 = v[:, :1].cuda().expand(B, T, H, d)
    ql, kl = (t.cuda().requires_grad_(True) for t in (q, k))
    o, _ = fp.fused_chunk_retention(ql, kl, v1, None, decays)
    o.backward(dO)
    qr, kr = (t.double().requires_grad_(True) for t in (q, k))
    o_ref, _ = orc.retention_chunkwise(qr, kr, v[:, :1].double().expand(B, T, H, d), None, decays, 64)
    o_ref.backward(dO.cpu().double())
    check("O", o, o_ref, torch.bfloat16, max_outside=1e-4)
    check("dQ", ql.grad, qr.grad, torch.bfloat16, max_outside=1e-4), check("dK", kl.grad, kr.grad, torch.bfloat16, max_outside=1e-4)
