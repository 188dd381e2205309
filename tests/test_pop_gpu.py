"""Parity of the POP operators with the CPU oracle: block states, ragged tails, several block ends
inside one 64-token chunk, blocks longer than a chunk, suffixes started from block states."""
import os

import numpy as np
import pytest
import torch

from oracle import retention_oracle as orc
from tests.util import check, make_inputs

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def run_pop(q, k, v, s, decays, block, dO, dBS, simt):
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib, fused_retention
    leaves = [None if t is None else t.cuda().requires_grad_(True) for t in (q, k, v, s)]
    ctx = fused_retention.cuda_core_kernels() if simt else _null()
    with ctx:
        o, bs = fp.flash_pop_retention(*leaves, decays, block)
        loss = (o.float() * dO.cuda().float()).sum()
        if bs.numel():
            loss = loss + (bs.float() * dBS.cuda().float()).sum()
        loss.backward()
    _lib.device_status()
    return o, bs, [None if t is None else t.grad for t in leaves]


class _null:
    def __enter__(self): return self
    def __exit__(self, *a): return False


POP_CASES = [
    # B, T, H, dk, dv, block, dtype, simt     (reference cases: tests/test_pop_retention.py:161-262)
    (2, 287, 2, 64, 128, 144, torch.bfloat16, True),    # "generation": one full block + tail
    (2, 28, 2, 64, 128, 15, torch.bfloat16, True),
    (1, 300, 2, 64, 64, 15, torch.float32, True),       # four block ends per 64 tokens
    (2, 160, 2, 32, 48, 80, torch.float32, True),
    (1, 512, 2, 64, 64, 500, torch.bfloat16, True),     # block longer than any chunk
    (2, 20, 2, 16, 16, 32, torch.float32, True),        # no full block at all
]


@pytest.mark.parametrize("B,T,H,dk,dv,block,dtype,simt", POP_CASES)
def test_pop_forward_backward(B, T, H, dk, dv, block, dtype, simt):
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s, g = make_inputs(4, B, T, H, dk, dv, dtype, scale=1.0 if dtype == torch.float32 else None)
    dO = torch.randn(B, T, H, dv, generator=g).to(dtype)
    dBS = torch.randn(B, T // block, H, dk, dv, generator=g).to(dtype)
    o, bs, grads = run_pop(q, k, v, s, decays, block, dO, dBS, simt)
    qd, kd, vd, sd = q.double(), k.double(), v.double(), s.double()
    o_ref, bs_ref = orc.pop_retention(qd, kd, vd, sd, decays, block)
    dQ, dK, dV, dS0 = orc.pop_retention_grads(qd, kd, vd, sd, decays, block, dO.double(), dBS.double(), 64)
    assert bs.shape == (B, T // block, H, dk, dv)
    check("O", o, o_ref, dtype), check("block_states", bs, bs_ref, dtype)
    check("dQ", grads[0], dQ, dtype), check("dK", grads[1], dK, dtype)
    check("dV", grads[2], dV, dtype), check("dS0", grads[3], dS0, dtype)


@pytest.mark.parametrize("name", ["pop_block15.npz", "pop_block40.npz"])
def test_pop_golden_fixture(name):
    z = np.load(os.path.join(GOLD, name))
    t = {n: torch.from_numpy(z[n]) for n in z.files}
    decays = tuple(z["decays"].tolist())
    o, bs, grads = run_pop(t["q"], t["k"], t["v"], t["s"], decays, int(z["block"]), t["dO"], t["dBS"], simt=False)
    check("O", o, t["o"], torch.float32), check("block_states", bs, t["block_states"], torch.float32)
    for got, n in zip(grads, ("dQ", "dK", "dV", "dS0")):
        check(n, got, t[n], torch.float32, rms_limit=1e-4)


@pytest.mark.parametrize("dtype,M_extra", [(torch.float32, 1), (torch.bfloat16, 0)])
def test_suffixes_start_from_block_states_and_send_gradients_back(dtype, M_extra):
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, H, dk, dv, N, P = 2, 2, 32, 32, 3, 20
    M = N + M_extra
    decays = orc.head_decays(H, (5, 12))
    g = torch.Generator().manual_seed(9)
    sc = 1.0 if dtype == torch.float32 else dk ** -0.5
    sq = (torch.randn(B, M, P, H, dk, generator=g) * sc).to(dtype)
    sk = (torch.randn(B, M, P, H, dk, generator=g) * sc).to(dtype)
    sv = (torch.randn(B, M, P, H, dv, generator=g) * sc).to(dtype)
    s0 = (torch.randn(B, H, dk, dv, generator=g) * sc).to(dtype)
    bs = (torch.randn(B, N, H, dk, dv, generator=g) * sc).to(dtype)
    dO = torch.randn(B, M, P, H, dv, generator=g).to(dtype)
    leaves = [t.cuda().requires_grad_(True) for t in (sq, sk, sv, s0, bs)]
    out = fp.pop_suffix_retention(*leaves, decays)
    (out.float() * dO.cuda().float()).sum().backward()
    _lib.device_status()
    ref_leaves = [t.double().requires_grad_(True) for t in (sq, sk, sv, s0, bs)]
    ref = orc.pop_suffix_retention(*ref_leaves, decays)
    (ref * dO.double()).sum().backward()
    check("suffix O", out, ref, dtype)
    for got, want, n in zip(leaves, ref_leaves, ("dQ", "dK", "dV", "dS0", "dBS")):
        check(n, got.grad, want.grad, dtype)
