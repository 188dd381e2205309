"""The CPU oracle against fixtures produced by the reference's own PyTorch functions
(tests/golden/make_golden.py).  This is what pins the oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import retention_oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    z = np.load(os.path.join(GOLD, name))
    out = {k: torch.from_numpy(z[k]) for k in z.files}
    out["decays"] = tuple(z["decays"].tolist())
    return out


def close(a, b, tol):
    assert a.shape == b.shape
    err = (a.double() - b.double()).abs().max().item()
    scale = b.double().abs().max().item() + 1e-12
    assert err <= tol * scale, f"max err {err:.3e} vs scale {scale:.3e}"


def test_decays_match_reference_formula():
    d = orc.head_decays(4)
    assert d == tuple(1 - 2.0 ** (-5 - h) for h in range(4))
    d = orc.head_decays(8, (5, 12))
    assert abs(d[0] - (1 - 2 ** -5)) < 1e-15 and abs(d[-1] - (1 - 2 ** -12)) < 1e-15


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.float64, 2e-5)])
def test_forward_forms(dtype, tol):
    g = load("fwd_ragged.npz")
    q, k, v, s = (g[n].to(dtype) for n in "qkvs")
    o, st = orc.retention_chunkwise(q, k, v, s, g["decays"], chunk_size=32)
    close(o, g["o_chunk32"], tol), close(st, g["s_chunk32"], tol)
    o, st = orc.retention_parallel(q, k, v, s, g["decays"])
    close(o, g["o_parallel"], tol), close(st, g["s_parallel"], tol)
    o, st = orc.retention_recurrent(q, k, v, s, g["decays"])
    close(o, g["o_recurrent"], 2e-5), close(st, g["s_recurrent"], 2e-5)
    # chunk-size invariance (tests/test_fused_retention.py:217-237 in the reference)
    o7, s7 = orc.retention_chunkwise(q, k, v, s, g["decays"], chunk_size=7)
    close(o7, g["o_parallel"], 5e-5), close(s7, g["s_parallel"], 5e-5)


def test_closed_form_grads():
    g = load("grads.npz")
    q, k, v, s = (g[n] for n in "qkvs")
    dQ, dK, dV, dS0 = orc.retention_grads(q, k, v, s, g["decays"], g["dO"], g["dS"])
    for mine, name in ((dQ, "dQ"), (dK, "dK"), (dV, "dV"), (dS0, "dS0")):
        close(mine, g[name], 5e-6)
        close(mine, g[name + "_autograd"], 1e-4)
    dQ, dK, dV, dS0 = orc.retention_grads_chunked(q, k, v, s, g["decays"], g["dO"], g["dS"], chunk_size=16)
    for mine, name in ((dQ, "dQ"), (dK, "dK"), (dV, "dV"), (dS0, "dS0")):
        close(mine, g[name + "_autograd"], 1e-4)
    o, st = orc.retention_chunkwise(q, k, v, s, g["decays"], chunk_size=16)
    close(o, g["o"], 2e-6), close(st, g["s_out"], 2e-6)


@pytest.mark.parametrize("name", ["pop_block15.npz", "pop_block40.npz"])
def test_pop_forward_and_grads(name):
    g = load(name)
    q, k, v, s = (g[n] for n in "qkvs")
    block = int(g["block"])
    o, bs = orc.pop_retention(q, k, v, s, g["decays"], block)
    close(o, g["o"], 2e-6), close(bs, g["block_states"], 2e-6)
    assert bs.shape[1] == q.shape[1] // block
    for chunk in (64, 16):
        dQ, dK, dV, dS0 = orc.pop_retention_grads(q, k, v, s, g["decays"], block, g["dO"], g["dBS"], chunk)
        close(dQ, g["dQ"], 1e-4), close(dK, g["dK"], 1e-4), close(dV, g["dV"], 1e-4), close(dS0, g["dS0"], 1e-4)


def test_pop_suffix_matches_plain_retention_from_block_start_states():
    g = load("pop_block15.npz")
    q, k, v, s = (g[n] for n in "qkvs")
    block = int(g["block"])
    _, bs = orc.pop_retention(q, k, v, s, g["decays"], block)
    B, N = bs.shape[:2]
    gen = torch.Generator().manual_seed(3)
    P = 9
    sq = torch.randn(B, N + 1, P, q.shape[2], q.shape[3], generator=gen)
    sk = torch.randn(B, N + 1, P, q.shape[2], q.shape[3], generator=gen)
    sv = torch.randn(B, N + 1, P, q.shape[2], v.shape[3], generator=gen)
    out = orc.pop_suffix_retention(sq, sk, sv, s, bs, g["decays"])
    for n in range(N + 1):
        start = s if n == 0 else bs[:, n - 1]
        ref, _ = orc.retention_recurrent(sq[:, n], sk[:, n], sv[:, n], start, g["decays"])
        close(out[:, n], ref, 5e-5)


def test_chunk_schedule_cuts_at_block_ends():
    assert orc.chunk_schedule(200, 80, 64) == [(0, 64), (64, 80), (80, 144), (144, 160), (160, 200)]
    assert orc.chunk_schedule(130, 1000, 64) == [(0, 64), (64, 128), (128, 130)]
    assert orc.chunk_schedule(30, 15, 64) == [(0, 15), (15, 30)]
