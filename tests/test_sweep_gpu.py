"""Sweeps over sequence lengths and POP block sizes on small shapes: every T from 1 to 3 chunks (tails, exact
multiples, single tokens) and block sizes around every chunk/block alignment case, forward and backward, on the
tensor-core kernels, each against the fp64 oracle (relative RMS, the reference's own criterion)."""
import pytest
import torch

from oracle import retention_oracle as orc

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
LIMIT = 5e-3      # the reference's own criterion (tests/test_fused_retention.py:119,131); the worst case measured is 3.4e-3 (dK at T=13, d=64)


def _inputs(T, d, seed):
    g = torch.Generator().manual_seed(seed)
    q, k, v = ((torch.randn(1, T, 2, d, generator=g) * d ** -0.5).to(BF) for _ in range(3))
    s = (torch.randn(1, 2, d, d, generator=g) * d ** -0.5).to(BF)
    dO = torch.randn(1, T, 2, d, generator=g).to(BF)
    return q, k, v, s, dO


def _rr(name, got, ref):
    if ref.numel() == 0:
        return
    r = orc.rel_rms(got.detach().float().cpu(), ref)
    assert r < LIMIT, f"{name}: rel-RMS {r:.3e}"


@pytest.mark.parametrize("d", [64, 128])
def test_every_length_up_to_three_chunks(d):
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    decays = orc.head_decays(2, (5, 12))
    for T in range(1, 193):
        q, k, v, s, dO = _inputs(T, d, T)
        leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, s)]
        o, s_out = fp.fused_chunk_retention(*leaves, decays)
        assert _lib.last_path() == _lib.PATH_TCGEN05
        (o.float() * dO.cuda().float()).sum().backward()
        qd, kd, vd, sd = (t.double() for t in (q, k, v, s))
        o_ref, s_ref = orc.retention_chunkwise(qd, kd, vd, sd, decays, 64)
        dQ, dK, dV, dS0 = orc.retention_grads_chunked(qd, kd, vd, sd, decays, dO.double(), None, 64)
        for name, got, ref in (("O", o, o_ref), ("S", s_out, s_ref), ("dQ", leaves[0].grad, dQ), ("dK", leaves[1].grad, dK),
                               ("dV", leaves[2].grad, dV), ("dS0", leaves[3].grad, dS0)):
            _rr(f"T={T} {name}", got, ref)
    _lib.device_status()


def test_block_sizes_around_every_alignment_case():
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    d, T = 64, 150
    # 80, 96, 112, 144: multiples of 16 above 64 - the forward walk keeps full chunks and emits those block states from
    # partial state increments
    decays = orc.head_decays(2, (5, 12))
    for block in (1, 2, 3, 7, 15, 16, 17, 31, 32, 33, 50, 63, 64, 65, 75, 80, 96, 100, 112, 127, 128, 129, 144, 149, 150, 151):
        q, k, v, s, dO = _inputs(T, d, block)
        g = torch.Generator().manual_seed(1000 + block)
        dBS = torch.randn(1, T // block, 2, d, d, generator=g).to(BF)
        leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, s)]
        o, bs = fp.flash_pop_retention(*leaves, decays, block)
        assert _lib.last_path() == _lib.PATH_TCGEN05 and bs.shape[1] == T // block
        loss = (o.float() * dO.cuda().float()).sum()
        if bs.numel():
            loss = loss + (bs.float() * dBS.cuda().float()).sum()
        loss.backward()
        qd, kd, vd, sd = (t.double() for t in (q, k, v, s))
        o_ref, bs_ref = orc.pop_retention(qd, kd, vd, sd, decays, block)
        dQ, dK, dV, dS0 = orc.pop_retention_grads(qd, kd, vd, sd, decays, block, dO.double(), dBS.double(), 64)
        for name, got, ref in (("O", o, o_ref), ("block states", bs, bs_ref), ("dQ", leaves[0].grad, dQ),
                               ("dK", leaves[1].grad, dK), ("dV", leaves[2].grad, dV), ("dS0", leaves[3].grad, dS0)):
            _rr(f"block={block} {name}", got, ref)
    _lib.device_status()
