"""The full-size problems on the GPU: chunked retention forward at B=8, H=16, T=8192, d=128; forward+backward at that
shape (the headline benchmark) and at B=4, H=32, T=16384, dk=128, dv=256; POP with 64 blocks of 80 tokens at d=64; and the
largest shapes of the reference's own tests (T=32768, B=256, POP block 144 over T=11520:
tests/test_fused_retention.py:184-214, tests/test_pop_retention.py:199-246).  The oracle cannot run a whole problem in
seconds, so each test checks one batch row (a few heads for the largest) against the oracle and the rest through
properties: bitwise repeatability, and "a sequence fed in two segments with the carried state equals the sequence fed
at once" (the operator's streaming contract, flash_pop/retnet.py:548-558)."""
import numpy as np
import pytest
import torch

from oracle import retention_oracle as orc
from tests.util import check as _check


def check(name, got, ref, dtype):
    _check(name, got, ref, dtype, max_outside=1e-4)

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _gen(B, T, H, dk, dv, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k = ((torch.randn(B, T, H, dk, generator=g, device="cuda") * dk ** -0.5).to(BF) for _ in range(2))
    v = (torch.randn(B, T, H, dv, generator=g, device="cuda") * dk ** -0.5).to(BF)
    dO = torch.randn(B, T, H, dv, generator=g, device="cuda").to(BF)
    return q, k, v, dO


def test_config2_forward_full_size():
    """B=8, H=16, T=8192, d=128, bf16, decays 1-2^-linspace(5,12,16); row 0 against the fp64 chunkwise oracle
    (which equals the recurrent form, tests/test_oracle_golden.py)."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, T, H, d = 8, 8192, 16, 128
    decays = orc.head_decays(H, (5, 12))
    q, k, v, _ = _gen(B, T, H, d, d, 2)
    o, s = fp.fused_chunk_retention(q, k, v, None, decays)
    assert _lib.last_path() == _lib.PATH_TCGEN05
    o2, s2 = fp.fused_chunk_retention(q, k, v, None, decays)
    assert torch.equal(o, o2) and torch.equal(s, s2)
    # streaming: first half, then second half from the carried state
    oa, sa = fp.fused_chunk_retention(q[:, :4096], k[:, :4096], v[:, :4096], None, decays)
    ob, sb = fp.fused_chunk_retention(q[:, 4096:], k[:, 4096:], v[:, 4096:], sa, decays)
    _lib.device_status()
    # the carried state is rounded to bf16 between the segments, so "equal" means to bf16 accuracy
    check("two segments O", torch.cat((oa, ob), 1), o.float().cpu(), BF)
    check("two segments S", sb, s.float().cpu(), BF)
    o_ref, s_ref = orc.retention_chunkwise(q[:1].cpu().double(), k[:1].cpu().double(), v[:1].cpu().double(), None, decays, 64)
    check("O row 0", o[:1], o_ref, BF), check("S row 0", s[:1], s_ref, BF)


def test_config3_forward_backward_full_size():
    """B=4, H=32, T=16384, dk=128, dv=256: all gradients; 4 heads of row 0 against oracle autograd."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, T, H, dk, dv = 4, 16384, 32, 128, 256
    decays = orc.head_decays(H, (5, 12))
    q, k, v, dO = _gen(B, T, H, dk, dv, 3)
    leaves = [t.requires_grad_(True) for t in (q, k, v)]
    o, s = fp.fused_chunk_retention(*leaves, None, decays)
    assert _lib.last_path() == _lib.PATH_TCGEN05
    o.backward(dO)
    assert _lib.last_path() == _lib.PATH_TCGEN05
    _lib.device_status()
    for t in leaves:
        assert torch.isfinite(t.grad).all()
    hs = slice(28, 32)       # the slowest decays: the longest memory
    sub = [t[:1, :, hs].detach().cpu().double() for t in (q, k, v)]
    dec = decays[28:32]
    o_ref, s_ref = orc.retention_chunkwise(*sub, None, dec, 64)
    dQ, dK, dV, _ = orc.retention_grads_chunked(*sub, None, dec, dO[:1, :, hs].cpu().double(), None, 64)
    check("O", o[:1, :, hs], o_ref, BF), check("S", s[:1, hs], s_ref, BF)
    check("dQ", q.grad[:1, :, hs], dQ, BF), check("dK", k.grad[:1, :, hs], dK, BF), check("dV", v.grad[:1, :, hs], dV, BF)


def test_config4_pop_full_size():
    """B=16, H=8, d=64, 64 blocks of 80 observation tokens + 80 prediction tokens per block; row 0 against the oracle."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, H, d, N, blk, P = 16, 8, 64, 64, 80, 80
    T = N * blk
    decays = orc.head_decays(H, (5, 12))
    q, k, v, dO = _gen(B, T, H, d, d, 4)
    g = torch.Generator(device="cuda").manual_seed(44)
    sq, sk, sv, dS = ((torch.randn(B, N, P, H, d, generator=g, device="cuda") * (1.0 if i == 3 else d ** -0.5)).to(BF) for i in range(4))
    leaves = [t.requires_grad_(True) for t in (q, k, v, sq, sk, sv)]
    o, bs = fp.flash_pop_retention(leaves[0], leaves[1], leaves[2], None, decays, blk)
    assert _lib.last_path() == _lib.PATH_TCGEN05 and bs.shape == (B, N, H, d, d)
    so = fp.pop_suffix_retention(leaves[3], leaves[4], leaves[5], None, bs, decays)
    ((o.float() * dO.float()).sum() + (so.float() * dS.float()).sum()).backward()
    _lib.device_status()
    ref = [t[:1].detach().cpu().double().requires_grad_(True) for t in leaves]
    o_ref, bs_ref = orc.pop_retention(ref[0], ref[1], ref[2], None, decays, blk)
    so_ref = orc.pop_suffix_retention(ref[3], ref[4], ref[5], torch.zeros(1, H, d, d, dtype=torch.float64), bs_ref, decays)
    ((o_ref * dO[:1].cpu().double()).sum() + (so_ref * dS[:1].cpu().double()).sum()).backward()
    check("O", o[:1], o_ref, BF), check("block states", bs[:1], bs_ref, BF), check("suffix O", so[:1], so_ref, BF)
    for got, want, name in zip(leaves, ref, ("dQ", "dK", "dV", "dQ sfx", "dK sfx", "dV sfx")):
        check(name, got.grad[:1], want.grad, BF)


def test_headline_forward_backward_full_size():
    """B=8, H=16, T=8192, dk=dv=128, forward and backward: the benchmarked step, through the fused reverse walk and the
    dQ walk at their full length (128 chunks of carried state in fp32 registers, a bf16 copy per chunk).  Row 0, the four
    slowest-decaying heads (the longest memory), against the fp64 oracle; all gradients bitwise repeatable."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, T, H, d = 8, 8192, 16, 128
    decays = orc.head_decays(H, (5, 12))
    q, k, v, dO = _gen(B, T, H, d, d, 2)

    def run():
        leaves = [t.detach().requires_grad_(True) for t in (q, k, v)]
        n0 = _lib.launch_count()
        o, s = fp.fused_chunk_retention(*leaves, None, decays)
        assert _lib.last_path() == _lib.PATH_TCGEN05
        o.backward(dO)
        assert _lib.last_path() == _lib.PATH_TCGEN05
        assert _lib.launch_count() - n0 == 3          # forward, dQ walk, fused reverse walk: this launch fills the GPU
        return o.detach(), s.detach(), leaves[0].grad, leaves[1].grad, leaves[2].grad

    first, second = run(), run()
    _lib.device_status()
    for a, b in zip(first, second):
        assert torch.equal(a, b)
    hs = slice(12, 16)
    sub = [t[:1, :, hs].cpu().double() for t in (q, k, v)]
    dec = decays[12:16]
    o_ref, s_ref = orc.retention_chunkwise(*sub, None, dec, 64)
    dQ, dK, dV, _ = orc.retention_grads_chunked(*sub, None, dec, dO[:1, :, hs].cpu().double(), None, 64)
    o, s_out, gq, gk, gv = first
    check("O", o[:1, :, hs], o_ref, BF), check("S", s_out[:1, hs], s_ref, BF)
    check("dQ", gq[:1, :, hs], dQ, BF), check("dK", gk[:1, :, hs], dK, BF), check("dV", gv[:1, :, hs], dV, BF)


@pytest.mark.parametrize("B,T,H,dk,dv", [(1, 32768, 4, 64, 128), (256, 256, 4, 64, 64)])
def test_largest_shapes_of_the_reference_tests(B, T, H, dk, dv):
    """T=32768 at B=1 (an under-filled launch: it runs split into T-segments) and B=256 at T=256, forward and backward,
    one row against the oracle."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    decays = orc.head_decays(H, (5, 12))
    q, k, v, dO = _gen(B, T, H, dk, dv, 32)
    leaves = [t.requires_grad_(True) for t in (q, k, v)]
    o, s = fp.fused_chunk_retention(*leaves, None, decays)
    assert _lib.last_path() == _lib.PATH_TCGEN05
    o.backward(dO)
    _lib.device_status()
    row = B - 1
    sub = [t[row:row + 1].detach().cpu().double() for t in (q, k, v)]
    o_ref, s_ref = orc.retention_chunkwise(*sub, None, decays, 64)
    dQ, dK, dV, _ = orc.retention_grads_chunked(*sub, None, decays, dO[row:row + 1].cpu().double(), None, 64)
    r = slice(row, row + 1)
    check("O", o[r], o_ref, BF), check("S", s[r], s_ref, BF)
    check("dQ", q.grad[r], dQ, BF), check("dK", k.grad[r], dK, BF), check("dV", v.grad[r], dV, BF)


def test_pop_training_shape_of_the_reference_tests():
    """POP "training" case: 80 blocks of 144 tokens (T=11520), d=64, with block-state gradients; row 0 against the oracle."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, H, d, blk = 4, 4, 64, 144
    T = 80 * blk
    decays = orc.head_decays(H, (5, 12))
    q, k, v, dO = _gen(B, T, H, d, d, 144)
    g = torch.Generator(device="cuda").manual_seed(145)
    dBS = (torch.randn(B, T // blk, H, d, d, generator=g, device="cuda") * 0.1).to(BF)
    leaves = [t.requires_grad_(True) for t in (q, k, v)]
    o, bs = fp.flash_pop_retention(*leaves, None, decays, blk)
    assert _lib.last_path() == _lib.PATH_TCGEN05 and bs.shape == (B, 80, H, d, d)
    ((o.float() * dO.float()).sum() + (bs.float() * dBS.float()).sum()).backward()
    _lib.device_status()
    ref = [t[:1].detach().cpu().double().requires_grad_(True) for t in leaves]
    o_ref, bs_ref = orc.pop_retention(*ref, None, decays, blk)
    ((o_ref * dO[:1].cpu().double()).sum() + (bs_ref * dBS[:1].cpu().double()).sum()).backward()
    check("O", o[:1], o_ref, BF), check("block states", bs[:1], bs_ref, BF)
    for got, want, name in zip(leaves, ref, ("dQ", "dK", "dV")):
        check(name, got.grad[:1], want.grad, BF)
