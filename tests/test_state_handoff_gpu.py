"""Carrying the state across calls (a long sequence fed in pieces, flash_pop/retnet.py:548-558): with fp32 states under
bf16 activations the hand-off adds no rounding, so eight pieces give the state of one call to fp32 accuracy; and the POP
generation scenario (one block and a suffix, tests/test_pop_retention.py:161-196) through fp32 block states."""
import pytest
import torch

from oracle import retention_oracle as orc
from tests.util import check as _check, make_inputs


def check(name, got, ref, dtype):
    _check(name, got, ref, dtype, max_outside=1e-4, plain=name != "dS0")

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.mark.parametrize("d", [64, 128])
def test_eight_pieces_with_fp32_state_equal_one_call(d):
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, T, H, P = 2, 8192, 4, 8
    decays = orc.head_decays(H, (5, 12))
    q, k, v, _, _ = make_inputs(31 + d, B, T, H, d, d, BF, state=False)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    o1, s1 = fp.fused_chunk_retention(qc, kc, vc, None, decays, torch.float32)
    assert s1.dtype == torch.float32 and _lib.last_path() == _lib.PATH_TCGEN05

    def pieces(state_dtype):
        s, outs = None, []
        for i in range(P):
            sl = slice(i * T // P, (i + 1) * T // P)
            o, s = fp.fused_chunk_retention(qc[:, sl], kc[:, sl], vc[:, sl], s, decays, state_dtype)
            assert s.dtype == state_dtype
            outs.append(o)
        return torch.cat(outs, 1), s

    o32, s32 = pieces(torch.float32)
    o16, s16 = pieces(BF)
    _lib.device_status()
    o_ref, s_ref = orc.retention_chunkwise(q.double(), k.double(), v.double(), None, decays, 64)
    check("O, fp32 hand-off", o32, o_ref, BF)
    # the fp32 hand-off loses nothing: the state crosses the calls as it sits in the registers of a single call; what is
    # left is the order of the fp32 additions (the calls cut their sequences into different T-segments) and, from that,
    # a bf16 output here and there that rounds the other way
    assert orc.rel_rms(s32.cpu(), s1.cpu().double()) < 1e-5
    assert orc.rel_rms(o32.float().cpu(), o1.float().cpu().double()) < 5e-4
    # the bf16 hand-off rounds the state eight times on the way: further from the single call, still within tolerance
    d16 = orc.rel_rms(s16.float().cpu(), s1.cpu().double())
    assert 1e-4 < d16 < 5e-3, d16
    e32, e16 = orc.rel_rms(s32.cpu(), s_ref), orc.rel_rms(s16.float().cpu(), s_ref)
    assert e32 < 5e-3 and e16 < 5e-3, (e32, e16)


def test_fp32_state_gradients():
    """fp32 s0 / s_out / dS through the backward (tensor-core and CUDA-core kernels) against the oracle."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    from flash_pop_b200.fused_retention import cuda_core_kernels
    B, T, H, dk, dv = 2, 300, 3, 128, 128
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s, g = make_inputs(77, B, T, H, dk, dv, BF)
    s = s.float() + torch.randn(s.shape, generator=g) * 1e-3      # not representable in bf16
    dO = torch.randn(B, T, H, dv, generator=g).to(BF)
    dS = torch.randn(B, H, dk, dv, generator=g)
    qd, kd, vd, sd = q.double(), k.double(), v.double(), s.double()
    o_ref, s_ref = orc.retention_chunkwise(qd, kd, vd, sd, decays, 64)
    refs = [o_ref, s_ref] + list(orc.retention_grads_chunked(qd, kd, vd, sd, decays, dO.double(), dS.double(), 64))
    for simt in (False, True):
        leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, s)]
        if simt:
            with cuda_core_kernels():
                o, s_out = fp.fused_chunk_retention(*leaves, decays)
                ((o.float() * dO.cuda().float()).sum() + (s_out * dS.cuda()).sum()).backward()
            assert _lib.last_path() == _lib.PATH_SIMT
        else:
            o, s_out = fp.fused_chunk_retention(*leaves, decays)
            ((o.float() * dO.cuda().float()).sum() + (s_out * dS.cuda()).sum()).backward()
            assert _lib.last_path() == _lib.PATH_TCGEN05
        _lib.device_status()
        assert s_out.dtype == torch.float32 and leaves[3].grad.dtype == torch.float32
        got = [o, s_out] + [t.grad for t in leaves]
        for name, a, r in zip(("O", "S", "dQ", "dK", "dV", "dS0"), got, refs):
            check(name, a, r, BF)
        # an fp32 state is not rounded on the way out
        assert orc.rel_rms(s_out.cpu(), s_ref) < 1e-3


def test_pop_generation_with_fp32_block_states():
    """One block of observations plus its suffix in one sequence (T=287, block 144): block state in fp32 feeds the
    suffix call in place; outputs and all gradients against the oracle."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, T, H, d, block, P = 2, 287, 4, 64, 144, 143
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s, g = make_inputs(287, B, T, H, d, d, BF)
    sq, sk, sv = ((torch.randn(B, 2, P, H, d, generator=g) * d ** -0.5).to(BF) for _ in range(3))
    dO = torch.randn(B, T, H, d, generator=g).to(BF)
    dSO = torch.randn(B, 2, P, H, d, generator=g).to(BF)
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, s, sq, sk, sv)]
    o, bs = fp.flash_pop_retention(leaves[0], leaves[1], leaves[2], leaves[3], decays, block, torch.float32)
    assert bs.dtype == torch.float32 and bs.shape == (B, 1, H, d, d)
    so = fp.pop_suffix_retention(leaves[4], leaves[5], leaves[6], leaves[3], bs, decays)
    ((o.float() * dO.cuda().float()).sum() + (so.float() * dSO.cuda().float()).sum()).backward()
    _lib.device_status()
    ref = [t.double().requires_grad_(True) for t in (q, k, v, s, sq, sk, sv)]
    o_ref, bs_ref = orc.pop_retention(ref[0], ref[1], ref[2], ref[3], decays, block)
    so_ref = orc.pop_suffix_retention(ref[4], ref[5], ref[6], ref[3], bs_ref, decays)
    ((o_ref * dO.double()).sum() + (so_ref * dSO.double()).sum()).backward()
    check("O", o, o_ref, BF), check("suffix O", so, so_ref, BF)
    assert orc.rel_rms(bs.cpu(), bs_ref) < 1e-3
    for name, got, want in zip(("dQ", "dK", "dV", "dS0", "dQ sfx", "dK sfx", "dV sfx"), leaves, ref):
        check(name, got.grad, want.grad, BF)
