"""T-segments: a call whose (batch x heads x tiles) launch would leave most of the GPU idle cuts every sequence into
pieces that are walked concurrently (local end states, a scan over them, the walk per piece).  The pieces must give what
the unsplit walk gives, up to fp32 rounding of the carried state, for the forward, the dQ walk and the fused reverse
walk, for ragged lengths, start states, state gradients and POP block structure; and the same bits on every run.
The unsplit walk is the same kernel with the split switched off in the diagnostics build."""
import pytest
import torch

from oracle import retention_oracle as orc
from tests.util import check as _check, make_inputs


def check(name, got, ref, dtype):
    # sequences of thousands of tokens: 10^5-10^6 elements per tensor, and state gradients (dS0) far above 1 in magnitude
    _check(name, got, ref, dtype, max_outside=1e-4, plain=name != "dS0")

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _fwd_bwd(q, k, v, s, decays, dO, dS):
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    leaves = [None if t is None else t.detach().clone().requires_grad_(True) for t in (q, k, v, s)]
    n0 = _lib.launch_count()
    o, s_out = fp.fused_chunk_retention(*leaves, decays)
    n_fwd = _lib.launch_count() - n0
    assert _lib.last_path() == _lib.PATH_TCGEN05
    loss = (o.float() * dO.float()).sum()
    if dS is not None:
        loss = loss + (s_out.float() * dS.float()).sum()
    n0 = _lib.launch_count()
    loss.backward()
    n_bwd = _lib.launch_count() - n0
    _lib.device_status()
    return [o.detach(), s_out.detach()] + [None if t is None else t.grad for t in leaves], n_fwd, n_bwd


@pytest.mark.parametrize("B,T,H,dk,dv,state", [
    (1, 4096, 2, 128, 128, True),
    (1, 4000, 3, 128, 128, False),      # ragged: the last piece is shorter and ends inside a chunk
    (2, 2048, 2, 64, 64, True),
    (1, 3000, 2, 64, 128, True),
    (1, 2048, 2, 128, 64, False),
    (1, 4096, 2, 128, 256, True),       # dv = 256: two CTAs per head (dv halves) in the dQ walk and the fused reverse walk
])
def test_split_walks_equal_unsplit(B, T, H, dk, dv, state):
    from flash_pop_b200 import _lib
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s, g = make_inputs(T + dk, B, T, H, dk, dv, BF, state=state)
    dO = torch.randn(B, T, H, dv, generator=g).to(BF)
    dS = torch.randn(B, H, dk, dv, generator=g).to(BF) if state else None
    dev = [None if t is None else t.cuda() for t in (q, k, v, s, dO, dS)]
    with _lib.diagnostics_build() as diag:
        try:
            diag.fpb_debug_segments(0)
            whole, nf0, nb0 = _fwd_bwd(dev[0], dev[1], dev[2], dev[3], decays, dev[4], dev[5])
            diag.fpb_debug_segments(1)
            split, nf1, nb1 = _fwd_bwd(dev[0], dev[1], dev[2], dev[3], decays, dev[4], dev[5])
            again, _, _ = _fwd_bwd(dev[0], dev[1], dev[2], dev[3], decays, dev[4], dev[5])
        finally:
            diag.fpb_debug_segments(1)
    assert nf0 == 1 and nf1 == 3, "the forward was not split (1 launch unsplit, 3 split)"
    assert nb1 > nb0
    for a, b in zip(split, again):
        assert (a is None and b is None) or torch.equal(a, b), "split walks are not repeatable bit for bit"
    qd, kd, vd = q.double(), k.double(), v.double()
    sd = None if s is None else s.double()
    o_ref, s_ref = orc.retention_chunkwise(qd, kd, vd, sd, decays, 64)
    refs = [o_ref, s_ref] + list(orc.retention_grads_chunked(qd, kd, vd, sd, decays, dO.double(), None if dS is None else dS.double(), 64))
    for name, got, want, ref in zip(("O", "S", "dQ", "dK", "dV", "dS0"), split, whole, refs):
        if got is None:
            continue
        check(name, got, ref, BF)
        # against the unsplit walk: the two differ only through fp32 rounding of the carried state and bf16 copies of it
        assert orc.rel_rms(got.float().cpu(), want.float().cpu().double()) < 3e-3, name


def test_release_build_splits_under_filled_calls():
    """The shipped library, no hooks: B=1, H=4 at T=8192 runs split (3 launches forward) and matches the oracle."""
    from flash_pop_b200 import _lib
    B, T, H, d = 1, 8192, 4, 128
    decays = orc.head_decays(H, (5, 12))
    q, k, v, _, g = make_inputs(5, B, T, H, d, d, BF, state=False)
    dO = torch.randn(B, T, H, d, generator=g).to(BF)
    res, n_fwd, n_bwd = _fwd_bwd(q.cuda(), k.cuda(), v.cuda(), None, decays, dO.cuda(), None)
    assert n_fwd == 3 and n_bwd == 6
    qd, kd, vd = q.double(), k.double(), v.double()
    o_ref, s_ref = orc.retention_chunkwise(qd, kd, vd, None, decays, 64)
    dQ, dK, dV, _ = orc.retention_grads_chunked(qd, kd, vd, None, decays, dO.double(), None, 64)
    for name, got, ref in zip(("O", "S", "dQ", "dK", "dV"), res, (o_ref, s_ref, dQ, dK, dV)):
        check(name, got, ref, BF)


@pytest.mark.parametrize("T,block,d", [(5120, 80, 64), (4096, 144, 64), (3072, 96, 128)])
def test_split_pop_walks(T, block, d):
    """POP with T-segments: block states and the injected block-state gradients land in the right pieces."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, H = 1, 2
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s, g = make_inputs(T + block, B, T, H, d, d, BF)
    N = T // block
    dO = torch.randn(B, T, H, d, generator=g).to(BF)
    dBS = (torch.randn(B, N, H, d, d, generator=g) * 0.1).to(BF)
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, s)]
    n0 = _lib.launch_count()
    o, bs = fp.flash_pop_retention(*leaves, decays, block)
    assert _lib.launch_count() - n0 == 3, "the POP forward was not split"
    ((o.float() * dO.cuda().float()).sum() + (bs.float() * dBS.cuda().float()).sum()).backward()
    _lib.device_status()
    ref = [t.double().requires_grad_(True) for t in (q, k, v, s)]
    o_ref, bs_ref = orc.pop_retention(*ref, decays, block)
    ((o_ref * dO.double()).sum() + (bs_ref * dBS.double()).sum()).backward()
    check("O", o, o_ref, BF), check("block states", bs, bs_ref, BF)
    for name, got, want in zip(("dQ", "dK", "dV", "dS0"), leaves, ref):
        check(name, got.grad, want.grad, BF)


def test_workspace_is_optional_and_checked():
    """Through the C ABI: no workspace -> one launch; a misaligned workspace is refused; a small one splits less."""
    import ctypes
    from flash_pop_b200 import _lib
    B, T, H, d = 1, 4096, 2, 128
    decays = orc.head_decays(H, (5, 12))
    q, k, v, _, _ = make_inputs(9, B, T, H, d, d, BF, state=False)
    q, k, v = q.cuda(), k.cuda(), v.cuda()
    o = torch.empty_like(v)
    s_out = torch.empty(B, H, d, d, device="cuda", dtype=BF)

    def call(ws, nbytes):
        dm = _lib.dims(q, d, decays)
        dm.workspace, dm.workspace_bytes = ws, nbytes
        n0 = _lib.launch_count()
        st = _lib.lib().fpb_retention_fwd(dm, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(None), _lib.seq(o),
                                          _lib.state(s_out), _lib.stream_ptr(q.device))
        return st, _lib.launch_count() - n0

    assert call(None, 0) == (0, 1)
    whole = o.clone()
    need = _lib.lib().fpb_workspace_bytes(ctypes.byref(_lib.dims(q, d, decays)))
    assert need > 0
    buf = torch.empty(need + 64, dtype=torch.uint8, device="cuda")
    assert call(buf.data_ptr() + 4, need)[0] == 12          # FPB_ERR_BAD_WORKSPACE
    assert call(buf.data_ptr(), need) == (0, 3)
    assert orc.rel_rms(o.float().cpu(), whole.float().cpu().double()) < 3e-3
    two = 2 * B * H * d * d * 4                             # room for two pieces per sequence
    assert call(buf.data_ptr(), two) == (0, 3)
    assert call(buf.data_ptr(), two - 16) == (0, 1)          # not even two pieces fit: walked whole
    _lib.device_status()
