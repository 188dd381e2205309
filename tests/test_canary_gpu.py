"""Every output of the C ABI is written inside its own bounds only: outputs are strided views in the middle of
sentinel-filled buffers (rows before and after, channels left and right), and after the call the surroundings
still hold the sentinel while the view holds the operator's result.  Ragged lengths and POP block ends on purpose:
those are the cases where whole-tile TMA stores would spill over."""
import pytest
import torch

from oracle import retention_oracle as orc

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
SENTINEL = -777.0


def _embedded(B, T, H, d):
    """A (B, T, H, d) view with 16-byte aligned strides inside a larger sentinel-filled buffer, and that buffer."""
    big = torch.full((B, T + 3, H, d + 16), SENTINEL, dtype=BF, device="cuda")
    return big[:, 1:T + 1, :, 8:8 + d], big


def _untouched_outside(view_shape, big):
    B, T, H, d = view_shape
    mask = torch.ones_like(big, dtype=torch.bool)
    mask[:, 1:T + 1, :, 8:8 + d] = False
    return bool((big[mask] == SENTINEL).all())


def _state_embedded(B, H, dk, dv):
    big = torch.full((B, H + 2, dk, dv), SENTINEL, dtype=BF, device="cuda")
    return big[:, 1:H + 1], big


@pytest.mark.parametrize("T,d,block,simt", [(70, 64, 0, False), (150, 128, 0, False), (150, 64, 40, False), (28, 64, 15, False),
                                            (300, 64, 80, False), (287, 64, 144, False),
                                            (70, 64, 0, True), (150, 64, 40, True)])
def test_outputs_stay_inside_their_views(T, d, block, simt):
    from flash_pop_b200 import _lib
    B, H = 2, 3
    decays = orc.head_decays(H, (5, 12))
    g = torch.Generator().manual_seed(T + d)
    q, k, v, dO = ((torch.randn(B, T, H, d, generator=g) * d ** -0.5).to(BF).cuda() for _ in range(4))
    s0 = (torch.randn(B, H, d, d, generator=g) * d ** -0.5).to(BF).cuda()
    flags = _lib.FLAG_FORCE_SIMT if simt else 0
    dims = _lib.dims(q, d, decays, block_size=block, flags=flags)
    stream = _lib.stream_ptr(q.device)
    L = _lib.lib()

    o, o_big = _embedded(B, T, H, d)
    if block:
        N = T // block
        bs_big = torch.full((B * N * H * d * d + 512,), SENTINEL, dtype=BF, device="cuda")
        bs = bs_big[256:256 + B * N * H * d * d]
        _lib.check(L.fpb_pop_retention_fwd(dims, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(s0), _lib.seq(o),
                                           bs.data_ptr(), stream))
    else:
        s_out, s_big = _state_embedded(B, H, d, d)
        _lib.check(L.fpb_retention_fwd(dims, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(s0), _lib.seq(o),
                                       _lib.state(s_out), stream))
    assert _lib.last_path() == (_lib.PATH_SIMT if simt else _lib.PATH_TCGEN05)
    dq, dq_big = _embedded(B, T, H, d)
    dk, dk_big = _embedded(B, T, H, d)
    dv, dv_big = _embedded(B, T, H, d)
    ds0, ds0_big = _state_embedded(B, H, d, d)
    if block:
        dbs = (torch.randn(B, N, H, d, d, generator=g) * 0.1).to(BF).cuda()
        _lib.check(L.fpb_pop_retention_bwd(dims, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(s0), _lib.seq(dO),
                                           dbs.data_ptr(), _lib.seq(dq), _lib.seq(dk), _lib.seq(dv), _lib.state(ds0), stream))
    else:
        _lib.check(L.fpb_retention_bwd(dims, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(s0), _lib.seq(dO),
                                       _lib.state(None), _lib.seq(dq), _lib.seq(dk), _lib.seq(dv), _lib.state(ds0), stream))
    _lib.device_status()

    for name, big in (("o", o_big), ("dq", dq_big), ("dk", dk_big), ("dv", dv_big)):
        assert _untouched_outside((B, T, H, d), big), f"{name}: wrote outside its view"
    for name, view, big in ((("s_out", s_out, s_big),) if not block else ()) + (("ds0", ds0, ds0_big),):
        assert bool((big[:, 0] == SENTINEL).all()) and bool((big[:, -1] == SENTINEL).all()), f"{name}: wrote outside its view"
        assert not bool((view == SENTINEL).any()), f"{name}: left unwritten"
    if block:
        assert bool((bs_big[:256] == SENTINEL).all()) and bool((bs_big[256 + bs.numel():] == SENTINEL).all())

    # and inside the views: the operator's results
    qd, kd, vd, sd = (t.double().cpu() for t in (q, k, v, s0))
    if block:
        o_ref, bs_ref = orc.pop_retention(qd, kd, vd, sd, decays, block)
        assert orc.rel_rms(bs.view(B, N, H, d, d).float().cpu(), bs_ref) < 5e-3
        grads = orc.pop_retention_grads(qd, kd, vd, sd, decays, block, dO.double().cpu(), dbs.double().cpu(), 64)
    else:
        o_ref, s_ref = orc.retention_chunkwise(qd, kd, vd, sd, decays, 64)
        assert orc.rel_rms(s_out.float().cpu(), s_ref) < 5e-3
        grads = orc.retention_grads_chunked(qd, kd, vd, sd, decays, dO.double().cpu(), None, 64)
    for name, got, ref in (("o", o, o_ref), ("dq", dq, grads[0]), ("dk", dk, grads[1]), ("dv", dv, grads[2]), ("ds0", ds0, grads[3])):
        assert orc.rel_rms(got.float().cpu(), ref) < 5e-3, name
