"""dk = 128 next to dv = 256 (twice the key width, the reference's usual value width): the gradient walks cut dv into two
128-wide halves - two CTAs per head on the 128 x 128 kernels - and the halves' partial results for dQ and dK are added
to the zeroed outputs by TMA.  Checked here: parity with the oracle through the C ABI with every output a strided view
inside a sentinel-filled buffer (the zero fill and the adds must stay inside the view), against the dk-tiled walks the
diagnostics build can switch back to, launch counts, and bitwise repeatability (two addends per element: their order
cannot matter)."""
import pytest
import torch

from oracle import retention_oracle as orc
from tests.util import check, make_inputs

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
SENTINEL = -777.0


def _embedded(B, T, H, d):
    big = torch.full((B, T + 3, H, d + 16), SENTINEL, dtype=BF, device="cuda")
    return big[:, 1:T + 1, :, 8:8 + d], big


def _clean_outside(view_shape, big):
    B, T, H, d = view_shape
    mask = torch.ones_like(big, dtype=torch.bool)
    mask[:, 1:T + 1, :, 8:8 + d] = False
    return bool((big[mask] == SENTINEL).all())


def _backward(_lib, dims, q, k, v, s0, dO, dS, stream):
    L = _lib.lib()
    B, T, H, dk = q.shape
    dv = v.shape[-1]
    outs = {"dq": _embedded(B, T, H, dk), "dk": _embedded(B, T, H, dk), "dv": _embedded(B, T, H, dv)}
    ds0 = torch.empty(B, H, dk, dv, dtype=BF, device="cuda")
    n0 = _lib.launch_count()
    _lib.check(L.fpb_retention_bwd(dims, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(s0), _lib.seq(dO), _lib.state(dS),
                                   _lib.seq(outs["dq"][0]), _lib.seq(outs["dk"][0]), _lib.seq(outs["dv"][0]), _lib.state(ds0), stream))
    n = _lib.launch_count() - n0
    _lib.device_status()
    assert _lib.last_path() == _lib.PATH_TCGEN05
    return outs, ds0, n


@pytest.mark.parametrize("B,T,H", [(2, 257, 2), (1, 1000, 3), (1, 64, 1)])
def test_dv256_gradients_in_strided_views(B, T, H):
    from flash_pop_b200 import _lib
    dk, dv = 128, 256
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s, g = make_inputs(T, B, T, H, dk, dv, BF, state=True)
    dO = torch.randn(B, T, H, dv, generator=g).to(BF)
    dS = (torch.randn(B, H, dk, dv, generator=g) * 0.1).to(BF)
    qc, kc, vc, sc, dOc, dSc = (t.cuda() for t in (q, k, v, s, dO, dS))
    dims = _lib.dims(qc, dv, decays)
    stream = _lib.stream_ptr(qc.device)
    with _lib.diagnostics_build() as diag:
        try:
            diag.fpb_debug_col_split(0)
            old, ds0_old, n_old = _backward(_lib, dims, qc, kc, vc, sc, dOc, dSc, stream)
        finally:
            diag.fpb_debug_col_split(1)
        new, ds0_new, n_new = _backward(_lib, dims, qc, kc, vc, sc, dOc, dSc, stream)
        again, ds0_again, _ = _backward(_lib, dims, qc, kc, vc, sc, dOc, dSc, stream)
    # dk-tiled: dQ walk, dV walk, dK walk.  dv halves: (zero fill + dQ walk) + (zero fill + fused reverse walk)
    assert n_old == 3 and n_new == 4
    refs = orc.retention_grads_chunked(q.double(), k.double(), v.double(), s.double(), decays, dO.double(), dS.double(), 64)
    for name, ref in zip(("dq", "dk", "dv"), refs):
        view, big = new[name]
        assert _clean_outside(view.shape, big), f"{name}: wrote outside its view"
        assert torch.equal(view, again[name][0]), f"{name}: not repeatable bit for bit"
        check(name, view, ref, BF, max_outside=1e-4)
        check(name + " (dk-tiled walks)", old[name][0], ref, BF, max_outside=1e-4)
    assert torch.equal(ds0_new, ds0_again)
    check("dS0", ds0_new, refs[3], BF, max_outside=1e-4, plain=False)
    # the halves' dV and dS_0 are complete results: they equal the separate reverse walk's bit for bit
    assert torch.equal(new["dv"][0], old["dv"][0]) and torch.equal(ds0_new, ds0_old)
