"""The bounded waits of the tcgen05 kernels.  Every in-kernel wait (mbarrier phases, polling loops) gives up after a
limit instead of hanging; the role that gives up records (role << 8 | detail) in the device status word, raises the CTA's
abort flag, the other roles leave their loops, copies in flight are awaited, tensor memory is freed and the kernel
RETURNS.  Here the limit is shortened to about a millisecond in the diagnostics build and the TMA producer is told to
withhold the second chunk of a two-chunk sequence, so the waits on it run out: the call must come back, the status must
say DEVICE_TIMEOUT, and the next ordinary call on the same context must be correct.  Nothing traps, faults or spins
without a limit."""
import pytest
import torch

from oracle import retention_oracle as orc
from tests.util import check, make_inputs

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.mark.parametrize("d,dv,backward", [(64, 64, False), (128, 128, False), (128, 128, True), (64, 64, True),
                                          (128, 256, True)])      # dv = 256: the score warps of the dQ walk meet at named barriers
def test_wait_limit_runs_out_and_the_context_survives(d, dv, backward):
    import ctypes
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, T, H = 1, 128, 2
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s, g = make_inputs(3, B, T, H, d, dv, BF)
    dO = torch.randn(B, T, H, dv, generator=g).to(BF)
    dev = [t.cuda() for t in (q, k, v, s, dO)]

    def step():
        leaves = [t.detach().clone().requires_grad_(True) for t in dev[:4]]
        o, s_out = fp.fused_chunk_retention(*leaves, decays)
        if backward:
            o.backward(dev[4])
        return o, s_out, [t.grad for t in leaves]

    with _lib.diagnostics_build() as diag:
        try:
            # ~1 ms at 2 GHz; chunk 1 of every sequence is never loaded
            diag.fpb_debug_tuning(2_000_000, 200, 1, 1)
            step()
            detail = ctypes.c_int32(0)
            status = diag.fpb_device_status(_lib.stream_ptr(torch.device("cuda")), ctypes.byref(detail))
            assert status == 9, f"expected FPB_ERR_DEVICE_TIMEOUT, got {status}"
            role = detail.value >> 8
            assert role in (1, 2, 3, 4, 5, 6), f"status word {detail.value:#x} names no role"   # producer, MMA warp, score, state warps, 2nd / 3rd MMA warp
            # the word was cleared by the read
            assert diag.fpb_device_status(_lib.stream_ptr(torch.device("cuda")), ctypes.byref(detail)) == 0
        finally:
            diag.fpb_debug_tuning(0, 0, 1, -1)
        # same context, same library, ordinary limits: results are right again
        o, s_out, grads = step()
        _lib.device_status()
    o_ref, s_ref = orc.retention_chunkwise(q.double(), k.double(), v.double(), s.double(), decays, 64)
    check("O", o, o_ref, BF), check("S", s_out, s_ref, BF)
    if backward:
        refs = orc.retention_grads_chunked(q.double(), k.double(), v.double(), s.double(), decays, dO.double(), None, 64)
        for name, got, want in zip(("dQ", "dK", "dV", "dS0"), grads, refs):
            check(name, got, want, BF)
    # and the release build, loaded in the same process, is untouched
    o2, _, _ = step()
    _lib.device_status()
    check("O (release build)", o2, o_ref, BF)
