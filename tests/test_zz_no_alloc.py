"""fpb_retention_fwd_static: the forward entry point for callers that may not allocate device memory (a host that gave
the whole GPU to one arena at start-up, a plugin forbidden to allocate on the hot path).  Its T-segment scratch is an
array inside the library image instead of caller memory.  Called through the C ABI on an under-filled shape - so that
the scratch really is used - it must give what fpb_retention_fwd gives with caller-provided scratch, on two calls in a
row (the array keeps the first call's contents when the second starts), must allocate nothing, and must refuse a shape
that would need more scratch than the array holds.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes

import pytest
import torch

from oracle import retention_oracle as orc
from tests.util import check, make_inputs

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _call(fn, dims, q, k, v, s0, o, s_out):
    from flash_pop_b200 import _lib
    return fn(dims, _lib.seq(q), _lib.seq(k), _lib.seq(v), _lib.state(s0), _lib.seq(o), _lib.state(s_out),
              _lib.stream_ptr(q.device))


def test_static_scratch_entry_point_matches_the_allocating_one():
    from flash_pop_b200 import _lib
    lib = _lib.lib()
    B, T, H, d = 1, 4096, 4, 128
    decays = orc.head_decays(H, (5, 12))
    outs = []
    for seed in (11, 12):                      # two calls in a row, different data: the second finds the first one's scratch
        q, k, v, s0, _ = make_inputs(seed, B, T, H, d, d, BF)
        q, k, v, s0 = (t.cuda() for t in (q, k, v, s0))
        # existing entry point, scratch from the caller
        dm = _lib.dims(q, d, decays, workspace=True)
        assert dm.workspace_bytes > 0, "this shape is meant to be split"
        o_ref, s_ref = torch.empty_like(v), torch.empty(B, H, d, d, device="cuda", dtype=BF)
        n0 = _lib.launch_count()
        _lib.check(_call(lib.fpb_retention_fwd, dm, q, k, v, s0, o_ref, s_ref))
        assert _lib.launch_count() - n0 == 3
        # the entry point under test: outputs allocated BEFORE the memory counters are read, nothing after
        o, s_out = torch.empty_like(v), torch.empty(B, H, d, d, device="cuda", dtype=BF)
        dm2 = _lib.dims(q, d, decays)
        torch.cuda.synchronize()
        free0, _ = torch.cuda.mem_get_info()
        n0 = _lib.launch_count()
        _lib.check(_call(lib.fpb_retention_fwd_static, dm2, q, k, v, s0, o, s_out))
        assert _lib.launch_count() - n0 == 3, "the call did not use its scratch (it ran unsplit)"
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info()
        if outs:                               # (the very first call may load the kernels' code: compare from the second on)
            assert free1 == free0, "device memory changed hands during the call"
        _lib.device_status()
        # same pieces, same arithmetic: the two entry points agree within the tolerance of the parity tests (in fact bit for bit)
        check("O", o, o_ref.float().cpu(), BF), check("S", s_out, s_ref.float().cpu(), BF)
        assert torch.equal(o, o_ref) and torch.equal(s_out, s_ref)
        o_orc, s_orc = orc.retention_chunkwise(q.cpu().double(), k.cpu().double(), v.cpu().double(), s0.cpu().double(), decays, 64)
        check("O vs oracle", o, o_orc, BF, max_outside=1e-4), check("S vs oracle", s_out, s_orc, BF, max_outside=1e-4)
        outs.append(o)
    assert not torch.equal(outs[0], outs[1])


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from flash_pop_b200 import _lib
    lib = _lib.lib()
    H = 8
    decays = orc.head_decays(H, (5, 12))
    # 8 heads of 128 x 256 states over 16384 tokens would be cut into 18 pieces each: 8 x 18 x 128 KB of scratch
    B, T, dk, dv = 1, 16384, 128, 256
    q = torch.zeros(B, T, H, dk, device="cuda", dtype=BF)
    v = torch.zeros(B, T, H, dv, device="cuda", dtype=BF)
    o, s_out = torch.empty_like(v), torch.empty(B, H, dk, dv, device="cuda", dtype=BF)
    dm = _lib.dims(q, dv, decays)
    need = lib.fpb_workspace_bytes(ctypes.byref(dm))
    assert need > _lib.STATIC_SCRATCH_BYTES
    assert _call(lib.fpb_retention_fwd_static, dm, q, q, v, None, o, s_out) == 11            # FPB_ERR_TOO_LARGE
    assert b"scratch" in lib.fpb_strerror(11)
    # a caller-provided workspace has no place here
    buf = torch.empty(1024, dtype=torch.uint8, device="cuda")
    dm.workspace, dm.workspace_bytes = buf.data_ptr(), 1024
    assert _call(lib.fpb_retention_fwd_static, dm, q, q, v, None, o, s_out) == 12            # FPB_ERR_BAD_WORKSPACE
    # a shape that fills the GPU unsplit needs no scratch and goes through
    B, d = 32, 128
    q = torch.zeros(B, 256, H, d, device="cuda", dtype=BF)
    o, s_out = torch.empty_like(q), torch.empty(B, H, d, d, device="cuda", dtype=BF)
    assert _call(lib.fpb_retention_fwd_static, _lib.dims(q, d, decays), q, q, q, None, o, s_out) == 0
    _lib.device_status()
