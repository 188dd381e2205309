"""Parity of the tcgen05 (tensor-core) kernels with the CPU oracle, on the shapes they serve:
dk in {64,128}, dv in {64,128,256}, bf16, any T (tails, T < one chunk), with and without a start state,
POP block ends inside / across chunks, suffix starts.  Every case asserts that the tensor-core path
really ran."""
import pytest
import torch

from oracle import retention_oracle as orc
from tests.util import check, make_inputs

pytestmark = pytest.mark.gpu
BF = torch.bfloat16

FWD_BWD_CASES = [
    # B, T, H, dk, dv, state, dS, scale
    (2, 200, 4, 64, 64, True, True, None),
    (1, 64, 2, 128, 128, False, False, None),
    (2, 333, 3, 128, 128, True, True, None),
    (1, 130, 2, 64, 128, True, False, None),
    (1, 100, 2, 128, 64, True, True, None),
    (2, 257, 2, 128, 256, True, True, None),
    (1, 150, 2, 64, 256, False, True, None),
    (3, 17, 2, 64, 64, True, True, None),        # shorter than one chunk
    (2, 1, 2, 128, 128, True, True, None),       # single token
    (1, 1024, 2, 128, 128, True, True, 1.0),     # unit-variance inputs (the reference tests' law)
]


def _run(q, k, v, s, decays, dO, dS):
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    leaves = [None if t is None else t.cuda().requires_grad_(True) for t in (q, k, v, s)]
    o, s_out = fp.fused_chunk_retention(*leaves, decays)
    path_f = _lib.last_path()
    loss = (o.float() * dO.cuda().float()).sum()
    if dS is not None:
        loss = loss + (s_out.float() * dS.cuda().float()).sum()
    loss.backward()
    path_b = _lib.last_path()
    _lib.device_status()
    return o, s_out, [None if t is None else t.grad for t in leaves], path_f, path_b


@pytest.mark.parametrize("B,T,H,dk,dv,state,with_dS,scale", FWD_BWD_CASES)
def test_retention_forward_backward(B, T, H, dk, dv, state, with_dS, scale):
    from flash_pop_b200 import _lib
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s, g = make_inputs(21, B, T, H, dk, dv, BF, scale=scale, state=state)
    dO = torch.randn(B, T, H, dv, generator=g).to(BF)
    dS = torch.randn(B, H, dk, dv, generator=g).to(BF) if with_dS else None
    o, s_out, grads, path_f, path_b = _run(q, k, v, s, decays, dO, dS)
    assert path_f == _lib.PATH_TCGEN05 and path_b == _lib.PATH_TCGEN05
    qd, kd, vd = q.double(), k.double(), v.double()
    sd = None if s is None else s.double()
    o_ref, s_ref = orc.retention_chunkwise(qd, kd, vd, sd, decays, 64)
    dQ, dK, dV, dS0 = orc.retention_grads_chunked(qd, kd, vd, sd, decays, dO.double(), None if dS is None else dS.double(), 64)
    if scale == 1.0:
        # unit-variance data: the elementwise 2e-2 bound is unattainable with bf16 operands (large
        # cancelling sums); the reference's own criterion is relative RMS < 0.005
        for name, got, ref in (("O", o, o_ref), ("S", s_out, s_ref), ("dQ", grads[0], dQ), ("dK", grads[1], dK), ("dV", grads[2], dV)):
            rr = orc.rel_rms(got.detach().float().cpu(), ref)
            assert rr < 5e-3, f"{name}: rel-RMS {rr:.3e}"
        return
    check("O", o, o_ref, BF), check("S", s_out, s_ref, BF)
    check("dQ", grads[0], dQ, BF), check("dK", grads[1], dK, BF), check("dV", grads[2], dV, BF)
    if state:
        check("dS0", grads[3], dS0, BF)


def test_default_decays_config():
    """gamma_h = 1 - 2^(-5-h): the strongest decay the layers use by default."""
    from flash_pop_b200 import _lib
    B, T, H, d = 2, 192, 4, 64
    decays = orc.head_decays(H)
    q, k, v, s, g = make_inputs(3, B, T, H, d, d, BF)
    dO = torch.randn(B, T, H, d, generator=g).to(BF)
    o, s_out, grads, pf, pb = _run(q, k, v, s, decays, dO, None)
    assert pf == _lib.PATH_TCGEN05
    o_ref, s_ref = orc.retention_chunkwise(q.double(), k.double(), v.double(), s.double(), decays, 64)
    check("O", o, o_ref, BF), check("S", s_out, s_ref, BF)


def test_runs_are_bitwise_repeatable():
    import flash_pop_b200 as fp
    B, T, H, d = 2, 300, 4, 128
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s, _ = make_inputs(8, B, T, H, d, d, BF)
    args = [t.cuda() for t in (q, k, v, s)]
    o1, s1 = fp.fused_chunk_retention(*args, decays)
    o2, s2 = fp.fused_chunk_retention(*args, decays)
    assert torch.equal(o1, o2) and torch.equal(s1, s2)


POP_CASES = [
    # B, T, H, dk, dv, block
    (2, 400, 2, 64, 64, 80),      # the configured POP layout: block 80 against 64-token chunks
    (2, 287, 2, 64, 128, 144),    # one full block + tail ("generation")
    (1, 300, 2, 64, 64, 15),      # four block ends per 64 tokens
    (1, 512, 2, 128, 128, 500),   # block longer than any chunk
    (2, 28, 2, 64, 128, 15),
    (1, 128, 2, 128, 128, 64),    # block == chunk
]


@pytest.mark.parametrize("B,T,H,dk,dv,block", POP_CASES)
def test_pop_forward_backward(B, T, H, dk, dv, block):
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s, g = make_inputs(4, B, T, H, dk, dv, BF)
    dO = torch.randn(B, T, H, dv, generator=g).to(BF)
    dBS = torch.randn(B, T // block, H, dk, dv, generator=g).to(BF)
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, s)]
    o, bs = fp.flash_pop_retention(*leaves, decays, block)
    assert _lib.last_path() == _lib.PATH_TCGEN05
    ((o.float() * dO.cuda().float()).sum() + (bs.float() * dBS.cuda().float()).sum()).backward()
    assert _lib.last_path() == _lib.PATH_TCGEN05
    _lib.device_status()
    qd, kd, vd, sd = q.double(), k.double(), v.double(), s.double()
    o_ref, bs_ref = orc.pop_retention(qd, kd, vd, sd, decays, block)
    dQ, dK, dV, dS0 = orc.pop_retention_grads(qd, kd, vd, sd, decays, block, dO.double(), dBS.double(), 64)
    check("O", o, o_ref, BF), check("block_states", bs, bs_ref, BF)
    check("dQ", leaves[0].grad, dQ, BF), check("dK", leaves[1].grad, dK, BF)
    check("dV", leaves[2].grad, dV, BF), check("dS0", leaves[3].grad, dS0, BF)


def test_suffixes_on_tensor_cores():
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, H, dk, dv, N, P = 2, 2, 64, 64, 4, 80
    M = N            # one suffix per block, the configured layout
    decays = orc.head_decays(H, (5, 12))
    g = torch.Generator().manual_seed(9)
    sc = dk ** -0.5
    sq, sk = ((torch.randn(B, M, P, H, dk, generator=g) * sc).to(BF) for _ in range(2))
    sv = (torch.randn(B, M, P, H, dv, generator=g) * sc).to(BF)
    s0 = (torch.randn(B, H, dk, dv, generator=g) * sc).to(BF)
    bs = (torch.randn(B, N, H, dk, dv, generator=g) * sc).to(BF)
    dO = torch.randn(B, M, P, H, dv, generator=g).to(BF)
    leaves = [t.cuda().requires_grad_(True) for t in (sq, sk, sv, s0, bs)]
    out = fp.pop_suffix_retention(*leaves, decays)
    assert _lib.last_path() == _lib.PATH_TCGEN05
    (out.float() * dO.cuda().float()).sum().backward()
    _lib.device_status()
    ref_leaves = [t.double().requires_grad_(True) for t in (sq, sk, sv, s0, bs)]
    ref = orc.pop_suffix_retention(*ref_leaves, decays)
    (ref * dO.double()).sum().backward()
    check("suffix O", out, ref, BF)
    for got, want, n in zip(leaves, ref_leaves, ("dQ", "dK", "dV", "dS0", "dBS")):
        check(n, got.grad, want.grad, BF)


def test_backward_runs_only_the_walks_that_are_needed():
    """dQ alone is one launch, dK/dV alone the other; results equal those of the full backward."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, T, H, d = 2, 200, 2, 128
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s, g = make_inputs(5, B, T, H, d, d, BF)
    dO = torch.randn(B, T, H, d, generator=g).to(BF).cuda()
    full = [t.cuda().requires_grad_(True) for t in (q, k, v)]
    o, _ = fp.fused_chunk_retention(*full, s.cuda(), decays)
    o.backward(dO)
    for wanted in ((0,), (1, 2), (2,)):
        leaves = [t.cuda().requires_grad_(i in wanted) for i, t in enumerate((q, k, v))]
        o, _ = fp.fused_chunk_retention(*leaves, s.cuda(), decays)
        before = _lib.launch_count()
        o.backward(dO)
        assert _lib.launch_count() - before == 1
        for i in range(3):
            if i in wanted:
                assert torch.equal(leaves[i].grad, full[i].grad)
            else:
                assert leaves[i].grad is None
    _lib.device_status()


@pytest.mark.parametrize("B,H,dk,dv,slices,head_groups", [(4, 2, 128, 128, 3, 1), (4, 2, 128, 128, 3, None), (3, 8, 64, 128, None, 4),
                                                          (2, 6, 128, 128, None, 3)])
def test_host_memory_pipeline_equals_direct_call(B, H, dk, dv, slices, head_groups):
    """Slices (batch rows x head groups) copied in / computed / copied out on three streams give the results of one
    direct call, bit for bit; a head group crosses as one two-dimensional copy and must touch nothing beside it."""
    import flash_pop_b200 as fp
    from flash_pop_b200.host_io import HostRetentionPipeline
    T = 300
    decays = orc.head_decays(H, (5, 12))
    q, k, v, _, g = make_inputs(6, B, T, H, dk, dv, BF, state=False)
    dO = torch.randn(B, T, H, dv, generator=g).to(BF)
    host = [t.pin_memory() for t in (q, k, v, dO)]
    outs = [torch.empty_like(t).pin_memory() for t in (v, q, k, v)]
    pipe = HostRetentionPipeline(q, v, "cuda", slices=slices, head_groups=head_groups)
    assert pipe.slices == (slices or B) * (head_groups or (H if (slices or B) * H <= pipe.TARGET_SLICES else 1))
    pipe.run(*host, decays, *outs)
    torch.cuda.synchronize()
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v)]
    o, _ = fp.fused_chunk_retention(*leaves, None, decays)
    o.backward(dO.cuda())
    for got, want in zip(outs, (o, leaves[0].grad, leaves[1].grad, leaves[2].grad)):
        assert torch.equal(got, want.detach().cpu())


def test_host_memory_pipeline_pop():
    """POP retention through the host pipeline (whole batch rows per slice) equals one direct call, bit for bit."""
    import flash_pop_b200 as fp
    from flash_pop_b200.host_io import HostRetentionPipeline
    B, T, H, d, block = 3, 400, 2, 64, 80
    decays = orc.head_decays(H, (5, 12))
    q, k, v, _, g = make_inputs(7, B, T, H, d, d, BF, state=False)
    dO = torch.randn(B, T, H, d, generator=g).to(BF)
    host = [t.pin_memory() for t in (q, k, v, dO)]
    outs = [torch.empty_like(q).pin_memory() for _ in range(4)]
    pipe = HostRetentionPipeline(q, v, "cuda", block_size=block)
    assert pipe.slices == B
    pipe.run(*host, decays, *outs)
    torch.cuda.synchronize()
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v)]
    o, _ = fp.flash_pop_retention(*leaves, None, decays, block)
    o.backward(dO.cuda())
    for got, want in zip(outs, (o, leaves[0].grad, leaves[1].grad, leaves[2].grad)):
        assert torch.equal(got, want.detach().cpu())


@pytest.mark.parametrize("M,N,P,d", [(8, 8, 80, 64), (12, 12, 40, 64), (9, 8, 80, 64), (6, 6, 100, 128)])
def test_grouped_suffix_walks_equal_one_cta_per_suffix(M, N, P, d):
    """Consecutive suffixes of a row walked by one CTA as one sequence (state replaced at every suffix start) give
    bit for bit what one CTA per suffix gives, forward and backward; odd counts and strided tensors fall back."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, H = 2, 3
    decays = orc.head_decays(H, (5, 12))
    g = torch.Generator().manual_seed(M * 100 + P)
    sq, sk, sv, sdo = ((torch.randn(B, M, P, H, d, generator=g) * d ** -0.5).to(BF).cuda() for _ in range(4))
    s0 = (torch.randn(B, H, d, d, generator=g) * d ** -0.5).to(BF).cuda()
    blocks = (torch.randn(B, N, H, d, d, generator=g) * d ** -0.5).to(BF).cuda()
    results = []
    with _lib.diagnostics_build() as diag:      # the schedule hooks exist in the diagnostics build only
        try:
            for limit, floor in ((1, 1), (16, 1)):
                diag.fpb_debug_suffix_group(limit, floor)
                leaves = [t.detach().clone().requires_grad_(True) for t in (sq, sk, sv, s0, blocks)]
                o = fp.pop_suffix_retention(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], decays)
                assert _lib.last_path() == _lib.PATH_TCGEN05
                o.backward(sdo)
                results.append([o.detach()] + [t.grad for t in leaves])
            _lib.device_status()
        finally:
            diag.fpb_debug_suffix_group(16, 3 * 296)
    for a, b in zip(*results):
        assert torch.equal(a, b)
    qd, kd, vd = (t.double().cpu() for t in (sq, sk, sv))
    o_ref = orc.pop_suffix_retention(qd, kd, vd, s0.double().cpu(), blocks.double().cpu(), decays)
    assert orc.rel_rms(results[1][0].float().cpu(), o_ref) < 5e-3
    _lib.device_status()


@pytest.mark.parametrize("T,block", [(5120, 80), (287, 144), (400, 96), (1000, 112)])
def test_block_states_from_partial_increments_match_the_block_aligned_walk(T, block):
    """POP forward at d = 64: the walk over full chunks with block states taken from partial state increments against
    the walk that cuts its chunks at block ends (same kernel, hook), and against the oracle."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    B, H, d = 2, 4, 64
    decays = orc.head_decays(H, (5, 12))
    q, k, v, s0, _ = make_inputs(T + block, B, T, H, d, d, BF)
    outs = []
    with _lib.diagnostics_build() as diag:
        try:
            for on in (0, 1):
                diag.fpb_debug_pop_emit(on)
                with torch.no_grad():
                    o, bs = fp.flash_pop_retention(q.cuda(), k.cuda(), v.cuda(), s0.cuda(), decays, block)
                assert _lib.last_path() == _lib.PATH_TCGEN05
                outs.append((o.cpu(), bs.cpu()))
            _lib.device_status()
        finally:
            diag.fpb_debug_pop_emit(1)
    o_ref, bs_ref = orc.pop_retention(q.double(), k.double(), v.double(), s0.double(), decays, block)
    for o, bs in outs:
        check("o", o, o_ref, BF)
        check("block states", bs, bs_ref, BF)
    # the two schedules differ in rounding only
    assert orc.rel_rms(outs[1][1].float(), outs[0][1].double()) < 5e-3
    _lib.device_status()
