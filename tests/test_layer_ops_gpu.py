"""The fused rotation and GroupNorm-gate kernels against their plain PyTorch expressions (fp64 on the same inputs)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
BF, F32 = torch.bfloat16, torch.float32


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == BF else dict(rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [BF, F32])
@pytest.mark.parametrize("start", [0, 37, "rows"])
def test_rotation_forward_and_backward(dtype, start):
    from flash_pop_b200.xpos_emb import XPos
    B, T, H, d = 3, 75, 4, 64
    g = torch.Generator().manual_seed(3)
    q0, k0, gq, gk = (torch.randn(B, T, H, d, generator=g).to(dtype).cuda() for _ in range(4))
    start_idx = torch.tensor([5, 0, 160], device="cuda") if start == "rows" else start
    fused, eager = XPos(d, seq_len_estimate=64, device="cuda"), XPos(d, seq_len_estimate=64, device="cuda")
    eager.fused = False
    res = []
    for xp, cast in ((fused, lambda t: t), (eager, lambda t: t.double())):
        q, k = cast(q0).detach().clone().requires_grad_(True), cast(k0).detach().clone().requires_grad_(True)
        if xp is eager:                       # the eager expression rounds through fp32; lift its table to fp64 instead
            ph = xp._rotation(T, start_idx).to(torch.complex128).unsqueeze(2)
            rq = torch.view_as_real(torch.view_as_complex(q.unflatten(-1, (-1, 2))) * ph).flatten(-2)
            rk = torch.view_as_real(torch.view_as_complex(k.unflatten(-1, (-1, 2))) * ph).flatten(-2)
        else:
            rq, rk = xp(q, k, start_idx)
            assert rq.dtype == dtype
        ((rq * cast(gq)).sum() + (rk * cast(gk)).sum()).backward()
        res.append((rq, rk, q.grad, k.grad))
    for got, ref in zip(*res):
        assert torch.allclose(got.double(), ref, **_tol(dtype))
        assert ((got.double() - ref).square().mean().sqrt() / ref.square().mean().sqrt()).item() < (5e-3 if dtype == BF else 1e-6)


def test_rotation_of_strided_views_and_to_bf16():
    from flash_pop_b200.layer_ops import rotary_qk
    from flash_pop_b200.xpos_emb import XPos
    B, T, H, d = 2, 40, 3, 128
    g = torch.Generator().manual_seed(4)
    qkv = torch.randn(B, T, 3, H, d, generator=g).cuda()            # q and k are strided views of one projection
    q, k = qkv[:, :, 0], qkv[:, :, 1]
    xp = XPos(d, device="cuda")
    ph = torch.view_as_real(xp._rotation(T, 11)).contiguous()
    rq, rk = rotary_qk(q, k, ph, BF)
    assert rq.dtype == BF
    xp.fused = False
    eq, ek = xp(q, k, 11)
    assert torch.allclose(rq.float(), eq, rtol=1e-2, atol=1e-2) and torch.allclose(rk.float(), ek, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dtype,dv,swish", [(BF, 128, True), (BF, 64, True), (F32, 128, True), (BF, 256, False),
                                            (F32, 72, True), (BF, 8, True)])
def test_groupnorm_gate_forward_and_backward(dtype, dv, swish):
    from flash_pop_b200.layer_ops import groupnorm_gate
    B, T, H, eps = 2, 33, 3, 1e-6
    g = torch.Generator().manual_seed(dv)
    o0, z0, dy = (torch.randn(B, T, H, dv, generator=g).to(dtype).cuda() for _ in range(3))
    o0 = o0 * 0.05 + 0.01                                               # small outputs with a mean, as retention gives
    o, z = o0.clone().requires_grad_(True), z0.clone().requires_grad_(True)
    y = groupnorm_gate(o, z, eps, swish)
    y.backward(dy)
    od, zd = o0.double().requires_grad_(True), z0.double().requires_grad_(True)
    n = F.group_norm(od.reshape(-1, H * dv), H, eps=eps).reshape(B, T, H, dv)
    ref = n * (F.silu(zd) if swish else zd)
    ref.backward(dy.double())
    assert y.dtype == dtype
    for name, got, want in (("y", y, ref), ("d_o", o.grad, od.grad), ("d_z", z.grad, zd.grad)):
        rr = ((got.double() - want).square().mean().sqrt() / want.square().mean().sqrt()).item()
        assert rr < (5e-3 if dtype == BF else 2e-5), f"{name}: rel-RMS {rr:.3e}"
        scale = want.abs().max().item()
        assert torch.allclose(got.double(), want.detach(), rtol=_tol(dtype)["rtol"], atol=_tol(dtype)["atol"] * max(scale, 1.0)), name


def test_layer_with_fused_passes_matches_layer_without():
    """The retention layer with the fused rotation / GroupNorm-gate against the same layer on the eager expressions."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import layer_ops, retnet
    cfg = fp.RetNetDecoderLayer.Config(num_heads=4, head_dim_v=64, dim_feedforward=128, dropout=0.0, device="cuda", dtype=BF)
    torch.manual_seed(0)
    layer = fp.RetNetDecoderLayer(cfg)
    x = torch.randn(2, 100, 256, device="cuda", dtype=BF)
    outs = []
    for fused in (True, False):
        layer.retention.xpos_embedder.fused = fused
        saved = retnet.groupnorm_gate_supported
        retnet.groupnorm_gate_supported = saved if fused else (lambda *a: False)
        try:
            xi = x.clone().requires_grad_(True)
            y, s = layer(xi)
            y.float().square().sum().backward()
            outs.append((y, s, xi.grad))
        finally:
            retnet.groupnorm_gate_supported = saved
    for a, b in zip(*outs):
        rr = ((a.float() - b.float()).square().mean().sqrt() / b.float().square().mean().sqrt()).item()
        assert rr < 2e-2, rr


@pytest.mark.parametrize("dtype,d,affine", [(BF, 1024, True), (BF, 256, True), (F32, 512, True), (BF, 264, False),
                                            (F32, 36, True), (BF, 8, True)])
def test_layer_norm_forward_and_backward(dtype, d, affine):
    from flash_pop_b200.layer_ops import layer_norm, layer_norm_supported
    rows_shape, eps = (3, 41), 1e-6
    g = torch.Generator().manual_seed(d)
    x0 = (torch.randn(*rows_shape, d, generator=g) * 1.5 + 0.3).to(dtype).cuda()
    dy = torch.randn(*rows_shape, d, generator=g).to(dtype).cuda()
    w0 = (1 + 0.1 * torch.randn(d, generator=g)).cuda() if affine else None
    b0 = (0.1 * torch.randn(d, generator=g)).cuda() if affine else None
    assert layer_norm_supported(x0, d)
    x = x0.clone().requires_grad_(True)
    w = None if w0 is None else w0.clone().requires_grad_(True)
    b = None if b0 is None else b0.clone().requires_grad_(True)
    y = layer_norm(x, w, b, eps)
    y.backward(dy)
    xd = x0.double().requires_grad_(True)
    wd = None if w0 is None else w0.double().requires_grad_(True)
    bd = None if b0 is None else b0.double().requires_grad_(True)
    ref = F.layer_norm(xd, (d,), wd, bd, eps)
    ref.backward(dy.double())
    pairs = [("y", y, ref), ("d_x", x.grad, xd.grad)]
    if affine:
        pairs += [("d_weight", w.grad, wd.grad), ("d_bias", b.grad, bd.grad)]
    for name, got, want in pairs:
        rr = ((got.double() - want).square().mean().sqrt() / want.square().mean().sqrt()).item()
        assert rr < (5e-3 if dtype == BF else 2e-5), f"{name}: rel-RMS {rr:.3e}"


def test_layer_norm_module_helper_matches_cast_norm_cast():
    from flash_pop_b200.layer_ops import norm_in_fp32
    torch.manual_seed(1)
    m = torch.nn.LayerNorm(512, device="cuda", dtype=F32)
    with torch.no_grad():
        m.weight.normal_(1.0, 0.1); m.bias.normal_(0.0, 0.1)
    x = torch.randn(4, 50, 512, device="cuda", dtype=BF)
    strided = torch.randn(4, 50, 1024, device="cuda", dtype=BF)[..., :512]       # rows 2048 bytes apart
    for t in (x, strided):
        want = m(t.float()).to(BF)
        got = norm_in_fp32(m, t)
        assert got.dtype == BF and torch.allclose(got.float(), want.float(), rtol=1e-2, atol=1e-2)
    big = torch.randn(2, 2048, device="cuda", dtype=BF)                          # wider than the kernel takes: eager path
    m2 = torch.nn.LayerNorm(2048, device="cuda", dtype=F32)
    assert torch.equal(norm_in_fp32(m2, big), m2(big.float()).to(BF))


@pytest.mark.parametrize("dtype,rows,V", [(BF, 300, 32000), (BF, 17, 1000), (F32, 64, 517), (BF, 5, 8)])
def test_cross_entropy_forward_and_backward(dtype, rows, V):
    from flash_pop_b200.layer_ops import FusedCrossEntropy, cross_entropy_supported
    g = torch.Generator().manual_seed(V)
    pad = (-V) % 8                                     # rows 16-byte aligned even when V is not a multiple of 8
    buf = (torch.randn(rows, V + pad, generator=g) * 3).to(dtype).cuda()
    logits0 = buf[:, :V]
    targets = torch.randint(0, V, (rows,), generator=g).cuda()
    targets[0] = -100                                   # ignored row
    assert cross_entropy_supported(logits0, targets)
    x = logits0.detach().requires_grad_(True)
    loss = FusedCrossEntropy.apply(x, targets)
    (loss * 1.7).backward()
    xd = logits0.double().detach().requires_grad_(True)
    ref = F.cross_entropy(xd, targets, ignore_index=-100, reduction="sum") / rows      # mean over ALL rows, ignored ones count as 0
    (ref * 1.7).backward()
    assert abs(loss.item() - ref.item()) < (2e-5 if dtype == F32 else 2e-4) * max(1.0, abs(ref.item()))
    rr = ((x.grad.double() - xd.grad).square().mean().sqrt() / xd.grad.square().mean().sqrt()).item()
    assert rr < (5e-3 if dtype == BF else 2e-5), rr
    assert x.grad.dtype == dtype and float(x.grad[0].abs().max()) == 0.0


def _rr(got, ref):
    return ((got.double() - ref).square().mean().sqrt() / ref.square().mean().sqrt().clamp_min(1e-30)).item()


@pytest.mark.parametrize("dtype", [BF, F32])
@pytest.mark.parametrize("Tm", [1, 4, 24])
@pytest.mark.parametrize("D", [256, 1024])
def test_adaln_modulate_and_gated_residual(dtype, Tm, D):
    """norm(x)(1 + scale) + shift and x + gate * branch with (B, Tm, D) operands shared by T / Tm tokens, taken in place as
    chunks of one (B, Tm, 3D) tensor (what the modulation MLP produces), against the fp64 PyTorch expressions: outputs,
    input gradients and the gradients of shift / scale / gate summed over the tokens that share them."""
    from flash_pop_b200.layer_ops import AdaLNModulate, GateResidual, row_broadcast_supported
    if dtype == F32 and D > 512:
        pytest.skip("fp32 rows are limited to 512 channels")
    B, T, eps = 3, 24, 1e-6
    g = torch.Generator().manual_seed(D + Tm)
    x, br, dy, dz = (torch.randn(B, T, D, generator=g).to(dtype).cuda() for _ in range(4))
    mod = (torch.randn(B, Tm, 3 * D, generator=g) * 0.5).to(dtype).cuda()
    leaves = [t.detach().clone().requires_grad_(True) for t in (x, br, mod)]
    shift, scale, gate = leaves[2].chunk(3, dim=-1)
    assert row_broadcast_supported(leaves[0], shift, scale)
    y = AdaLNModulate.apply(leaves[0], shift, scale, eps)
    z = GateResidual.apply(y, leaves[1], gate)
    ((y * dy).sum() + (z * dz).sum()).backward()
    ref = [t.double().detach().clone().requires_grad_(True) for t in (x, br, mod)]
    rs, rc, rg = (t.repeat_interleave(T // Tm, dim=1) for t in ref[2].chunk(3, dim=-1))
    yr = F.layer_norm(ref[0], (D,), None, None, eps) * (1 + rc) + rs
    # the fused chain hands the residual kernel y rounded to `dtype`; do the same in the reference
    y_in = y.detach().double()
    zr = y_in + ref[1] * rg
    ((yr * dy.double()).sum() + (zr * dz.double()).sum()).backward()
    lim = 4e-3 if dtype == BF else 2e-6
    assert _rr(y, yr.detach()) < lim and _rr(z, zr.detach()) < lim
    # d_x of the chain = d_y from the modulate (dy) + the residual's pass-through (dz) through the norm: build the same
    xr2 = x.double().detach().clone().requires_grad_(True)
    yr2 = F.layer_norm(xr2, (D,), None, None, eps) * (1 + rc.detach()) + rs.detach()
    (yr2 * (dy.double() + dz.double())).sum().backward()
    assert _rr(leaves[0].grad, xr2.grad) < lim
    assert _rr(leaves[1].grad, ref[1].grad) < lim
    # modulation gradients: shift <- sum(dy + dz), scale <- sum((dy + dz) n), gate <- sum(dz * branch)
    n = F.layer_norm(x.double(), (D,), None, None, eps)
    tot = (dy.double() + dz.double())
    want = torch.cat([tot.view(B, Tm, T // Tm, D).sum(2), (tot * n).view(B, Tm, T // Tm, D).sum(2),
                      (dz.double() * br.double()).view(B, Tm, T // Tm, D).sum(2)], dim=-1)
    assert _rr(leaves[2].grad, want) < (8e-3 if dtype == BF else 2e-6)


def test_adaln_modules_on_the_fused_path():
    """AdaLayerNormZero / AdaLayerNorm on CUDA against the same modules' arithmetic in fp64 (the reference's expression:
    fp32 LayerNorm, modulate, gate), for the three conditioning shapes."""
    from flash_pop_b200.modules.adaln import AdaLayerNormZero, gated_residual
    B, T, D = 2, 12, 256
    torch.manual_seed(0)
    m = AdaLayerNormZero(D, device="cuda", dtype=BF)
    torch.nn.init.normal_(m.modulation[-1].weight, std=0.05)
    torch.nn.init.normal_(m.modulation[-1].bias, std=0.05)
    x = torch.randn(B, T, D, device="cuda").to(BF)
    branch = torch.randn(B, T, D, device="cuda").to(BF)
    for c in (torch.randn(B, D, device="cuda").to(BF), torch.randn(B, 3, D, device="cuda").to(BF), torch.randn(B, T, D, device="cuda").to(BF)):
        y, gate_tokens = m(x, c)
        y2, gate_rows = m.forward_rows(x, c)
        assert torch.equal(y, y2) and gate_tokens.shape == x.shape
        out = gated_residual(y, branch, gate_rows)
        c3 = c.unsqueeze(1) if c.dim() == 2 else c
        modv = m.modulation(c3).double().repeat_interleave(T // c3.size(1), dim=1)
        shift, scale, gate = modv.chunk(3, dim=-1)
        y_ref = F.layer_norm(x.double(), (D,), None, None, m.norm.eps) * (1 + scale) + shift
        assert _rr(y, y_ref) < 4e-3
        assert _rr(gate_tokens, gate) < 1e-6
        assert _rr(out, y.double() + branch.double() * gate) < 4e-3


def test_cross_entropy_paths_share_one_definition_and_run_in_place():
    """Ignored / out-of-range targets: the fused kernel and the PyTorch fallback (taken for unaligned logits) give the
    same loss - a mean over ALL rows; and the backward may overwrite the logits buffer with the gradient."""
    import ctypes
    from flash_pop_b200 import _lib
    from flash_pop_b200.layer_ops import cross_entropy, cross_entropy_supported
    rows, V = 64, 1000
    g = torch.Generator().manual_seed(1)
    logits = (torch.randn(rows, V, generator=g) * 2).to(BF).cuda()
    targets = torch.randint(0, V, (rows,), generator=g).cuda()
    targets[3], targets[10], targets[11] = -100, V + 5, -1
    assert cross_entropy_supported(logits, targets)
    unaligned = torch.empty(rows, V + 3, dtype=BF, device="cuda")[:, 1:V + 1]      # rows start off 16-byte boundaries
    unaligned.copy_(logits)
    assert not cross_entropy_supported(unaligned, targets)
    a, b = logits.detach().requires_grad_(True), unaligned.detach().requires_grad_(True)
    la, lb = cross_entropy(a, targets), cross_entropy(b, targets)
    la.backward(), lb.backward()
    assert abs(la.item() - lb.item()) < 2e-4 * max(1.0, abs(lb.item()))
    assert _rr(a.grad, b.grad.double()) < 5e-3
    for r in (3, 10, 11):
        assert float(a.grad[r].abs().max()) == 0.0 and float(b.grad[r].abs().max()) == 0.0
    # in place through the C ABI: d_logits = the logits buffer
    loss = torch.empty(rows, device="cuda"); lse = torch.empty(rows, device="cuda")
    scale = torch.ones(1, device="cuda")
    buf = logits.clone()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = _lib.stream_ptr(buf.device)
    _lib.check(_lib.lib().fpb_cross_entropy_fwd(rows, V, _lib.FPB_BF16, p(buf), V, p(targets), p(loss), p(lse), st))
    _lib.check(_lib.lib().fpb_cross_entropy_bwd(rows, V, _lib.FPB_BF16, p(buf), V, p(targets), p(lse), p(scale), 1.0 / rows, p(buf), V, st))
    torch.cuda.synchronize()
    assert torch.equal(buf, a.grad)
