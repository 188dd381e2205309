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
