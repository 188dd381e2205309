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
