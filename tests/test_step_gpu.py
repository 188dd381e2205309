"""The recurrent decoding step kernel against the oracle's token-by-token form and against the chunked operator."""
import pytest
import torch

from oracle import retention_oracle as orc
from util import check

pytestmark = pytest.mark.gpu
BF, F32 = torch.bfloat16, torch.float32


def _case(B, H, dk, dv, dtype, seed, with_state=True):
    g = torch.Generator().manual_seed(seed)
    q, k = ((torch.randn(B, H, dk, generator=g) * dk ** -0.5).to(dtype) for _ in range(2))
    v = (torch.randn(B, H, dv, generator=g) * dk ** -0.5).to(dtype)
    s = (torch.randn(B, H, dk, dv, generator=g) * dk ** -0.5) if with_state else None
    return q, k, v, s


@pytest.mark.parametrize("B,H,dk,dv,dtype,sdtype", [
    (3, 4, 64, 64, BF, BF), (2, 8, 128, 128, BF, F32), (2, 3, 128, 256, BF, BF), (5, 2, 64, 128, F32, F32),
    (2, 2, 48, 36, BF, BF),          # dv not a multiple of 8: the element-wise variant
    (2, 2, 40, 20, F32, F32), (1, 1, 8, 8, F32, BF), (4, 16, 256, 256, BF, F32),
])
def test_step_matches_oracle(B, H, dk, dv, dtype, sdtype):
    import flash_pop_b200 as fp
    decays = orc.head_decays(H, (5, 12) if H > 1 else None)
    q, k, v, s = _case(B, H, dk, dv, dtype, seed=B * 100 + dk)
    s = s.to(sdtype)
    o, s_new = fp.retention_step(q.cuda(), k.cuda(), v.cuda(), decays, s.cuda())
    assert o.dtype == dtype and s_new.dtype == sdtype and tuple(o.shape) == (B, H, dv)
    o_ref, s_ref = orc.retention_recurrent(q.double().unsqueeze(1), k.double().unsqueeze(1), v.double().unsqueeze(1),
                                           s.double(), decays)
    check("o", o.cpu(), o_ref[:, 0], dtype)
    check("state", s_new.cpu(), s_ref, sdtype)


def test_step_without_state_and_in_place():
    import flash_pop_b200 as fp
    decays = orc.head_decays(4, (5, 12))
    q, k, v, s = _case(3, 4, 64, 64, BF, seed=9)
    o0, s0 = fp.retention_step(q.cuda(), k.cuda(), v.cuda(), decays, None)
    o_ref, s_ref = orc.retention_recurrent(q.double().unsqueeze(1), k.double().unsqueeze(1), v.double().unsqueeze(1), None, decays)
    check("o", o0.cpu(), o_ref[:, 0], BF)
    check("state", s0.cpu(), s_ref, BF)
    sd = s.float().cuda()
    keep = sd.clone()
    o1, s1 = fp.retention_step(q.cuda(), k.cuda(), v.cuda(), decays, keep)
    o2, s2 = fp.retention_step(q.cuda(), k.cuda(), v.cuda(), decays, sd, in_place=True)
    assert s2.data_ptr() == sd.data_ptr() and torch.equal(s1, s2) and torch.equal(o1, o2)
    assert torch.equal(keep, s.float().cuda())          # the out-of-place call leaves its input alone


def test_decoding_token_by_token_equals_the_chunked_operator():
    """70 decoding steps with an fp32 state reproduce the chunked operator's outputs and end state."""
    import flash_pop_b200 as fp
    B, T, H, d = 2, 70, 4, 64
    decays = orc.head_decays(H, (5, 12))
    g = torch.Generator().manual_seed(21)
    q, k, v = ((torch.randn(B, T, H, d, generator=g) * d ** -0.5).to(BF).cuda() for _ in range(3))
    o_chunk, s_chunk = fp.fused_chunk_retention(q, k, v, None, decays)
    state, outs = None, []
    for t in range(T):
        o, state = fp.retention_step(q[:, t], k[:, t], v[:, t], decays, state, state_dtype=F32, in_place=True)
        outs.append(o)
    o_ref, s_ref = orc.retention_recurrent(q.double().cpu(), k.double().cpu(), v.double().cpu(), None, decays)
    check("o stepwise", torch.stack(outs, 1).cpu(), o_ref, BF)
    check("state stepwise", state.cpu(), s_ref, F32, rms_limit=1e-5)
    check("o chunked", o_chunk.cpu(), o_ref, BF)
    assert orc.rel_rms(torch.stack(outs, 1).float().cpu(), o_chunk.float().cpu().double()) < 5e-3


def test_layer_recurrent_path_uses_the_step_kernel():
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    cfg = fp.RetNetDecoderLayer.Config(num_heads=4, head_dim_v=64, dim_feedforward=128, dropout=0.0, device="cuda",
                                       dtype=F32)
    torch.manual_seed(0)
    dec = fp.RetNetDecoder(cfg, 2).eval()
    x = torch.randn(2, 6, 256, device="cuda")
    with torch.no_grad():
        y_chunk, _ = dec.forward_chunkwise(x)
        n0 = _lib.launch_count()
        state, ys = None, []
        for t in range(6):
            y, state = dec.forward_recurrent(x[:, t], state)
            ys.append(y)
        # per token and layer at least the step kernel (the fused GroupNorm-gate and LayerNorm kernels count as well)
        assert _lib.launch_count() - n0 >= 6 * 2 and _lib.last_path() == _lib.PATH_SIMT
    # the chunked path rounds q, k, v to bf16 (as the reference's does); the recurrent one stays in fp32
    assert torch.allclose(torch.stack(ys, 1), y_chunk, rtol=3e-2, atol=3e-2)
