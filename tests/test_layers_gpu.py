"""The layer stacks over the CUDA operators against outputs of the reference's own stacks (computed on
CPU through its PyTorch retention path by tests/golden/make_golden_layers.py, same deterministic
weights)."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def gold():
    z = np.load(os.path.join(GOLD, "layers.npz"))
    return {k: torch.from_numpy(z[k]) for k in z.files}


def _helpers():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden_layers", os.path.join(GOLD, "make_golden_layers.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def close(name, got, ref, tol=2e-2):
    got, ref = got.detach().float().cpu(), ref.float()
    assert got.shape == ref.shape, f"{name}: {tuple(got.shape)} vs {tuple(ref.shape)}"
    err = (got - ref).abs()
    rms = ref.square().mean().sqrt().item()
    assert (err <= tol * rms + tol * ref.abs()).all(), f"{name}: max err {err.max():.3e} (rms of reference {rms:.3e})"


def _common(h):
    d = h.DIMS
    return dict(num_heads=d["H"], head_dim_v=d["dv"], head_dim_qk=d["dk"], dim_feedforward=d["ffn"], dropout=0.0,
                device="cuda", dtype=torch.float32)


@pytest.mark.parametrize("fused", [True, False])
def test_retnet_stack_matches_reference_stack(gold, fused):
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    h = _helpers()
    d = h.DIMS
    x, _, _ = h.inputs()
    net = fp.RetNetDecoder(fp.RetNetDecoderLayer.Config(use_fused_version=fused, **_common(h)), d["layers"])
    h.fill_parameters(net)
    with torch.no_grad():
        y, st = net(x.cuda())                       # no state given: the decoder starts from zeros
        assert _lib.last_path() == (_lib.PATH_TCGEN05 if fused else _lib.PATH_SIMT)
        y2, st2 = net.forward_chunkwise(x.cuda(), st)
    _lib.device_status()
    assert st.index == d["T"] and st2.index == 2 * d["T"] and st.state.shape == (d["layers"], d["B"], d["H"], d["dk"], d["dv"])
    close("y", y, gold["retnet_y"]), close("state", st.state, gold["retnet_state"])
    close("y (second segment)", y2, gold["retnet_y2"]), close("state (second segment)", st2.state, gold["retnet_state2"])


def test_recurrent_steps_agree_with_chunkwise(gold):
    import flash_pop_b200 as fp
    h = _helpers()
    d = h.DIMS
    x, _, _ = h.inputs()
    net = fp.RetNetDecoder(fp.RetNetDecoderLayer.Config(**_common(h)), d["layers"])
    h.fill_parameters(net)
    xs = x.cuda()[:, :12]
    with torch.no_grad():
        y_chunk, st_chunk = net.forward_chunkwise(xs)
        st, ys = None, []
        for t in range(xs.size(1)):
            y_t, st = net.forward_recurrent(xs[:, t], st)
            ys.append(y_t)
    close("recurrent y", torch.stack(ys, 1), y_chunk.cpu())
    close("recurrent state", st.state, st_chunk.state.cpu())
    assert st.index == 12


def test_pop_stack_with_suffixes_matches_reference(gold):
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    h = _helpers()
    d = h.DIMS
    x, sfx, _ = h.inputs()
    net = fp.POPRetNetDecoder(fp.POPDecoderLayer.Config(block_size=d["block"], head_decays_range=(5, 12), **_common(h)), d["layers"])
    h.fill_parameters(net)
    with torch.no_grad():
        y, st, out_sfx = net.pop_forward(x.cuda(), None, sfx.cuda())
        y_only, st_blocks, none = net.pop_forward(x.cuda(), None, None)
    _lib.device_status()
    close("pop y", y, gold["pop_y"]), close("pop carried state", st.state, gold["pop_state"])
    close("pop suffixes", out_sfx, gold["pop_sfx"])
    assert none is None and st_blocks.state.shape == (d["layers"], d["B"], d["T"] // d["block"], d["H"], d["dk"], d["dv"])
    close("pop y without suffixes", y_only, gold["pop_y"])


def test_pop_generation_scenario_matches_reference(gold):
    """One full block plus a partial one in a single sequence and the two suffixes that start from S_0 and from the one
    block state (the reference's generation scenario, tests/test_pop_retention.py:161-196), through
    POPRetNetDecoder.pop_forward, against outputs of the reference's own stack."""
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    h = _helpers()
    d = h.DIMS
    x, sfx, _ = h.inputs()
    Tg = d["block"] + 7
    net = fp.POPRetNetDecoder(fp.POPDecoderLayer.Config(block_size=d["block"], head_decays_range=(5, 12), **_common(h)), d["layers"])
    h.fill_parameters(net)
    with torch.no_grad():
        y, st, out_sfx = net.pop_forward(x[:, :Tg].cuda(), None, sfx[:, :2].cuda())
    _lib.device_status()
    close("generation y", y, gold["popgen_y"]), close("generation carried state", st.state, gold["popgen_state"])
    close("generation suffixes", out_sfx, gold["popgen_sfx"])


def test_pop_stack_trains(gold):
    """Gradients reach the weights through both POP operators (stream and suffixes)."""
    import flash_pop_b200 as fp
    h = _helpers()
    d = h.DIMS
    x, sfx, _ = h.inputs()
    cfg = _common(h)
    cfg["dtype"] = torch.bfloat16
    net = fp.POPRetNetDecoder(fp.POPDecoderLayer.Config(block_size=d["block"], head_decays_range=(5, 12), **cfg), 1)
    y, st, out_sfx = net.pop_forward(x.cuda().bfloat16(), None, sfx.cuda().bfloat16())
    (y.float().square().mean() + out_sfx.float().square().mean()).backward()
    grads = [p.grad for p in net.parameters()]
    assert all(g is not None and torch.isfinite(g).all() for g in grads)
    assert sum(g.abs().sum().item() for g in grads) > 0


def test_diffusion_stack_matches_reference(gold):
    import flash_pop_b200 as fp
    h = _helpers()
    d = h.DIMS
    x, _, c = h.inputs()
    lc = fp.DiffusionRetNetDecoderLayer.Config(**_common(h))
    net = fp.DiffusionRetNetDecoder(fp.DiffusionRetNetDecoder.Config(layer_config=lc, num_layers=d["layers"]))
    fin = fp.DiffusionRetNetFinalLayer(fp.DiffusionRetNetFinalLayer.Config(layer_config=lc, out_dim=24))
    h.fill_parameters(net), h.fill_parameters(fin)
    with torch.no_grad():
        y, st = net(x.cuda(), c.cuda())
        out = fin(y, c.cuda())
    close("diffusion y", y, gold["diff_y"]), close("diffusion state", st.state, gold["diff_state"])
    close("final layer", out, gold["diff_final"])
