"""Host-side logic of the layer callers that needs no GPU: parameter names (checkpoint compatibility with
the reference, whose names are listed here from flash_pop/retnet.py:194-210,430-446 and
flash_pop/diffusion_retnet.py:79-97,178-186), rotary tables, decays, state container, AdaLN broadcasting."""
import math

import pytest
import torch

import flash_pop_b200 as fp
from flash_pop_b200.modules import AdaLayerNorm, AdaLayerNormZero, TimestepEmbedder
from flash_pop_b200.retnet import get_decays, retention_recurrent
from flash_pop_b200.xpos_emb import XPos

CPU = dict(device="cpu", dtype=torch.float32)


def test_exported_names_match_reference_package():
    for name in ("fused_chunk_retention", "flash_pop_retention", "RetNetDecoderLayer", "RetNetDecoder", "POPRetNetDecoder",
                 "POPDecoderLayer", "DiffusionRetNetDecoder", "DiffusionRetNetDecoderLayer", "DiffusionRetNetFinalLayer",
                 "RecurrentState"):
        assert hasattr(fp, name), name


def test_retnet_parameter_names():
    net = fp.RetNetDecoder(fp.RetNetDecoderLayer.Config(num_heads=2, head_dim_v=16, head_dim_qk=8, dim_feedforward=32, **CPU), 1)
    names = set(net.state_dict())
    expected = {f"layers.0.{m}.{p}" for m in ("norm1", "norm2", "linear1", "linear2") for p in ("weight", "bias")}
    expected |= {f"layers.0.retention.{m}.{p}" for m in ("q_proj", "k_proj", "v_proj", "g_proj", "out_proj") for p in ("weight", "bias")}
    assert names == expected
    assert net.layers[0].retention.q_proj.weight.shape == (16, 32) and net.layers[0].retention.v_proj.weight.shape == (32, 32)


def test_diffusion_parameter_names():
    lc = fp.DiffusionRetNetDecoderLayer.Config(num_heads=2, head_dim_v=16, dim_feedforward=32, ada_ln_lora_dim=4, **CPU)
    net = fp.DiffusionRetNetDecoder(fp.DiffusionRetNetDecoder.Config(layer_config=lc, num_layers=1))
    names = set(net.state_dict())
    for n in ("layers.0.ada_ln1.modulation.1.weight", "layers.0.ada_ln1.modulation.2.weight", "layers.0.ada_ln1.modulation.2.bias",
              "layers.0.ada_ln2.modulation.1.weight", "layers.0.retention.q_proj.weight", "layers.0.linear1.weight"):
        assert n in names, n
    fin = fp.DiffusionRetNetFinalLayer(fp.DiffusionRetNetFinalLayer.Config(layer_config=lc, out_dim=5))
    assert {"final_ada_ln.modulation.1.weight", "final_linear.weight", "final_linear.bias"} <= set(fin.state_dict())


def test_decays():
    assert get_decays(4).tolist() == [1 - 2.0 ** (-5 - h) for h in range(4)]
    d = get_decays(8, (5, 12))
    assert abs(d[0] - (1 - 2 ** -5)) < 1e-15 and abs(d[-1] - (1 - 2 ** -12)) < 1e-15


def test_rotary_matches_pairwise_rotation_formula():
    xp = XPos(8, device="cpu")
    q = torch.randn(2, 5, 3, 8)
    k = torch.randn(2, 5, 3, 8)
    theta = 1.0 / (10000 ** torch.linspace(0, 1, 4))
    for start in (0, 11):
        rq, rk = xp(q, k, start)
        for t in range(5):
            ang = (start + t) * theta
            want0 = q[:, t, :, 0::2] * ang.cos() - q[:, t, :, 1::2] * ang.sin()
            want1 = q[:, t, :, 0::2] * ang.sin() + q[:, t, :, 1::2] * ang.cos()
            assert torch.allclose(rq[:, t, :, 0::2], want0, atol=1e-5) and torch.allclose(rq[:, t, :, 1::2], want1, atol=1e-5)
    # one offset per batch row (the POP suffixes)
    starts = torch.tensor([3, 40])
    rq, _ = xp(q, k, starts)
    for b in range(2):
        alone, _ = xp(q[b:b + 1], k[b:b + 1], int(starts[b]))
        assert torch.allclose(rq[b:b + 1], alone, atol=1e-6)
    # a single decoding step at position p equals row p of the sequence form
    step_q, _ = xp(q[:, 2], k[:, 2], 13)
    seq_q, _ = xp(q, k, 11)
    assert torch.allclose(step_q, seq_q[:, 2], atol=1e-6)
    sin, cos = xp.get_sin_cos(5, 0)
    assert sin.shape == (1, 5, 1, 8) and torch.allclose(sin[0, 1, 0, 0::2], theta.sin(), atol=1e-6)


def test_recurrent_step_formula():
    q, k, v = torch.randn(2, 3, 4), torch.randn(2, 3, 4), torch.randn(2, 3, 5)
    g = torch.tensor([0.9, 0.8, 0.7]).view(1, 3, 1, 1)
    s_prev = torch.randn(2, 3, 4, 5)
    o, s = retention_recurrent(q, k, v, g, s_prev)
    want = s_prev * g + torch.einsum("bhk,bhv->bhkv", k / 2.0, v)
    assert torch.allclose(s, want, atol=1e-6) and torch.allclose(o, torch.einsum("bhk,bhkv->bhv", q, want), atol=1e-5)


def test_recurrent_state_container():
    rs = fp.RecurrentState(torch.zeros(2, 1, 1, 2, 2), 5)
    c = rs.clone()
    c.state += 1
    assert rs.state.sum() == 0 and c.index == 5 and set(rs.to_dict()) == {"state", "index"}
    assert rs.cpu_clone().state.device.type == "cpu" and rs.to_device("cpu") is rs


def test_decoder_rejects_wrong_number_of_states():
    net = fp.RetNetDecoder(fp.RetNetDecoderLayer.Config(num_heads=2, head_dim_v=16, dim_feedforward=32, **CPU), 2)
    with pytest.raises(ValueError):
        net._validate_and_init_state(fp.RecurrentState(torch.zeros(3, 1, 2, 16, 16), 0))
    fresh = net._validate_and_init_state(None)
    assert fresh.state == [None, None] and fresh.index == 0


def test_adaln_broadcasting_and_zero_init():
    x = torch.randn(2, 6, 8)
    ada = AdaLayerNormZero(8, **CPU)
    for c in (torch.randn(2, 8), torch.randn(2, 3, 8), torch.randn(2, 6, 8)):
        y, gate = ada(x, c)
        assert y.shape == x.shape and gate.shape == x.shape
        assert torch.allclose(y, torch.nn.functional.layer_norm(x, (8,), eps=1e-6), atol=1e-6) and gate.abs().sum() == 0
    lora = AdaLayerNorm(8, lora_hidden_dim=2, **CPU)
    assert lora(x, torch.randn(2, 8)).shape == x.shape
    with torch.no_grad():
        for p in ada.modulation.parameters():
            p.normal_()
    c = torch.randn(2, 3, 8)
    y, gate = ada(x, c)            # per-frame conditioning: each of the 3 frames covers 2 consecutive tokens
    assert torch.allclose(gate[:, 0], gate[:, 1]) and not torch.allclose(gate[:, 1], gate[:, 2])


def test_timestep_embedding():
    emb = TimestepEmbedder(16, frequency_embedding_size=8, **CPU)
    t = torch.tensor([[0.0, 1.5], [2.0, 3.0]])
    f = TimestepEmbedder.timestep_embedding(t, 8)
    assert f.shape == (2, 2, 8) and torch.allclose(f[0, 0], torch.tensor([1.0] * 4 + [0.0] * 4))
    freqs = torch.exp(-math.log(10000) * torch.arange(4) / 4)
    assert torch.allclose(f[0, 1, :4], (1.5 * freqs).cos(), atol=1e-6)
    assert TimestepEmbedder.timestep_embedding(t, 7).shape == (2, 2, 7) and emb(t).shape == (2, 2, 16)
