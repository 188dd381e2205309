"""Golden outputs of the reference's own layer stacks (RetNetDecoder, POPRetNetDecoder.pop_forward,
DiffusionRetNetDecoder) run on CPU through their PyTorch retention path (use_fused_version=False for the
plain stacks; the POP operator is replaced by the reference's ``ref_pop`` test helper because its kernel
needs a GPU).  Weights are not stored: both sides fill every parameter from ``fill_parameters`` below.

    python tests/golden/make_golden_layers.py /path/to/flash-pop
"""
from __future__ import annotations

import ast
import os
import sys
from math import ceil

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
DIMS = dict(H=2, dk=64, dv=64, ffn=128, layers=2, B=2, T=48, block=16, P=8)


def fill_parameters(module: torch.nn.Module) -> None:
    """Deterministic weights that depend only on parameter name order, shape and index."""
    with torch.no_grad():
        for i, (name, p) in enumerate(sorted(module.named_parameters())):
            n = p.numel()
            vals = torch.sin(torch.arange(n, dtype=torch.float64) * 0.7371 + i * 1.618) * (0.5 / max(1, p.shape[-1]) ** 0.5)
            if name.endswith("norm1.weight") or name.endswith("norm2.weight"):
                vals = 1.0 + 0.1 * vals
            p.copy_(vals.reshape(p.shape).to(p.dtype))


def inputs(seed=0):
    g = torch.Generator().manual_seed(seed)
    D = DIMS["H"] * DIMS["dv"]
    x = torch.randn(DIMS["B"], DIMS["T"], D, generator=g)
    n_sfx = DIMS["T"] // DIMS["block"] + 1
    sfx = torch.randn(DIMS["B"], n_sfx, DIMS["P"], D, generator=g)
    c = torch.randn(DIMS["B"], D, generator=g)
    return x, sfx, c


def main(ref_root):
    sys.path.insert(0, ref_root)
    import flash_pop.xpos_emb as xp
    for n in ("_multiply_by_i", "_theta_shift", "_get_sin_cos"):      # run the rotary helpers eagerly
        f = getattr(xp, n)
        setattr(xp, n, getattr(f, "_torchdynamo_orig_callable", f))
    from flash_pop.fused_retention.reference import chunkwise_retention_
    from flash_pop.retnet import RetNetDecoder, RetNetDecoderLayer
    from flash_pop.pop_retnet import POPRetNetDecoder, POPDecoderLayer, POPMultiScaleRetention
    from flash_pop.diffusion_retnet import DiffusionRetNetDecoder, DiffusionRetNetDecoderLayer, DiffusionRetNetFinalLayer
    from flash_pop.recurrent_state import RecurrentState

    tree = ast.parse(open(os.path.join(ref_root, "tests", "test_pop_retention.py")).read())
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "ref_pop"][0]
    ns = {"ceil": ceil, "torch": torch, "chunkwise_retention_": chunkwise_retention_}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "ref_pop", "exec"), ns)
    ref_pop = ns["ref_pop"]

    d = DIMS
    x, sfx, c = inputs()
    common = dict(num_heads=d["H"], head_dim_v=d["dv"], head_dim_qk=d["dk"], dim_feedforward=d["ffn"], dropout=0.0,
                  device="cpu", dtype=torch.float32)
    out = {}
    torch.set_grad_enabled(False)

    # plain stack, chunk 16 so that several chunks are walked
    net = RetNetDecoder(RetNetDecoderLayer.Config(use_fused_version=False, chunk_size=16, **common), d["layers"])
    fill_parameters(net)
    y, st = net.forward_chunkwise(x, RecurrentState([None] * d["layers"], 0))
    y2, st2 = net.forward_chunkwise(x, RecurrentState(st.state, st.index))      # continue from the carried state
    out.update(retnet_y=y, retnet_state=st.state, retnet_y2=y2, retnet_state2=st2.state)

    # POP stack with suffixes; the POP operator is served by the reference's test helper
    def pop_kernel(self, q, k, v, prev_state):
        o, states = ref_pop(q.bfloat16(), k.bfloat16(), v.bfloat16(), prev_state.bfloat16(), self.head_decays, self.config.block_size)
        return o.to(v.dtype), states.to(v.dtype)
    POPMultiScaleRetention._pop_retention_kernel = pop_kernel
    pnet = POPRetNetDecoder(POPDecoderLayer.Config(block_size=d["block"], head_decays_range=(5, 12), use_fused_version=False,
                                                   chunk_size=64, **common), d["layers"])
    for layer in pnet.layers:      # the reference's POP layer does not forward this flag to its retention module
        layer.retention.config.use_fused_version = False
        layer.retention.config.chunk_size = 64
    fill_parameters(pnet)
    py, pst, psfx = pnet.pop_forward(x, RecurrentState([None] * d["layers"], 0), sfx)
    out.update(pop_y=py, pop_state=pst.state, pop_sfx=psfx)
    # generation scenario (the reference's tests/test_pop_retention.py:161-196): one full block plus a partial one in a
    # single sequence, and the suffixes that start from S_0 and from the one block state
    Tg = d["block"] + 7
    gy, gst, gsfx = pnet.pop_forward(x[:, :Tg], RecurrentState([None] * d["layers"], 0), sfx[:, :2])
    out.update(popgen_y=gy, popgen_state=gst.state, popgen_sfx=gsfx)

    # diffusion stack + final layer
    dcfg = DiffusionRetNetDecoderLayer.Config(use_fused_version=False, chunk_size=16, **common)
    dnet = DiffusionRetNetDecoder(DiffusionRetNetDecoder.Config(layer_config=dcfg, num_layers=d["layers"]))
    fin = DiffusionRetNetFinalLayer(DiffusionRetNetFinalLayer.Config(layer_config=dcfg, out_dim=24))
    fill_parameters(dnet), fill_parameters(fin)
    dy, dst = dnet.forward_chunkwise(x, c, RecurrentState([None] * d["layers"], 0))
    out.update(diff_y=dy, diff_state=dst.state, diff_final=fin(dy, c))

    np.savez_compressed(os.path.join(HERE, "layers.npz"), **{k: v.float().numpy() for k, v in out.items()})
    print({k: tuple(v.shape) for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} <checkout of leor-c/flash-pop>")
    main(sys.argv[1])
