"""Generate the golden fixtures in this folder from the reference project itself.

Run where the reference tree is available:

    python tests/golden/make_golden.py /path/to/flash-pop

It imports the reference's PyTorch retention functions
(flash_pop/fused_retention/reference.py: chunkwise_retention, reference_grads;
flash_pop/retnet.py: retention_recurrent) and executes the reference test helper ``ref_pop``
(tests/test_pop_retention.py:13-32; that test module is not importable as shipped, so the
function's source is compiled out of the file with ``ast``), all on CPU with seeded inputs,
and stores inputs and outputs as ``.npz`` files.  Nothing of the reference is copied into
this repository; only its numerical outputs are.
"""
from __future__ import annotations

import ast
import os
import sys
from math import ceil  # noqa: F401  (used by the exec'd reference helper)

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _decays(num_heads, decay_range):
    if decay_range is None:
        e = -5.0 - np.arange(num_heads)
    else:
        e = -np.linspace(decay_range[0], decay_range[1], num_heads)
    return tuple((1 - np.exp2(e)).tolist())


def _load_ref_pop(ref_root, chunkwise_retention_):
    path = os.path.join(ref_root, "tests", "test_pop_retention.py")
    tree = ast.parse(open(path).read())
    fn = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "ref_pop"][0]
    ns = {"ceil": ceil, "torch": torch, "chunkwise_retention_": chunkwise_retention_}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), path, "exec"), ns)
    return ns["ref_pop"]


def _inputs(seed, B, T, H, dk, dv, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, dk, generator=g) * scale
    k = torch.randn(B, T, H, dk, generator=g) * scale
    v = torch.randn(B, T, H, dv, generator=g) * scale
    s = torch.randn(B, H, dk, dv, generator=g) * 0.5
    return q, k, v, s, g


def main(ref_root):
    sys.path.insert(0, ref_root)
    from flash_pop.fused_retention.reference import chunkwise_retention, chunkwise_retention_, reference_grads
    from flash_pop.retnet import retention_recurrent
    ref_pop = _load_ref_pop(ref_root, chunkwise_retention_)
    torch.manual_seed(0)
    torch.set_num_threads(4)

    def save(name, **arrs):
        np.savez_compressed(os.path.join(HERE, name), **{k: np.asarray(v) for k, v in arrs.items()})
        print("wrote", name, {k: tuple(np.asarray(v).shape) for k, v in arrs.items()})

    # ---- forward, chunkwise + recurrent, ragged T, non-zero start state, dk != dv -------------
    B, T, H, dk, dv = 2, 70, 3, 16, 24
    decays = _decays(H, (5, 12))
    q, k, v, s, g = _inputs(11, B, T, H, dk, dv)
    o32, st32 = chunkwise_retention(q, k, v, s, decays, chunk_size=32)
    o_full, st_full = chunkwise_retention(q, k, v, s, decays, chunk_size=T)
    gam = torch.tensor(decays, dtype=torch.float32).view(1, H, 1, 1)
    S = s.clone()
    o_rec = []
    for t in range(T):
        o_t, S = retention_recurrent(q[:, t], k[:, t], v[:, t], gam, S)
        o_rec.append(o_t)
    o_rec = torch.stack(o_rec, 1)
    save("fwd_ragged.npz", q=q, k=k, v=v, s=s, decays=np.array(decays), o_chunk32=o32, s_chunk32=st32,
         o_parallel=o_full, s_parallel=st_full, o_recurrent=o_rec, s_recurrent=S)

    # ---- closed-form grads + autograd through the chunkwise reference (q, k, v ~ N(0,1) * d^-0.5, default decays) --
    B, T, H, dk, dv = 2, 48, 4, 16, 16
    decays = _decays(H, None)
    q, k, v, s, g = _inputs(0, B, T, H, dk, dv, scale=dk ** -0.5)
    dO = torch.randn(B, T, H, dv, generator=g)
    dS = torch.randn(B, H, dk, dv, generator=g)
    dQ, dK, dV, dS0 = reference_grads(q, k, v, s, decays, dO, dS)
    leaves = [x.clone().requires_grad_(True) for x in (q, k, v, s)]
    o, st = chunkwise_retention(*leaves, decays, chunk_size=16)
    ((o * dO).sum() + (st * dS).sum()).backward()
    save("grads.npz", q=q, k=k, v=v, s=s, decays=np.array(decays), dO=dO, dS=dS,
         dQ=dQ, dK=dK, dV=dV, dS0=dS0, o=o.detach(), s_out=st.detach(),
         dQ_autograd=leaves[0].grad, dK_autograd=leaves[1].grad, dV_autograd=leaves[2].grad,
         dS0_autograd=leaves[3].grad)

    # ---- POP: block states, ragged tail, several block ends per 64-token chunk, and grads ------
    for name, (B, T, H, dk, dv, block) in {
        "pop_block15.npz": (2, 70, 2, 16, 24, 15),
        "pop_block40.npz": (1, 95, 3, 16, 16, 40),
    }.items():
        decays = _decays(H, (5, 12))
        q, k, v, s, g = _inputs(4, B, T, H, dk, dv)
        leaves = [x.clone().requires_grad_(True) for x in (q, k, v, s)]
        o, bs = ref_pop(*leaves, decays, block)
        dO = torch.randn(o.shape, generator=g)
        dBS = torch.randn(bs.shape, generator=g)
        ((o * dO).sum() + (bs * dBS).sum()).backward()
        save(name, q=q, k=k, v=v, s=s, decays=np.array(decays), block=np.array(block), o=o.detach(),
             block_states=bs.detach(), dO=dO, dBS=dBS, dQ=leaves[0].grad, dK=leaves[1].grad,
             dV=leaves[2].grad, dS0=leaves[3].grad)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} <checkout of leor-c/flash-pop>")
    main(sys.argv[1])
