"""Diagnostics for the tensor-core kernels, on the diagnostics build of the library (the release sources compiled with
-DFPB_DIAGNOSTICS, which adds clock stamps to the warp roles): where the time of one chunk goes.

    python -m flash_pop_b200.diagnostics [B H T d [fwd|dq]]

prints, for the first CTA of a forward (or dQ) walk, the events of a few chunks in order - copies issued, tile rescaled,
each product issued, scores / accumulator seen by the score warps, state copy published - in SM clock cycles, and the mean
period of each event over 40 chunks, and what the MMA-issuing thread spends per chunk in barrier tests, commits, tcgen05.mma
issue and fences.  A chunk's period is what bounds the walk; the lag of an event behind the issue of the chunk's copies
shows which hand-off the chunk waits on."""
from __future__ import annotations

import ctypes
import sys

EVENTS = {0: "mma: scores issued", 1: "mma: state term issued", 2: "mma: state term begins", 3: "mma: intra term issued",
          4: "mma: increment issued", 5: "mma: stage released", 6: "score warps: scores seen", 7: "score warps: P' written",
          8: "score warps: accumulator seen", 9: "score warps: epilogue begins", 10: "score warps: epilogue done",
          11: "state warps: tile rescaled", 12: "state warps: increment seen", 13: "state warps: state copy published",
          14: "producer: copies issued", 15: "mma: intra term begins"}


def chunk_timeline(B: int = 8, H: int = 16, T: int = 8192, d: int = 128, walk: str = "fwd", first_chunk: int = 20, show: int = 3):
    import numpy as np
    import torch
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    decays = tuple((1 - np.exp2(-np.linspace(5, 12, H))).tolist())
    q, k, v, dO = (torch.randn(B, T, H, d, device="cuda", dtype=torch.bfloat16) * d ** -0.5 for _ in range(4))
    with _lib.diagnostics_build() as diag:
        if walk == "fwd":
            def run():
                with torch.no_grad():
                    fp.fused_chunk_retention(q, k, v, None, decays)
        else:
            ql = q.detach().requires_grad_(True)
            o, _ = fp.fused_chunk_retention(ql, k, v, None, decays)
            run = lambda: torch.autograd.grad(o, [ql], dO, retain_graph=True)
        for _ in range(3):
            run()
        stamps = torch.zeros(64 * 16, dtype=torch.int64, device="cuda")
        diag.fpb_debug_trace(ctypes.c_void_p(stamps.data_ptr()))
        run()
        torch.cuda.synchronize()
        diag.fpb_debug_trace(None)
        _lib.device_status()
    t = stamps.cpu().numpy().reshape(64, 16)
    lines = [f"B={B} H={H} T={T} d={d} walk={walk}: SM clock cycles, CTA (0,0,0)"]
    base = t[first_chunk][t[first_chunk] > 0].min()
    for c in range(first_chunk, first_chunk + show):
        ev = sorted((int(t[c][i] - base), EVENTS[i]) for i in range(16) if t[c][i] > 0)
        lines.append(f"chunk {c}: " + "; ".join(f"{name} @{x}" for x, name in ev))
    lo, hi = 10, min(50, (T + 63) // 64)
    for i in sorted(EVENTS):
        col = t[lo:hi, i]
        if hi - lo > 2 and (col > 0).all():
            lines.append(f"{EVENTS[i]:38s} period {np.diff(col).mean():7.0f}   lag behind the copies' issue {np.mean(col - t[lo:hi, 14]):7.0f}")
    acct = t[63][:8]
    chunks = (T + 63) // 64
    if acct[4:].any():
        names = ("barrier tests", "commits", "tcgen05.mma issue", "tcgen05 fences")
        lines.append(f"MMA-issuing thread, whole walk ({chunks} chunks): " + "; ".join(
            f"{names[i]} {acct[i] / chunks:.0f} cycles per chunk in {acct[4 + i] / chunks:.1f} calls" for i in range(4)))
    return "\n".join(lines)


if __name__ == "__main__":
    args = sys.argv[1:]
    nums = [int(a) for a in args[:4]] if len(args) >= 4 else [8, 16, 8192, 128]
    print(chunk_timeline(*nums, walk=args[4] if len(args) > 4 else "fwd"))
