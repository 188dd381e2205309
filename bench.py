#!/usr/bin/env python
"""Benchmark of the chunked-retention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload ns|c3|c4|c5|decode|layer]

Workload "ns" (default) is the configuration the headline metric is quoted on: chunked retention
forward+backward, bf16, B=8, H=16, T=8192, dk=dv=128 per GPU, decays 1-2^-linspace(5,12,H), seeded
synthetic inputs q,k,v ~ N(0,1)*d^-0.5, dO ~ N(0,1).  A step is one forward and one backward of the
operator through the C ABI.  With N GPUs every rank runs the same per-GPU problem on its own batch
rows (weak scaling, no collective on the data path); the time is the max over ranks.

Prints ONE JSON line (rank 0).  `value` is algorithmic TFLOP/s with inputs resident in HBM; `e2e` is
the same metric with host buffers (pinned) copied in and every result copied back inside the timed
region (`e2e.copy_only_ms`: the same copies without the kernels).  The default line carries two sub-records:
`strong` - the SAME B=8 problem split over the ranks with flash_pop_b200.parallel.partition - and `c5` - a few steps
of the full 12-layer RetNet training step under DistributedDataParallel (tokens/s).  `--impl reference` times the
reference's PyTorch CPU algorithm (the CPU port in oracle/) on the host cores over a bounded sample of the same
workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B, H, T, dk, dv, pop block (0 = plain retention)
    "ns": dict(B=8, H=16, T=8192, dk=128, dv=128, block=0),
    "c3": dict(B=4, H=32, T=16384, dk=128, dv=256, block=0),
    "c4": dict(B=16, H=8, T=5120, dk=64, dv=64, block=80),
    # reduced cases for profiler captures: inputs still larger than L2, launches not under-filled (so the same kernels
    # run unsplit), at most a few GB on the device
    "small": dict(B=5, H=16, T=8192, dk=128, dv=128, block=0),
    "c3s": dict(B=2, H=32, T=16384, dk=128, dv=256, block=0),
}
# the full RetNet stack under data parallelism: 12 layers, d_model 1024, global batch 64 x 4096 fixed (strong scaling)
STACK = dict(layers=12, heads=8, head_dim=128, ffn=4096, vocab=32000, B=64, T=4096, micro_batch=32)
CHUNK = 64


def flops_per_token_head(dk, dv, C=CHUNK):
    ch = (C + 1) / 2
    fwd = 2 * ch * (dk + dv) + 4 * dk * dv
    bwd = 2 * ch * (3 * dk + 2 * dv) + 8 * dk * dv
    return fwd, bwd


def bytes_per_token_head(dk, dv, e=2):
    return e * (2 * dk + 2 * dv), e * (4 * dk + 3 * dv)


def decays_for(H):
    import numpy as np
    return tuple((1 - np.exp2(-np.linspace(5, 12, H))).tolist())


def make_host_inputs(w, seed, pin, rows=None):
    """q, k, v, dO of the workload (bf16, host).  Every (tensor, batch row) has its own seed, so a rank that owns only
    some rows of the problem builds exactly those (`rows` = a range of batch rows; default all)."""
    B, H, T, dk, dv = w["B"], w["H"], w["T"], w["dk"], w["dv"]
    rows = range(B) if rows is None else rows
    out = []
    for i, (d, sc) in enumerate(((dk, dk ** -0.5), (dk, dk ** -0.5), (dv, dk ** -0.5), (dv, 1.0))):
        t = torch.empty(len(rows), T, H, d, dtype=torch.bfloat16)
        for j, b in enumerate(rows):   # row by row keeps the fp32 temporary small
            g = torch.Generator().manual_seed((seed * 8 + i) * 4096 + b)
            t[j] = (torch.randn(T, H, d, generator=g) * sc).to(torch.bfloat16)
        out.append(t.pin_memory() if pin else t)
    return out   # q, k, v, dO


# --------------------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self.proc = index, [], None

    def run(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])
        except Exception:
            pass

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        self.join(timeout=2)
        sm, reasons, mx = [], set(), None
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx = float(r[1])
            except Exception:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def event_time_ms(fn, steps):
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def graph_time_ms(fn, steps):
    """`fn` captured once in a CUDA graph and replayed: the device time of a step whose kernels are short enough for the
    Python call overhead (tens of microseconds per operator call) to show in an eager loop."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    for _ in range(3):
        graph.replay()
    return event_time_ms(graph.replay, steps)


# --------------------------------------------------------------------------------------------------
def cpu_reference_pass(w, rows, threads):
    """One forward+backward of the reference's PyTorch CPU algorithm (its restatement in oracle/, pinned bit for bit to
    the reference's own functions by the committed fixtures) on `rows` batch rows of the workload; returns seconds."""
    from oracle import retention_oracle as orc
    torch.set_num_threads(threads)
    H, T, dk, dv = w["H"], w["T"], w["dk"], w["dv"]
    dec = decays_for(H)
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(rows, T, H, d, generator=g) * dk ** -0.5 for d in (dk, dk, dv))
    dO = torch.randn(rows, T, H, dv, generator=g)
    leaves = [t.requires_grad_(True) for t in (q, k, v)]
    t0 = time.perf_counter()
    if w["block"]:
        o, _ = orc.pop_retention(*leaves, None, dec, w["block"])
    else:
        o, _ = orc.retention_chunkwise(*leaves, None, dec, chunk_size=CHUNK)
    (o * dO).sum().backward()
    return time.perf_counter() - t0


def cpu_reference_tflops(w, rows, passes, warmup, threads):
    """Mean over `passes` timed passes after `warmup` untimed ones - the one method both CPU figures use."""
    for _ in range(warmup):
        cpu_reference_pass(w, rows, threads)
    dt = sum(cpu_reference_pass(w, rows, threads) for _ in range(passes)) / passes
    ff, fb = flops_per_token_head(w["dk"], w["dv"])
    return (ff + fb) * rows * w["T"] * w["H"] / dt / 1e12, dt


def cpu_sample_text(w, rows, passes):
    return (f"{rows} of {w['B']} batch rows (H={w['H']}, T={w['T']}), fp32 torch CPU, chunk {CHUNK}, mean of {passes} "
            f"pass(es) after a warm-up")


def op_config(args, w):
    """The `config` object of an operator workload: identical for both arms."""
    return {"workload": workload_name(args, w), "l2": "inputs (1 GB+) larger than the 126 MB L2; no flush",
            "flop_count": "algorithmic, causal half of intra-chunk tiles (C=64)"}


def run_reference(args, w, rank):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows = 1
    tf, dt = cpu_reference_tflops(w, rows, args.steps, max(args.warmup, 1), threads)
    line = {
        "impl": "reference", "metric": "chunked_retention_fwd_bwd_tflops", "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "tokens_per_s": rows * w["T"] / dt,
        "config": op_config(args, w),
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": cpu_sample_text(w, rows, args.steps)},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_decode(args):
    """Recurrent decoding step over a (layers, B, H, dk, dv) state set: one kernel launch per layer per token, the
    token's launches captured in a CUDA graph (the loop is launch-bound from Python otherwise).
    Metric: state bytes streamed per second (read + write), against the measured HBM copy bandwidth."""
    from flash_pop_b200 import _lib, retention_step
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the decoding-step workload is reported for the CUDA "
                          "kernel only; the reference arm covers the operator workloads"}))
        return
    dev = torch.device("cuda", 0)
    L, B, H, d = 12, 256, 8, 128
    dec = decays_for(H)
    g = torch.Generator().manual_seed(6)
    q, k, v = ((torch.randn(L, B, H, d, generator=g) * d ** -0.5).to(torch.bfloat16).to(dev) for _ in range(3))
    out = {}
    for name, sdt in (("bf16", torch.bfloat16), ("f32", torch.float32)):
        states = [torch.zeros(B, H, d, d, device=dev, dtype=sdt) for _ in range(L)]

        def token():
            for l in range(L):
                retention_step(q[l], k[l], v[l], dec, states[l], in_place=True)
        side = torch.cuda.Stream(dev)
        with torch.cuda.stream(side):                      # warm up off the default stream, then capture one token
            for _ in range(args.warmup):
                token()
        torch.cuda.current_stream(dev).wait_stream(side)
        n0 = _lib.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            token()
        launches = (_lib.launch_count() - n0) * args.steps  # the graph replays the captured launches every step
        for _ in range(3):
            graph.replay()
        ms = event_time_ms(graph.replay, args.steps)
        nbytes = 2 * L * B * H * d * d * states[0].element_size()
        out[name] = {"ms_per_token": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "bytes": nbytes, "launches": launches}
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]; src = "measured"
    except Exception:
        peak = 6650.0; src = "fallback"
    top = out["bf16"]
    print(json.dumps({
        "metric": "retention_decode_step_state_gbs", "value": top["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": top["ms_per_token"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"recurrent decoding step, {L} layers x B={B} H={H} dk=dv={d}, bf16 activations, "
                               f"bf16 state updated in place (fp32 state beside it)",
                   "l2": f"state set {top['bytes'] // 2 / 1e6:.0f} MB per token, larger than L2"},
        "roofline": {"bound": "hbm", "achieved": top["gbs"], "peak": peak, "unit": "GB/s", "frac": top["gbs"] / peak,
                     "peak_source": src, "traffic": None},
        "f32_state": out["f32"], "tokens_per_s": B / (top["ms_per_token"] * 1e-3), "gpu_launches": top["launches"],
    }), flush=True)


def run_layer_passes(args):
    """The fused elementwise passes of a retention layer at the full-stack shape (16 x 4096 tokens, 8 heads of 128):
    GB/s of each kernel over its algorithmic bytes (every tensor read or written once)."""
    from flash_pop_b200 import _lib
    from flash_pop_b200.layer_ops import _rotate, groupnorm_gate, layer_norm
    from flash_pop_b200.xpos_emb import XPos
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the layer-pass workload is reported for the CUDA kernels "
                          "only; the reference arm covers the operator workloads"}))
        return
    dev = torch.device("cuda", 0)
    B, T, H, d = 16, 4096, 8, 128
    g = torch.Generator().manual_seed(7)
    q, k, o, z, dy = (torch.randn(B, T, H, d, generator=g).to(torch.bfloat16).to(dev) for _ in range(5))
    ph = torch.view_as_real(XPos(d, seq_len_estimate=T, device=dev)._rotation(T, 0)).contiguous()
    tensor_bytes = q.numel() * 2
    o.requires_grad_(True); z.requires_grad_(True)
    y = groupnorm_gate(o, z, 1e-6, True)
    x = q.view(B * T, H * d).detach().requires_grad_(True)
    lw = torch.ones(H * d, device=dev, requires_grad=True); lb = torch.zeros(H * d, device=dev, requires_grad=True)
    ln_y = layer_norm(x, lw, lb, 1e-6)
    ln_dy = dy.view(B * T, H * d)
    cases = {
        "layer_norm forward": (lambda: layer_norm(x.detach(), lw.detach(), lb.detach(), 1e-6), 2 * tensor_bytes),
        "layer_norm backward": (lambda: torch.autograd.grad(ln_y, (x, lw, lb), ln_dy, retain_graph=True), 3 * tensor_bytes),
        "rotary (q and k)": (lambda: _rotate(q, k, ph, False, torch.bfloat16), 4 * tensor_bytes),
        "groupnorm_gate forward": (lambda: groupnorm_gate(o.detach(), z.detach(), 1e-6, True), 3 * tensor_bytes),
        "groupnorm_gate backward": (lambda: torch.autograd.grad(y, (o, z), dy, retain_graph=True), 5 * tensor_bytes),
    }
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]; src = "measured"
    except Exception:
        peak = 6650.0; src = "fallback"
    out, n0 = {}, _lib.launch_count()
    for name, (fn, nbytes) in cases.items():
        for _ in range(args.warmup):
            fn()
        ms = event_time_ms(fn, args.steps)
        out[name] = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac": nbytes / (ms * 1e-3) / 1e9 / peak, "bytes": nbytes}
    top = out["groupnorm_gate backward"]
    print(json.dumps({
        "metric": "layer_pass_gbs", "value": top["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": top["ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"fused layer passes, bf16 (B,T,H,d)=({B},{T},{H},{d}); value = GroupNorm-gate backward",
                   "l2": f"each tensor {tensor_bytes / 1e6:.0f} MB, every pass moves 3-5 of them: larger than L2"},
        "roofline": {"bound": "hbm", "achieved": top["gbs"], "peak": peak, "unit": "GB/s", "frac": top["frac"],
                     "peak_source": src, "traffic": None},
        "passes": out, "gpu_launches": _lib.launch_count() - n0,
    }), flush=True)


def workload_name(args, w):
    kind = "POP retention" if w["block"] else "chunked retention"
    return (f"{kind} fwd+bwd bf16 B={w['B']} H={w['H']} T={w['T']} dk={w['dk']} dv={w['dv']} C={CHUNK}"
            + (f" block={w['block']}" if w["block"] else "") + " per GPU")


# --------------------------------------------------------------------------------------------------
def stack_record(args, dev, rank, world, steps, warmup, sample_clocks=True):
    """Full 12-layer RetNet training step (embedding, stack, head, cross entropy, AdamW), bf16, global batch 64 x 4096
    tokens split over the ranks (strong scaling), micro-batches with gradient accumulation, NCCL gradient all-reduce
    through DistributedDataParallel on the last micro-batch.  Metric: tokens/s.  Uses the default process group when
    world > 1; returns the record on rank 0 (None elsewhere)."""
    import contextlib
    import torch.distributed as dist
    from flash_pop_b200 import _lib
    from flash_pop_b200.layer_ops import cross_entropy
    from flash_pop_b200.stack_lm import RetNetLM
    local = dev.index
    c = STACK
    torch.manual_seed(0)
    model = RetNetLM(c["vocab"], c["layers"], c["heads"], c["head_dim"], c["ffn"], device=dev)
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], gradient_as_bucket_view=True) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)
    rows = c["B"] // world
    mb = min(args.micro_batch or c["micro_batch"], rows)
    g = torch.Generator().manual_seed(5 + rank)
    host_tokens = torch.randint(0, c["vocab"], (rows, c["T"] + 1), generator=g).pin_memory()
    tokens = torch.empty_like(host_tokens, device=dev)

    def loss_of(tok):                                          # through `net` so that DDP's gradient hooks are armed
        logits, _ = net(tok[:, :-1])
        return cross_entropy(logits.flatten(0, 1), tok[:, 1:].flatten())   # fp32 arithmetic on the bf16 logits, one kernel each way

    def step():
        tokens.copy_(host_tokens, non_blocking=True)           # the step's input comes from the host
        opt.zero_grad(set_to_none=True)
        total = torch.zeros((), device=dev)
        n_mb = rows // mb
        for i in range(n_mb):
            sync = contextlib.nullcontext() if (world == 1 or i == n_mb - 1) else net.no_sync()
            with sync:                                         # gradients are all-reduced on the last micro-batch only
                loss = loss_of(tokens[i * mb:(i + 1) * mb]) / n_mb
                loss.backward()
            total += loss.detach()
        opt.step()
        return total

    for _ in range(warmup):
        step()
    _lib.device_status(dev)
    sampler = ClockSampler(local) if (rank == 0 and sample_clocks) else None
    if sampler:
        sampler.start(); time.sleep(0.3)
    launches0 = _lib.launch_count()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    last = None
    for _ in range(steps):
        last = step().item()                                   # device -> host read of the step's loss
    b.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = a.elapsed_time(b) / steps
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()
    launches = _lib.launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    flops_per_token = model.flops_per_token(c["T"])
    del net, opt, model, tokens
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    toks = c["B"] * c["T"]
    flops = flops_per_token * toks
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))); src = "measured"
    except Exception:
        peaks = {"bf16_tflops_sustained": 1400.0}; src = "fallback"
    tf = flops / (ms * 1e-3) / 1e12
    peak = peaks.get("bf16_tflops_sustained", 1400.0) * world
    return {
        "metric": "retnet_stack_train_tokens_per_s", "value": toks / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "loss": last,
        "config": {"workload": f"RetNet stack train step: {c['layers']} layers, d_model {c['heads'] * c['head_dim']}, {c['heads']} heads, "
                               f"FFN {c['ffn']}, vocab {c['vocab']}, global batch {c['B']} x {c['T']}, micro-batch {mb}, "
                               f"DDP over {world} GPU(s), AdamW", "l2": "activations far larger than L2"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                     "peak_source": src + " (sustained cuBLAS bf16)", "traffic": None,
                     "note": "whole step, cuBLAS GEMMs dominate; retention kernels are about 2 % of the FLOPs"},
        "e2e": {"value": toks / (ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": host_tokens.numel() * 8, "d2h_bytes_per_step": 4,
                "note": "the timed step already copies its token ids from pinned host memory and reads the loss back"},
        "clocks": clocks, "gpu_launches": launches}


def run_stack(args):
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the full-stack configuration has no CPU-sized reference run; "
                              "the reference arm covers the operator workloads"}))
        return
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rec = stack_record(args, dev, rank, world, args.steps, args.warmup)
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the kernels as captured with ncu.  "ns" and
# "c3" were captured on a reduced batch (5 of 8 and 2 of 4 rows: same kernels, launches not under-filled) and are scaled to
# the full launch by the token-heads processed - traffic grows in proportion, every CTA streams its own sequence once.
def _traffic(read_b, write_b, scale, what):
    return {"bytes": (read_b + write_b) * scale, "source": what}


NCU_TRAFFIC = {
    ("ns", "fwd"): _traffic(503399936, 145707776, 8 / 5, "ncu at B=5, scaled x8/5 by token-heads"),
    ("ns", "dq"): _traffic(503390720, 146074624, 8 / 5, "ncu at B=5, scaled x8/5 by token-heads"),
    ("ns", "rev"): _traffic(671247104, 304547328, 8 / 5, "ncu at B=5, scaled x8/5 by token-heads"),
    ("c3", "fwd"): _traffic(1073861888, 506872064, 2, "ncu at B=2, scaled x2 by token-heads"),
    ("c3", "dq"): _traffic(20992 + 1610695168, 211433984 + 253492736, 2,
                           "ncu at B=2 (zero fill of dQ and the dQ walk over the two halves of dv), scaled x2 by token-heads"),
    ("c3", "rev"): _traffic(21248 + 1914728704, 211275776 + 790550272, 2,
                            "ncu at B=2 (zero fill of dK and the fused reverse walk over the two halves of dv), scaled x2 by token-heads"),
    ("c4", "fwd"): _traffic(251772416, 112364800, 1, "ncu at the full workload"),
    ("c4", "dq"): _traffic(251708672, 60882944, 1, "ncu at the full workload"),
    ("c4", "rev"): _traffic(402802432, 141126400, 1, "ncu at the full workload (block-state gradients read)"),
}


# --------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="ns", choices=sorted(WORKLOADS) + ["c5", "decode", "layer"])
    ap.add_argument("--micro-batch", type=int, default=0, help="c5 only: rows per micro-batch (0 = the workload's default)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="leave out the sub-records of the default line (the same problem split over the ranks; the full-stack step)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.workload == "c5":
        return run_stack(args)
    if args.workload == "decode":
        return run_decode(args)
    if args.workload == "layer":
        return run_layer_passes(args)
    w = WORKLOADS[args.workload]

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, w, rank)
        return

    import torch.distributed as dist
    import flash_pop_b200 as fp
    from flash_pop_b200 import _lib
    from flash_pop_b200.parallel import partition
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    B, H, T, dk, dv = w["B"], w["H"], w["T"], w["dk"], w["dv"]
    dec = decays_for(H)
    from flash_pop_b200.host_io import allocate_near
    with allocate_near(dev):                 # pinned host buffers in the memory of the GPU's own NUMA node
        hq, hk, hv, hdO = make_host_inputs(w, seed=2 + rank, pin=True)
    q, k, v, dO = (t.to(dev, non_blocking=True) for t in (hq, hk, hv, hdO))
    torch.cuda.synchronize()

    def op(q_, k_, v_, decays=dec):
        if w["block"]:
            return fp.flash_pop_retention(q_, k_, v_, None, decays, w["block"])[0]
        return fp.fused_chunk_retention(q_, k_, v_, None, decays)[0]

    # POP: in training the block states feed the prediction suffixes, so their gradient comes back into the backward of the
    # observation stream (added to the carried state gradient at every block end); the step has it, seeded like dO
    d_blocks = None
    if w["block"]:
        gb = torch.Generator(device=dev).manual_seed(70 + rank)
        d_blocks = (torch.randn(B, T // w["block"], H, dk, dv, generator=gb, device=dev) * 0.1).to(torch.bfloat16)

    def outputs_and_grads(q_, k_, v_):
        """What the backward starts from: (outputs that carry a gradient, those gradients)."""
        if w["block"]:
            o, blocks = fp.flash_pop_retention(q_, k_, v_, None, dec, w["block"])
            return (o, blocks), (dO, d_blocks)
        o = fp.fused_chunk_retention(q_, k_, v_, None, dec)[0]
        return (o,), (dO,)

    def step():
        ql, kl, vl = (t.detach().requires_grad_(True) for t in (q, k, v))
        outs, grads = outputs_and_grads(ql, kl, vl)
        torch.autograd.backward(outs, grads)
        return outs[0], ql.grad, kl.grad, vl.grad

    def fwd_only():
        with torch.no_grad():
            return op(q, k, v)

    for _ in range(args.warmup):
        step()
    _lib.device_status(dev)
    path = _lib.last_path()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    launches0 = _lib.launch_count()
    barrier()
    ms = event_time_ms(step, args.steps)
    barrier()
    launches = _lib.launch_count() - launches0
    clocks = sampler.stop() if sampler else None

    # per-launch device times for the roofline (same inputs, > L2, so no flush needed): the forward launch, and
    # the two backward walks singled out by asking for only dQ / only dK,dV (the operator skips the other walk)
    ms_fwd = event_time_ms(fwd_only, max(args.steps, 5))
    ms_bwd = max(ms - ms_fwd, 1e-6)

    def only_grads(of):
        leaves = [t.detach().requires_grad_(i in of) for i, t in enumerate((q, k, v))]
        outs, grads = outputs_and_grads(*leaves)
        wanted = [leaves[i] for i in of]
        return lambda: torch.autograd.grad(outs, wanted, grads, retain_graph=True)

    fn_dq, fn_rev = only_grads((0,)), only_grads((1, 2))
    fn_dq(); fn_rev()
    n0 = _lib.launch_count(); fn_dq(); launches_dq = _lib.launch_count() - n0
    n0 = _lib.launch_count(); fn_rev(); launches_rev = _lib.launch_count() - n0
    ms_dq = event_time_ms(fn_dq, max(args.steps, 5))
    ms_rev = event_time_ms(fn_rev, max(args.steps, 5))

    # end to end: host (pinned) -> device, forward+backward, every result back to the host
    e2e_ms = copy_only_ms = None
    h2d = sum(t.numel() * 2 for t in (hq, hk, hv, hdO))
    d2h = (2 * hq.numel() + 2 * hv.numel()) * 2
    if not args.no_e2e:
        with allocate_near(dev):
            outs_host = [torch.empty_like(hv).pin_memory(), torch.empty_like(hq).pin_memory(),
                         torch.empty_like(hk).pin_memory(), torch.empty_like(hv).pin_memory()]
        # the package's host-memory helper: slices (batch rows x head groups; whole rows for POP), copies in / kernels /
        # copies out on three streams
        from flash_pop_b200.host_io import HostRetentionPipeline
        pipe = HostRetentionPipeline(hq, hv, dev, block_size=w["block"] or 0)

        def e2e_step(copy_only=False):
            pipe.run(hq, hk, hv, hdO, dec, *outs_host, copy_only=copy_only)

        e2e_step()
        barrier()
        # The host link is shared with whatever else runs on the box, and a burst of foreign traffic during a handful
        # of steps once doubled one figure and not the other.  So: three rounds of (the step, then the same buffers,
        # slices and streams without the kernels - what the host link alone allows), the median round of each.
        n_e2e = max(3, min(args.steps, 5))
        rounds = []
        for _ in range(3):
            t_step = event_time_ms(e2e_step, n_e2e)
            barrier()
            t_copy = event_time_ms(lambda: e2e_step(True), n_e2e)
            barrier()
            rounds.append((t_step, t_copy))
        e2e_ms = sorted(r[0] for r in rounds)[1]
        copy_only_ms = sorted(r[1] for r in rounds)[1]
        del outs_host

    # POP only: the prediction-token suffixes (one per block, 80 tokens each) run from the block states in place
    suffix = None
    if w["block"]:
        N, P = T // w["block"], w["block"]
        gs = torch.Generator().manual_seed(40 + rank)
        sq, sk, sv = ((torch.randn(B, N, P, H, d_, generator=gs) * dk ** -0.5).to(torch.bfloat16).to(dev) for d_ in (dk, dk, dv))
        sdo = torch.randn(B, N, P, H, dv, generator=gs).to(torch.bfloat16).to(dev)
        with torch.no_grad():
            blocks = fp.flash_pop_retention(q, k, v, None, dec, w["block"])[1]

        def suffix_step():
            leaves = [t.detach().requires_grad_(True) for t in (sq, sk, sv)]
            bs = blocks.detach().requires_grad_(True)
            so = fp.pop_suffix_retention(*leaves, None, bs, dec)
            so.backward(sdo)

        def suffix_fwd():
            with torch.no_grad():
                fp.pop_suffix_retention(sq, sk, sv, None, blocks, dec)
        for _ in range(3):
            suffix_step()
        s_ms, s_fwd = event_time_ms(suffix_step, args.steps), event_time_ms(suffix_fwd, args.steps)
        s_units = B * N * P * H
        s_bytes = (bf_ := bytes_per_token_head(dk, dv))[0] * s_units + bf_[1] * s_units
        s_state_bytes = 2 * B * N * H * dk * dv * 2          # start states read, their gradients written
        suffix = {"ms_fwd_bwd": s_ms, "ms_fwd": s_fwd, "suffixes": B * N, "tokens_each": P,
                  "hbm_gbs_algorithmic": (s_bytes + s_state_bytes) / (s_ms * 1e-3) / 1e9,
                  "algorithmic_bytes": s_bytes + s_state_bytes,
                  "note": "start states read in place from block_states; state gradients written back to d_block_states"}
        del sq, sk, sv, sdo, blocks

    # The same problem split over the ranks (strong scaling): every rank takes its piece of ONE B-row problem (seed 2,
    # the rows of rank 0's own tensors) with flash_pop_b200.parallel.partition; no data crosses between GPUs.  Each
    # piece is an under-filled launch, which the operator cuts into T-segments.
    strong = None
    if not args.no_extras and not w["block"]:
        sh = partition(B, H, rank, world)
        rows = range(sh.batch.start, sh.batch.stop)
        if rank == 0:
            piece = [t[sh.batch, :, sh.heads] for t in (q, k, v, dO)]
        elif len(rows):
            piece = [t.to(dev)[:, :, sh.heads] for t in make_host_inputs(w, seed=2, pin=False, rows=rows)]
        else:
            piece = None
        ms_strong = 0.0
        n_strong = 0
        if piece is not None and piece[0].numel():
            pq, pk, pv, pdo = piece
            pdec = sh.take_decays(dec)

            def strong_step():
                leaves = [t.detach().requires_grad_(True) for t in (pq, pk, pv)]
                o = op(*leaves, decays=pdec)
                o.backward(pdo)
            for _ in range(3):
                strong_step()
            n0 = _lib.launch_count(); strong_step(); n_strong = _lib.launch_count() - n0
            barrier()
            ms_strong_eager = event_time_ms(strong_step, args.steps)
            try:        # the pieces' kernels take tens of microseconds: replay them from a CUDA graph as a training loop would
                ms_strong = graph_time_ms(strong_step, args.steps)
            except Exception:
                ms_strong = ms_strong_eager
        else:
            barrier()
            ms_strong_eager = 0.0
        barrier()
        strong = (ms_strong, n_strong, ms_strong_eager)
        del piece

    # the copy bandwidth of THIS GPU right now (read + write of a 1 GiB device-to-device copy): boxes of the pool differ,
    # and the kernel closest to the HBM roof follows it
    src_buf = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    dst_buf = torch.empty_like(src_buf)
    for _ in range(3):
        dst_buf.copy_(src_buf)
    copy_gbs = 2 * src_buf.numel() / (event_time_ms(lambda: dst_buf.copy_(src_buf), 10) * 1e-3) / 1e9
    del src_buf, dst_buf

    t_ms = torch.tensor([ms, ms_fwd, ms_bwd, e2e_ms or 0.0, ms_dq, ms_rev, copy_only_ms or 0.0, strong[0] if strong else 0.0,
                         strong[2] if strong else 0.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    ms, ms_fwd, ms_bwd, e2e_max, ms_dq, ms_rev, copy_max, strong_max, strong_eager_max = t_ms.tolist()
    _lib.device_status(dev)

    # the full-stack training step (12 layers, DDP over the ranks, NCCL gradient all-reduce), a few steps
    c5 = None
    if not args.no_extras and args.workload == "ns":
        import gc
        del q, k, v, dO, hq, hk, hv, hdO, fn_dq, fn_rev      # (and what they keep alive: graphs holding the inputs)
        gc.collect()
        torch.cuda.empty_cache()
        c5 = stack_record(args, dev, rank, world, steps=3, warmup=2, sample_clocks=True)

    if rank == 0:
        ff, fb = flops_per_token_head(dk, dv)
        bf, bb = bytes_per_token_head(dk, dv)
        units = B * T * H                       # token-heads per GPU per step
        total_flop = (ff + fb) * units * world
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
            peak_src = "measured"
        except Exception:
            peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
            peak_src = "fallback"
        value = total_flop / (ms * 1e-3) / 1e12
        pop_state = (2 * dk * dv * 2 * H * B * (T // w["block"])) if w["block"] else 0     # block states written / their gradients read
        # the launches of a step with their algorithmic bytes: forward (read q,k,v; write o), the dQ walk (read dO,k,v; write
        # dQ), the reverse walk(s) (read q,k,v,dO; write dK,dV) - one fused launch, or two launches where dv = 256
        # (dk, dv up to 128: one fused launch, three when cut into T-segments; dk = 128 beside dv = 256 without POP blocks:
        # the fused kernel over the two halves of dv after a zero fill of dK; otherwise two reverse walks)
        fused = max(dk, dv) <= 128 or (dk == 128 and dv == 256 and not w["block"])
        kernels = {
            "fwd": {"kernel": "scan_kernel<MODE_FWD, forward>", "ms": ms_fwd, "bytes": bf * units + pop_state // 2},
            "dq": {"kernel": "scan_kernel<MODE_DQ, forward> (dQ walk)", "ms": ms_dq, "bytes": 2 * (dk + 2 * dv + dk) * units,
                   "launches": launches_dq},
            "rev": {"kernel": "bwd_fused_kernel (reverse walk: dK, dV, dS0)" if fused else
                              "scan_kernel reverse walks (dV + dS0, then dK): two launches timed together",
                    "ms": ms_rev, "bytes": 2 * (2 * dk + 2 * dv) * units + 2 * (dk + dv) * units + pop_state // 2,
                    "launches": launches_rev},
        }

        def roof(key):
            kk = kernels[key]
            gbs = kk["bytes"] / (kk["ms"] * 1e-3) / 1e9
            tr = NCU_TRAFFIC.get((args.workload, key))
            out = {"bound": "hbm", "kernel": kk["kernel"], "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                   "frac": gbs / peaks["hbm_gbs"], "peak_source": peak_src, "algorithmic_bytes": kk["bytes"], "ms_per_launch": kk["ms"],
                   "traffic": tr["bytes"] if tr else None,
                   "traffic_source": tr["source"] if tr else "no ncu capture of this kernel at this workload"}
            if "launches" in kk:
                out["launches"] = kk["launches"]
            return out

        top = max(kernels, key=lambda name: kernels[name]["ms"])       # the launch with the largest share of the step
        step_gbs = (bf + bb) * units / (ms * 1e-3) / 1e9
        line = {
            "metric": "chunked_retention_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "tokens_per_s": B * T * world / (ms * 1e-3),
            "pct_bf16_peak_nominal": 100 * value / world / 2250.0,
            "pct_bf16_peak_measured": 100 * value / world / peaks.get("bf16_tflops", 1590.0),
            "hbm_gbs_algorithmic": (bf + bb) * units / (ms * 1e-3) / 1e9,
            "ms_fwd": ms_fwd, "ms_bwd": ms_bwd, "ms_bwd_dq": ms_dq, "ms_bwd_dkdv": ms_rev,
            "path": {1: "cuda-core", 2: "tcgen05"}.get(path, "none"),
            "config": op_config(args, w),
            "roofline": dict(roof(top), copy_gbs_this_gpu=copy_gbs, frac_of_copy_here=roof(top)["achieved"] / copy_gbs),
            "roofline_fwd": roof("fwd"), "roofline_dq": roof("dq"), "roofline_rev": roof("rev"),
            "roofline_step": {"bound": "hbm", "kernels": "all launches of a step (forward, dQ walk, reverse walk)", "achieved": step_gbs,
                              "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": step_gbs / peaks["hbm_gbs"],
                              "algorithmic_bytes": (bf + bb) * units},
            "clocks": clocks,
            "gpu_launches": launches,
        }
        if suffix is not None:
            line["pop_suffixes"] = suffix
        if e2e_ms is not None:
            line["e2e"] = {"value": total_flop / (e2e_max * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_max,
                           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                           "copy_only_ms": copy_max, "frac_of_copy_only": copy_max / e2e_max,
                           "host_link_gbs_each_way": world * h2d / (copy_max * 1e-3) / 1e9,
                           "note": "copy_only_ms = the same pinned buffers, slices and streams with the kernels left out; both are the median of "
                                   "three alternating rounds of a few steps each"}
        if strong is not None:
            one_gpu_flop = (ff + fb) * units
            line["strong"] = {"what": f"ONE problem of B={B} rows (seed 2) split over {world} rank(s) by batch row, then by heads; "
                                      "no data exchange; under-filled pieces run as T-segments",
                              "ms_per_step": strong_max, "value": one_gpu_flop / (strong_max * 1e-3) / 1e12, "unit": "TFLOP/s",
                              "timing": "one step captured in a CUDA graph and replayed; ms_per_step_eager is the same step called "
                                        "from Python each time (the pieces' kernels are shorter than the call overhead)",
                              "ms_per_step_eager": strong_eager_max, "launches_per_step_rank0": strong[1],
                              "speedup_vs_one_gpu": ms / strong_max, "efficiency": ms / strong_max / world,
                              "one_gpu_ms": ms}
        if c5 is not None:
            line["c5"] = {kk: c5[kk] for kk in ("metric", "value", "unit", "ms_per_step", "steps", "warmup", "scaling", "loss", "config",
                                              "roofline", "clocks", "gpu_launches")}
        if not args.no_cpu_baseline and world == 1:
            threads = os.cpu_count() or 1
            passes = 3
            tf, dt = cpu_reference_tflops(w, 1, passes, 1, threads)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                    "sample": cpu_sample_text(w, 1, passes) + f", {dt:.2f} s per pass"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
