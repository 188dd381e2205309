"""Forward + backward of fused chunked retention for tensors that live in (pinned) HOST memory.

The operator itself works on device tensors.  When inputs and results have to cross PCIe every step, the copies
dominate (about 20 ms per GB and direction against under 1 ms of kernel time per GB), so this helper slices the
batch (and the heads) and runs three streams: slice i+1 is copied in while slice i is computed and slice i-1 is copied out.
Host-to-device and device-to-host copies then overlap each other (PCIe is full duplex) and the kernels.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from flash_pop_b200 import _lib
from flash_pop_b200.fused_retention import retention_forward_backward_into
from flash_pop_b200.pop_retention import pop_retention_forward_backward_into


class HostRetentionPipeline:
    """Reusable device staging buffers and streams for `run`.  All host tensors should be pinned.

    A slice is a group of batch rows and, when the batch alone gives too few slices to hide the pipeline's fill and
    drain (the first slice's copy in and the last one's copy out overlap nothing: one slice in nine at B = 8), a group of
    heads of those rows.  A head group of a contiguous (B, T, H, d) tensor is strided; it crosses PCIe as ONE
    two-dimensional copy (`fpb_copy_rows_async`), which runs at the link rate where a tensor-wise strided copy reaches a
    quarter of it, and the operator takes the strided views as they are."""

    TARGET_SLICES = 32

    def __init__(self, like_q: torch.Tensor, like_v: torch.Tensor, device, slices: Optional[int] = None,
                 head_groups: Optional[int] = None, block_size: int = 0):
        """block_size > 0: POP retention with blocks of that many tokens (the block states of a slice stay on the device
        in `self.block_states`; they are contiguous over all heads, so POP slices are whole batch rows)."""
        B, T, H, dk = like_q.shape
        row_slices = min(B, slices or B)
        self.block_size = int(block_size)
        if self.block_size > 0:
            if head_groups not in (None, 1):
                raise ValueError("POP slices are whole batch rows")
            head_groups = 1
        if head_groups is None:
            # the largest divisor of H that keeps the slice count at or below the target
            head_groups = max(g for g in range(1, H + 1) if H % g == 0 and (g == 1 or row_slices * g <= self.TARGET_SLICES))
        if H % head_groups:
            raise ValueError(f"{head_groups} head groups do not divide {H} heads")
        per = H // head_groups
        rows = [(B * i // row_slices, B * (i + 1) // row_slices) for i in range(row_slices)]
        self.parts = [(a, b, g * per, (g + 1) * per) for a, b in rows for g in range(head_groups)]
        self.slices = len(self.parts)
        self.device = torch.device(device)
        mk = lambda t: torch.empty(t.shape, dtype=t.dtype, device=self.device)
        self.q, self.k, self.dq, self.dk = mk(like_q), mk(like_q), mk(like_q), mk(like_q)
        self.v, self.do, self.o, self.dv = mk(like_v), mk(like_v), mk(like_v), mk(like_v)
        self.block_states = None
        if self.block_size > 0:
            rows_max = max(b - a for a, b, _, _ in self.parts)
            self.block_states = torch.empty((rows_max, T // self.block_size, H, dk, like_v.shape[-1]), dtype=like_q.dtype,
                                            device=self.device)
        self.s_in, self.s_comp, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))

    def _copy(self, dst: torch.Tensor, src: torch.Tensor, a: int, b: int, h0: int, h1: int) -> None:
        """dst[a:b, :, h0:h1] <- src[a:b, :, h0:h1] on the current stream (same shape and layout on both sides)."""
        B, T, H, d = src.shape
        if (h0, h1) == (0, H) or not (src.is_contiguous() and dst.is_contiguous()):
            dst[a:b, :, h0:h1].copy_(src[a:b, :, h0:h1], non_blocking=True)
            return
        item = src.element_size()
        pitch, offset = H * d * item, (a * T * H + h0) * d * item
        _lib.check(_lib.lib().fpb_copy_rows_async(ctypes.c_void_p(dst.data_ptr() + offset), pitch,
                                                  ctypes.c_void_p(src.data_ptr() + offset), pitch, (h1 - h0) * d * item,
                                                  (b - a) * T, _lib.stream_ptr(self.device)))

    def run(self, hq, hk, hv, hdo, head_decays: Sequence[float], ho, hdq, hdk, hdv, copy_only: bool = False) -> None:
        """Reads hq, hk, hv, hdo (host), writes ho, hdq, hdk, hdv (host).  Returns when everything has been queued
        and the calling stream has been made to wait for it.  The kernels write their results straight into the
        staging buffers (the C ABI takes output pointers), so a slice costs its two PCIe crossings and nothing else.
        `copy_only` queues the same copies on the same streams without the kernels: what the host link alone allows."""
        head_decays = tuple(float(g) for g in head_decays)
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(cur)
        with torch.cuda.device(self.device):
            for a, b, h0, h1 in self.parts:
                with torch.cuda.stream(self.s_in):
                    for dst, src in ((self.q, hq), (self.k, hk), (self.v, hv), (self.do, hdo)):
                        self._copy(dst, src, a, b, h0, h1)
                    landed = self.s_in.record_event()
                with torch.cuda.stream(self.s_comp):
                    self.s_comp.wait_event(landed)
                    if not copy_only:
                        part = lambda t: t[a:b, :, h0:h1]
                        if self.block_size > 0:
                            pop_retention_forward_backward_into(part(self.q), part(self.k), part(self.v), part(self.do), head_decays,
                                                                self.block_size, part(self.o), self.block_states[:b - a],
                                                                part(self.dq), part(self.dk), part(self.dv))
                        else:
                            retention_forward_backward_into(part(self.q), part(self.k), part(self.v), part(self.do), head_decays[h0:h1],
                                                            part(self.o), part(self.dq), part(self.dk), part(self.dv))
                    done = self.s_comp.record_event()
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(done)
                    for dst, src in ((ho, self.o), (hdq, self.dq), (hdk, self.dk), (hdv, self.dv)):
                        self._copy(dst, src, a, b, h0, h1)
        cur.wait_stream(self.s_out)


def _parse_cpulist(text: str) -> set:
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


class allocate_near:
    """Context manager: while it is open, the calling thread runs on the CPUs that sit next to `device` (the PCI
    device's ``local_cpulist`` in sysfs), so host buffers allocated and pinned inside land in that NUMA node's memory
    and copies to the GPU do not cross the socket interconnect.  Does nothing where the topology cannot be read."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.saved = None

    def __enter__(self):
        try:
            import os
            p = torch.cuda.get_device_properties(self.device)
            bus = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
            with open(f"/sys/bus/pci/devices/{bus}/local_cpulist") as f:
                near = _parse_cpulist(f.read())
            allowed = os.sched_getaffinity(0)
            if near & allowed and (near & allowed) != allowed:
                self.saved = allowed
                os.sched_setaffinity(0, near & allowed)
        except Exception:
            self.saved = None
        return self

    def __exit__(self, *exc):
        if self.saved is not None:
            import os
            os.sched_setaffinity(0, self.saved)
        return False
