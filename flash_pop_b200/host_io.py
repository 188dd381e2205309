"""Forward + backward of fused chunked retention for tensors that live in (pinned) HOST memory.

The operator itself works on device tensors.  When inputs and results have to cross PCIe every step, the copies
dominate (about 20 ms per GB and direction against under 1 ms of kernel time per GB), so this helper slices the
batch and runs three streams: slice i+1 is copied in while slice i is computed and slice i-1 is copied out.
Host-to-device and device-to-host copies then overlap each other (PCIe is full duplex) and the kernels.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from flash_pop_b200.fused_retention import retention_forward_backward_into


class HostRetentionPipeline:
    """Reusable device staging buffers and streams for `run`.  All host tensors should be pinned."""

    def __init__(self, like_q: torch.Tensor, like_v: torch.Tensor, device, slices: Optional[int] = None):
        B = like_q.shape[0]
        self.slices = min(B, slices or B)
        self.rows = [(B * i // self.slices, B * (i + 1) // self.slices) for i in range(self.slices)]
        self.device = torch.device(device)
        mk = lambda t: torch.empty(t.shape, dtype=t.dtype, device=self.device)
        self.q, self.k, self.dq, self.dk = mk(like_q), mk(like_q), mk(like_q), mk(like_q)
        self.v, self.do, self.o, self.dv = mk(like_v), mk(like_v), mk(like_v), mk(like_v)
        self.s_in, self.s_comp, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))

    def run(self, hq, hk, hv, hdo, head_decays: Sequence[float], ho, hdq, hdk, hdv, copy_only: bool = False) -> None:
        """Reads hq, hk, hv, hdo (host), writes ho, hdq, hdk, hdv (host).  Returns when everything has been queued
        and the calling stream has been made to wait for it.  The kernels write their results straight into the
        staging buffers (the C ABI takes output pointers), so a slice costs its two PCIe crossings and nothing else.
        `copy_only` queues the same copies on the same streams without the kernels: what the host link alone allows."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(cur)
        for a, b in self.rows:
            with torch.cuda.stream(self.s_in):
                for dst, src in ((self.q, hq), (self.k, hk), (self.v, hv), (self.do, hdo)):
                    dst[a:b].copy_(src[a:b], non_blocking=True)
                landed = self.s_in.record_event()
            with torch.cuda.stream(self.s_comp):
                self.s_comp.wait_event(landed)
                if not copy_only:
                    retention_forward_backward_into(self.q[a:b], self.k[a:b], self.v[a:b], self.do[a:b], head_decays,
                                                    self.o[a:b], self.dq[a:b], self.dk[a:b], self.dv[a:b])
                done = self.s_comp.record_event()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for dst, src in ((ho, self.o), (hdq, self.dq), (hdk, self.dk), (hdv, self.dv)):
                    dst[a:b].copy_(src[a:b], non_blocking=True)
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
