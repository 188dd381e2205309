"""Register-spill guard for the hot kernels.  The 128 x 128 instances of the tcgen05 kernels run at their register
cap (512 threads per CTA); a handful of extra live values spills the fp32 state, which has cost the headline shape 31 %
once.  This compiles the two kernel files with ptxas' resource report (no GPU needed) and checks the spill bytes."""
import os
import re
import shutil
import subprocess

import pytest

from flash_pop_b200 import _lib

# (kernel, template arguments of the hot instance: bf16 states, full walk) -> max spill-store bytes
LIMITS = {
    ("bwd_fused_kernel", "128ELi128ELb0E"): 64,
    ("scan_kernel", "0ELi0ELi128ELi128ELb0ELb0E"): 64,          # forward
    ("scan_kernel", "1ELi0ELi128ELi128ELb0ELb0E"): 128,         # dQ (108 bytes of walk-invariant values: measured harmless)
    ("bwd_fused_kernel", "64ELi64ELb0E"): 0,
    ("scan_kernel", "0ELi0ELi64ELi64ELb0ELb0E"): 16,
    ("scan_kernel", "1ELi0ELi64ELi64ELb0ELb0E"): 16,
}


def test_hot_kernels_do_not_spill(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    report = ""
    for name in ("retention_scan_sm100.cu", "retention_bwd_fused_sm100.cu"):
        res = subprocess.run([nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-Xptxas=-v", "--threads", "0",
                              "-cubin", "-o", str(tmp_path / (name + ".cubin")), os.path.join(_lib.CSRC_DIR, name)],
                             capture_output=True, text=True)
        assert res.returncode == 0, res.stderr[-2000:]
        report += res.stderr
    found = {}
    current = None
    for line in report.splitlines():
        m = re.search(r"Compiling entry function '(\S+)'", line)
        if m:
            current = m.group(1)
        m = re.search(r"(\d+) bytes spill stores", line)
        if m and current:
            found[current] = int(m.group(1))
    for (kernel, args), limit in LIMITS.items():
        hits = [v for k, v in found.items() if kernel in k and ("ILi" + args) in k]
        assert hits, f"no instance of {kernel}<{args}> in the ptxas report"
        assert max(hits) <= limit, f"{kernel}<{args}> spills {max(hits)} bytes (limit {limit})"
