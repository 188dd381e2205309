"""The shared library loads without a GPU and exports every entry point the header declares; the
argument checks that need no device answer with the documented codes."""
import ctypes
import os
import re

import pytest

from flash_pop_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def handle():
    _lib.build()
    return _lib.lib()


def test_every_declared_symbol_is_exported(handle):
    header = open(os.path.join(ROOT, "include", "flash_pop_b200.h")).read()
    declared = set(re.findall(r"^(?:int|int64_t|const char\*)\s+(fpb_[a-z0-9_]+)\s*\(", header, re.M))
    assert declared, "no declarations found"
    assert declared == set(_lib.exported_symbols())
    for name in declared:
        assert hasattr(handle, name), name


def test_version_and_strerror(handle):
    assert handle.fpb_version() >= 100
    assert handle.fpb_strerror(0) == b"ok"
    assert b"dtype" in handle.fpb_strerror(3)
    assert handle.fpb_launch_count() == 0 or handle.fpb_launch_count() > 0


def _dims(**kw):
    decays = (ctypes.c_double * 4)(0.9, 0.9, 0.9, 0.9)
    base = dict(dtype=0, B=1, T=8, H=4, dk=64, dv=64, block_size=0, flags=0)
    base.update(kw)
    d = _lib._Dims(base["dtype"], base["B"], base["T"], base["H"], base["dk"], base["dv"], base["block_size"],
                   base["flags"], ctypes.cast(decays, ctypes.POINTER(ctypes.c_double)))
    d._keep = decays
    return d


def test_argument_checks_return_codes_without_a_device(handle):
    seq = _lib._Seq(None, 0, 0, 0)
    st = _lib._State(None, 0, 0)
    call = lambda d: handle.fpb_retention_fwd(d, seq, seq, seq, st, seq, st, None)
    assert call(_dims(dtype=7)) == 3
    assert call(_dims(dk=0)) == 2
    assert call(_dims(dk=512)) == 2
    assert call(_dims(H=1000)) == 2
    assert call(_dims()) == 1                       # null data pointers with a non-empty problem
    assert handle.fpb_pop_retention_fwd(_dims(block_size=0), seq, seq, seq, st, seq, None, None) == 6
    bad = _dims()
    bad._keep[1] = 1.5
    assert call(bad) == 5
    assert handle.fpb_retention_fwd(None, seq, seq, seq, st, seq, st, None) == 1


def test_operators_refuse_cpu_tensors():
    import torch
    import flash_pop_b200 as fp
    q = torch.randn(1, 8, 2, 16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fp.fused_chunk_retention(q, q, q, None, (0.9, 0.9))
    with pytest.raises(RuntimeError, match="no CPU path"):
        fp.flash_pop_retention(q, q, q, None, (0.9, 0.9), 4)


def test_layer_pass_and_step_entry_points_check_arguments_without_a_device(handle):
    seq = _lib._Seq(None, 0, 0, 0)
    st = _lib._State(None, 0, 0)
    # rotation: d must be a multiple of 8, dtypes known, phasors given
    assert handle.fpb_rotary(1, 4, 2, 12, 0, 0, 0, None, 0, seq, seq, seq, seq, None) == 2
    assert handle.fpb_rotary(1, 4, 2, 16, 5, 0, 0, None, 0, seq, seq, seq, seq, None) == 3
    assert handle.fpb_rotary(1, 4, 2, 16, 0, 0, 0, None, 0, seq, seq, seq, seq, None) == 1
    # GroupNorm-gate: even width up to 256
    assert handle.fpb_groupnorm_gate_fwd(1, 4, 2, 7, 0, 1e-6, 1, seq, seq, seq, None) == 2
    assert handle.fpb_groupnorm_gate_fwd(1, 4, 2, 512, 0, 1e-6, 1, seq, seq, seq, None) == 2
    assert handle.fpb_groupnorm_gate_bwd(1, 4, 2, 64, 9, 1e-6, 1, seq, seq, seq, seq, seq, None) == 3
    assert handle.fpb_groupnorm_gate_fwd(1, 4, 2, 64, 0, 1e-6, 1, seq, seq, seq, None) == 1
    # LayerNorm: width a multiple of 8 (bf16) and at most 1024
    assert handle.fpb_layernorm_fwd(8, 12, 0, 1e-6, None, 12, None, None, None, 12, None) == 2
    assert handle.fpb_layernorm_fwd(8, 2048, 0, 1e-6, None, 2048, None, None, None, 2048, None) == 2
    assert handle.fpb_layernorm_fwd(8, 64, 0, 1e-6, None, 64, None, None, None, 64, None) == 1
    assert handle.fpb_layernorm_bwd(8, 64, 3, 1e-6, None, 64, None, None, 64, None, None, None, None) == 3
    # two-dimensional copy: nothing to do is fine, pointers and pitches are checked before anything is queued
    assert handle.fpb_copy_rows_async(None, 64, None, 64, 32, 0, None) == 0
    assert handle.fpb_copy_rows_async(None, 64, None, 64, 32, 4, None) == 1
    assert handle.fpb_copy_rows_async(0x1000, 16, 0x2000, 64, 32, 4, None) == 4
    # decoding step: one token per row
    assert handle.fpb_retention_step(_dims(T=2), 0, seq, seq, seq, st, seq, st, None) == 2
    assert handle.fpb_retention_step(_dims(T=1), 4, seq, seq, seq, st, seq, st, None) == 3
    assert handle.fpb_retention_step(_dims(T=1), 0, seq, seq, seq, st, seq, st, None) == 1


def test_cpu_list_parser_of_the_numa_helper():
    from flash_pop_b200.host_io import _parse_cpulist
    assert _parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert _parse_cpulist("") == set()
