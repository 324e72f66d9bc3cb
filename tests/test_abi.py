"""CPU tests of the C-ABI surface: the library loads, exports every symbol the header declares, and
the host-side validators reject bad arguments before touching a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    text = open(os.path.join(ROOT, "include", "bm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bm_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(bm):
    names = header_functions()
    assert len(names) >= 14
    raw = C.CDLL(bm._ffi.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/bm_b200.h but not exported"
    assert set(names) == set(bm._ffi.SYMBOLS), "ctypes table and header disagree"


def test_version_and_error_string(bm):
    assert bm.lib.bm_version() >= 1
    assert b"sm_100a" in bm.lib.bm_build_info()
    assert bm.lib.bm_ssd2_fwd(None, None, 0, None) == bm._ffi.BM_ERR_NULL_POINTER
    assert b"NULL" in bm.lib.bm_last_error_string()


def test_validators_reject_before_any_launch(bm):
    f = bm._ffi
    a = f.Ssd2FwdArgs(batch=1, seqlen=8, nheads=4, headdim=8, state_rank=8, ngroups=3, chunk_len=4, dtype=0, path=0)
    assert bm.lib.bm_ssd2_fwd(C.byref(a), None, 0, None) == f.BM_ERR_BAD_SHAPE  # nheads % ngroups
    a.ngroups = 1
    a.chunk_len = 0
    assert bm.lib.bm_ssd2_fwd(C.byref(a), None, 0, None) == f.BM_ERR_BAD_SHAPE
    a.chunk_len = 4
    a.seqlen = 0  # "sequence length must be at least 1" (src/mamba2/ssd/serial_recalculated/serial_recalculated.rs:39)
    assert bm.lib.bm_ssd2_fwd(C.byref(a), None, 0, None) == f.BM_ERR_BAD_SHAPE
    a.seqlen = 8
    assert bm.lib.bm_ssd2_fwd(C.byref(a), None, 0, None) == f.BM_ERR_NULL_POINTER
    a.x = 0x1008  # misaligned
    assert bm.lib.bm_ssd2_fwd(C.byref(a), None, 0, None) == f.BM_ERR_BAD_ALIGNMENT
    s = f.Step2Args(batch=1, nheads=2, headdim=4, state_rank=4, ngroups=1, dtype=7)
    assert bm.lib.bm_step2(C.byref(s), None) == f.BM_ERR_UNSUPPORTED
    m = f.Step3Args(batch=1, nheads=1, headdim=4, state_rank=8, mimo_rank=9, rope_dim=8)
    assert bm.lib.bm_step3(C.byref(m), None) == f.BM_ERR_UNSUPPORTED


def test_workspace_bytes_is_pure_host(bm):
    f = bm._ffi
    a = f.Ssd2FwdArgs(batch=2, seqlen=100, nheads=4, headdim=8, state_rank=16, ngroups=1, chunk_len=32, dtype=0,
                      path=f.BM_PATH_EXACT)
    n = bm.lib.bm_ssd2_fwd_workspace_bytes(C.byref(a))
    nchunks = 4
    assert n >= 2 * 2 * 4 * nchunks * 32 * 4 + 2 * nchunks * 4 * 8 * 16 * 4
    a.chunk_states = 0x1000  # caller-provided chunk-state buffer: workspace shrinks
    assert bm.lib.bm_ssd2_fwd_workspace_bytes(C.byref(a)) < n


def test_ops_refuse_cpu_tensors(bm):
    import torch
    x = torch.zeros(1, 4, 2, 8)
    with pytest.raises(ValueError, match="CUDA"):
        bm.ops.ssd2_fwd(x, torch.zeros(1, 4, 2), torch.zeros(2), torch.zeros(1, 4, 1, 8), torch.zeros(1, 4, 1, 8))
