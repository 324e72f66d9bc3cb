"""The allocation-free SSD entry point (bm_ssd2_fwd_noalloc), collected last on purpose.

Some users of the library cannot hand it a workspace: their process has a device-memory budget that
is carved up once at start-up, or they sit behind a framework that passes them raw tensor pointers and
keeps its allocator to itself.  For them the library carries its own scratch array.  These tests call
the entry point through the C ABI and hold it to the same results as bm_ssd2_fwd, twice in a row,
because the scratch is shared between calls and keeps whatever the previous call left in it.
"""
import ctypes as C

import numpy as np
import pytest
import torch


def _inputs(seed, b, s, h, p, r, g, with_host=False):
    from oracle import inputs
    cfg = inputs.ssd2_prefill(seed=seed, batch=b, seqlen=s, nheads=h, headdim=p, state_rank=r, ngroups=g, h0_std=0.1)
    t = {k: torch.from_numpy(np.ascontiguousarray(v)).cuda() for k, v in cfg.items()}
    return (t, cfg) if with_host else t


@pytest.mark.gpu
def test_noalloc_matches_workspace_entry_point_on_two_calls_in_a_row(bm):
    from oracle.numerics import rel_l2
    # two different problems back to back: the second must not see anything of the first in the scratch
    cases = [(3, 2, 200, 4, 32, 64, 2, 64), (4, 1, 130, 8, 64, 64, 1, 32)]
    for seed, b, s, h, p, r, g, q in cases:
        t, cfg = _inputs(seed, b, s, h, p, r, g, with_host=True)
        want_y, want_h = bm.ops.ssd2_fwd(t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], t["h0"], chunk_len=q,
                                         path="exact")
        before = torch.cuda.memory_allocated()
        y, hf = bm.ops.ssd2_fwd_noalloc(t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], t["h0"], chunk_len=q)
        torch.cuda.synchronize()
        # the wrapper allocates exactly the two outputs and nothing else (no workspace tensor)
        assert torch.cuda.memory_allocated() - before <= y.numel() * y.element_size() + hf.numel() * 4 + 1024
        assert rel_l2(y.cpu().numpy(), want_y.cpu().numpy()) <= 1e-4
        assert rel_l2(hf.cpu().numpy(), want_h.cpu().numpy()) <= 1e-4
        # and to the CPU oracle directly, so that this test stands without the other entry point
        from oracle import mamba2
        ref_y, ref_h = mamba2.ssd_serial(cfg["x"], cfg["dt"], cfg["a"], cfg["b"], cfg["c"], cfg["d"], cfg["h0"], q)
        assert rel_l2(y.cpu().numpy(), ref_y) <= 1e-4 and rel_l2(hf.cpu().numpy(), ref_h) <= 1e-4
    # and the same problem twice in a row gives the same answer both times
    t = _inputs(5, 2, 96, 4, 16, 16, 1)
    y1, h1 = bm.ops.ssd2_fwd_noalloc(t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], t["h0"], chunk_len=32)
    y2, h2 = bm.ops.ssd2_fwd_noalloc(t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], t["h0"], chunk_len=32)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2) and torch.equal(h1, h2)


def test_noalloc_refuses_what_does_not_fit_and_the_tensor_path(bm):
    """Pure host checks: the size limit and the path restriction are enforced before any launch."""
    f = bm._ffi
    # 8 x 4096 x 80 heads at P 64, N 128 needs hundreds of MB of chunk states: far beyond the built-in scratch
    a = f.Ssd2FwdArgs(batch=8, seqlen=4096, nheads=80, headdim=64, state_rank=128, ngroups=1, chunk_len=256,
                      dtype=f.BM_DTYPE_F32, path=f.BM_PATH_EXACT)
    assert bm.lib.bm_ssd2_fwd_workspace_bytes(C.byref(a)) > f.BM_SSD2_NOALLOC_SCRATCH_BYTES
    for name in ("x", "dt", "a", "b", "c", "y", "h_final"):
        setattr(a, name, 0x10000)  # never dereferenced: the call is refused on the host
    assert bm.lib.bm_ssd2_fwd_noalloc(C.byref(a), None) == f.BM_ERR_WORKSPACE_TOO_SMALL
    assert b"built-in scratch" in bm.lib.bm_last_error_string()
    a.batch, a.seqlen, a.nheads, a.path = 1, 128, 2, f.BM_PATH_TENSOR
    assert bm.lib.bm_ssd2_fwd_noalloc(C.byref(a), None) == f.BM_ERR_UNSUPPORTED
