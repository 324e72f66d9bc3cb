"""GPU parity at the shapes the benchmark configurations name (not just at their head shapes).

Sizes are cut only along axes that are independent in the algorithm (batch rows, heads), never along
the sequence: long sequences are where bf16 operand rounding of the carried state could drift.
Tolerances as everywhere: rel-L2 2e-2 for bfloat16 activations, 1e-4 for float32; gradients of the
bf16 runs are held to 2e-2 as well (the reference's own gradient tolerance is 1e-3 max-abs in float32 at
tiny shapes, which the float32 tests in test_gpu_parity.py keep).
"""
import numpy as np
import pytest
import torch

from oracle import backward, inputs, mamba1, mamba2, mamba3
from oracle.numerics import bf16_round, rel_l2, silu

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    return t.float().cpu().numpy()


# ------------------------------------------------------------------ Mamba-2 SSD prefill, 2.7B shape, L = 4096
def test_ssd2_tensor_path_full_sequence_matches_serial_oracle_and_float64_recurrence(bm):
    """P 64, N 128, G 1, Q 256, L 4096 with the prefill configuration's distributions: 32 tiles of carried
    state per head, against the chunked oracle and against the float64 token-by-token recurrence."""
    cfg = inputs.ssd2_prefill(seed=2, batch=1, seqlen=4096, nheads=4, headdim=64, state_rank=128, ngroups=1)
    x, b, c = (bf16_round(cfg[k]) for k in ("x", "b", "c"))
    want_y, want_h = mamba2.ssd_serial(x, cfg["dt"], cfg["a"], b, c, cfg["d"], cfg["h0"], 256)
    true_y, true_h = mamba2.ssd_recurrence(x, cfg["dt"], cfg["a"], b, c, cfg["d"], cfg["h0"])
    y, hf = bm.ops.ssd2_fwd(dev(x, BF), dev(cfg["dt"]), dev(cfg["a"]), dev(b, BF), dev(c, BF), dev(cfg["d"]), None,
                            chunk_len=256, path="tensor", check_status=True)
    assert rel_l2(host(y), want_y) <= 2e-2 and rel_l2(host(hf), want_h) <= 2e-2
    assert rel_l2(host(y), true_y) <= 2e-2 and rel_l2(host(hf), true_h) <= 2e-2
    # the last tile alone: drift would show here first
    assert rel_l2(host(y)[:, -128:], true_y[:, -128:]) <= 2e-2


def test_sequence_slices_from_folded_entering_states_equal_the_whole_sequence_bf16(bm):
    """The time-cut form of the prefill on one GPU: four slices of 1024 tokens run from zero, their maps folded into
    the entering states (shard.entering_state / slice_decay), each slice run again from its state; y and the final
    state against the single call over all 4096 tokens (tensor path, P 64, N 128, Q 256)."""
    cfg = inputs.ssd2_prefill(seed=17, batch=2, seqlen=4096, nheads=4, headdim=64, state_rank=128, ngroups=1, h0_std=0.2)
    x, b, c = (dev(bf16_round(cfg[k]), BF) for k in ("x", "b", "c"))
    dt, a, d, h0 = dev(cfg["dt"]), dev(cfg["a"]), dev(cfg["d"]), dev(cfg["h0"])
    fwd = lambda *t: bm.ops.ssd2_fwd(*t, chunk_len=256, path="tensor", check_status=True)
    y_full, h_full = fwd(x, dt, a, b, c, d, h0)
    world, s_loc = 4, 1024
    cut = [slice(k * s_loc, (k + 1) * s_loc) for k in range(world)]
    sl = lambda t, k: t[:, cut[k]].contiguous()
    first = [fwd(sl(x, k), sl(dt, k), a, sl(b, k), sl(c, k), d, h0 if k == 0 else None) for k in range(world)]
    h_locs = [hf for _, hf in first]
    decays = [bm.shard.slice_decay(sl(dt, k), a) for k in range(world)]
    ys = [first[0][0]]
    for k in range(1, world):
        ys.append(fwd(sl(x, k), sl(dt, k), a, sl(b, k), sl(c, k), d, bm.shard.entering_state(h_locs, decays, k))[0])
    y = torch.cat(ys, dim=1)
    assert rel_l2(host(y), host(y_full)) <= 1e-3
    assert rel_l2(host(bm.shard.entering_state(h_locs, decays, world)), host(h_full)) <= 1e-5


def test_ssd2_tensor_path_more_heads_than_sms_at_full_length(bm):
    """160 heads x L 4096 (more units than SMs, 32 tiles each): a random subset of heads against the oracle."""
    H = 160
    cfg = inputs.ssd2_prefill(seed=12, batch=1, seqlen=4096, nheads=H, headdim=64, state_rank=128, ngroups=1)
    x, b, c = (bf16_round(cfg[k]) for k in ("x", "b", "c"))
    y, hf = bm.ops.ssd2_fwd(dev(x, BF), dev(cfg["dt"]), dev(cfg["a"]), dev(b, BF), dev(c, BF), dev(cfg["d"]), None,
                            chunk_len=256, path="tensor", check_status=True)
    y, hf = host(y), host(hf)
    heads = np.random.default_rng(0).choice(H, 6, replace=False)
    for h in [0, H - 1, 147, 148] + list(heads):
        sl = slice(h, h + 1)
        want_y, want_h = mamba2.ssd_serial(x[:, :, sl], cfg["dt"][:, :, sl], cfg["a"][sl], b, c, cfg["d"][sl],
                                           cfg["h0"][:, sl], 256)
        assert rel_l2(y[:, :, sl], want_y) <= 2e-2 and rel_l2(hf[:, sl], want_h) <= 2e-2, h


def test_ssd2_tensor_path_batch_of_benchmark_heads(bm):
    """Batch 2 x 80 heads x L 4096, the benchmark's head count: tensor path against the float32 exact
    path on device for every unit, and against the oracle for a few."""
    cfg = inputs.ssd2_prefill(seed=22, batch=2, seqlen=4096, nheads=80, headdim=64, state_rank=128, ngroups=1)
    x, b, c = (bf16_round(cfg[k]) for k in ("x", "b", "c"))
    t = dict(x=dev(x, BF), dt=dev(cfg["dt"]), a=dev(cfg["a"]), b=dev(b, BF), c=dev(c, BF), d=dev(cfg["d"]))
    y, hf = bm.ops.ssd2_fwd(t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], None, chunk_len=256, path="tensor",
                            check_status=True)
    ye, he = bm.ops.ssd2_fwd(t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], None, chunk_len=256, path="exact")
    num = (y.float() - ye.float()).square().sum(dim=(1, 3)).sqrt()
    den = ye.float().square().sum(dim=(1, 3)).sqrt()
    assert float((num / den).max()) <= 2e-2            # per (batch, head) unit
    assert rel_l2(host(hf), host(he)) <= 2e-2
    for bi, h in [(0, 0), (1, 79), (1, 33)]:
        sl = slice(h, h + 1)
        want_y, want_h = mamba2.ssd_serial(x[bi:bi + 1, :, sl], cfg["dt"][bi:bi + 1, :, sl], cfg["a"][sl],
                                           b[bi:bi + 1], c[bi:bi + 1], cfg["d"][sl], cfg["h0"][bi:bi + 1, sl], 256)
        assert rel_l2(host(y[bi:bi + 1, :, sl]), want_y) <= 2e-2
        assert rel_l2(host(hf[bi:bi + 1, sl]), want_h) <= 2e-2


def test_ssd2_tensor_path_tiny_step_in_a_strongly_decaying_tile_keeps_the_skip_term(bm):
    """One token with dt ~ 1e-9 at the start of a tile whose total log2 decay is ~ -95: the per-row weight
    dt * 2^(cend - cum) falls far below the float32 normal range, so the factored mask form (which
    recovers D x by dividing by that weight) must not be chosen for this tile."""
    cfg = inputs.ssd2_prefill(seed=35, batch=1, seqlen=256, nheads=2, headdim=64, state_rank=128, h0_std=0.1)
    a = np.float32([-1.0, -1.0])
    dt = np.full((1, 256, 2), 95.0 / (128 * 1.4426950408889634), np.float32)   # cend ~ -95 per 128-token tile
    dt[0, 0, 0] = 1e-9
    dt[0, 128, 1] = 1e-30
    cfg.update(a=a, dt=dt)
    x, b, c = (bf16_round(cfg[k]) for k in ("x", "b", "c"))
    want_y, want_h = mamba2.ssd_serial(x, dt, a, b, c, cfg["d"], cfg["h0"], 128)
    y, hf = bm.ops.ssd2_fwd(dev(x, BF), dev(dt), dev(a), dev(b, BF), dev(c, BF), dev(cfg["d"]), dev(cfg["h0"]),
                            chunk_len=128, path="tensor", check_status=True)
    assert torch.isfinite(y.float()).all() and torch.isfinite(hf).all()
    assert rel_l2(host(y), want_y) <= 2e-2 and rel_l2(host(hf), want_h) <= 2e-2
    for t, h in [(0, 0), (128, 1)]:   # the rows of the tiny steps: y = C h + D x
        assert rel_l2(host(y)[0, t, h], want_y[0, t, h]) <= 2e-2


# ------------------------------------------------------------------ a2: Minimal variant with a learnable initial state
def test_minimal_path_with_init_state_matches_minimal_oracle(bm):
    """Mamba2SsdPath::Minimal adds init_state_hpr to the initial state (src/mamba2/ssd/minimal.rs:317-328)."""
    cfg = inputs.ssd2_prefill(seed=41, batch=2, seqlen=192, nheads=4, headdim=32, state_rank=64, ngroups=2, h0_std=0.1)
    rng = np.random.default_rng(3)
    init = (0.2 * rng.standard_normal((4, 32, 64))).astype(np.float32)
    want_y, want_h = mamba2.ssd_minimal(cfg["x"], cfg["dt"], cfg["a"], cfg["b"], cfg["c"], cfg["d"], cfg["h0"], 64,
                                        init_state_hpr=init)
    n, l = 3, 64
    inp = bm.Mamba2SsdInput(dev(cfg["x"]).reshape(2, n, l, 4, 32), dev(cfg["dt"]).reshape(2, n, l, 4), dev(cfg["a"]),
                            dev(cfg["b"]).reshape(2, n, l, 2, 64), dev(cfg["c"]).reshape(2, n, l, 2, 64),
                            dev(cfg["d"]), dev(cfg["h0"]), init_state_hpr=dev(init))
    y, hf = inp.run(bm.Mamba2SsdPath.minimal(64), kernel_path="exact")
    assert rel_l2(host(y).reshape(2, 192, 4, 32), want_y) <= 1e-4 and rel_l2(host(hf), want_h) <= 1e-4
    # without it the result differs (the term is really there), and the serial variants refuse it
    y0, _ = bm.Mamba2SsdInput(inp.x_bnlhp, inp.dt_bnlh, inp.a_decay_h, inp.b_bnlgr, inp.c_bnlgr, inp.d_h,
                              inp.initial_state_bhpr).run(bm.Mamba2SsdPath.minimal(64), kernel_path="exact")
    assert rel_l2(host(y0).reshape(2, 192, 4, 32), want_y) > 1e-3
    with pytest.raises(AssertionError):
        inp.run(bm.Mamba2SsdPath.serial_recalculated(64))


# ------------------------------------------------------------------ Mamba-1 selective scan at its configuration
def test_selscan1_at_the_configured_shape_bf16(bm):
    """batch 4, L 2048, d_inner 1536, N 16, bf16 inputs / float32 state, gate through SiLU."""
    cfg = inputs.selscan1(seed=1)
    u, delta, bb, cc, z = (bf16_round(cfg[k]) for k in ("u", "delta", "b", "c", "z"))
    want_y, want_h = mamba1.selective_scan(delta, cfg["a"], bb, cc, cfg["d"], u, cfg["h0"], dtype=np.float64)
    want_y = want_y * silu(z.astype(np.float64))
    y, hf = bm.ops.selscan1_fwd(dev(u, BF), dev(delta, BF), dev(cfg["a"]), dev(bb, BF), dev(cc, BF), dev(cfg["d"]),
                                z=dev(z, BF))
    assert rel_l2(host(y), want_y) <= 2e-2 and rel_l2(host(hf), want_h) <= 2e-2
    assert tuple(y.shape) == (4, 2048, 1536) and tuple(hf.shape) == (4, 1536, 16)


def test_selscan1_general_decay_matrix_and_initial_state_long_sequence(bm):
    """A decay matrix that is not the S4D-real ramp, a non-zero initial state and a ragged length."""
    cfg = inputs.selscan1(seed=5, batch=2, seqlen=1500, d_inner=96, state_rank=16)
    rng = np.random.default_rng(9)
    a = -np.exp(rng.uniform(-1.0, 2.5, cfg["a"].shape)).astype(np.float32)
    h0 = (0.3 * rng.standard_normal(cfg["h0"].shape)).astype(np.float32)
    want_y, want_h = mamba1.selective_scan(cfg["delta"], a, cfg["b"], cfg["c"], cfg["d"], cfg["u"], h0, dtype=np.float64)
    y, hf = bm.ops.selscan1_fwd(dev(cfg["u"]), dev(cfg["delta"]), dev(a), dev(cfg["b"]), dev(cfg["c"]), dev(cfg["d"]),
                                h0=dev(h0))
    assert rel_l2(host(y), want_y) <= 1e-4 and rel_l2(host(hf), want_h) <= 1e-4


@pytest.mark.parametrize("gate,softplus,ramp", [(True, False, True), (False, True, False), (True, True, False),
                                                 (False, False, True)])
def test_selscan1_rows_staged_by_tma_ragged_length_and_partial_channel_tile_bf16(bm, gate, softplus, ramp):
    """bf16 with d_inner a multiple of 8 takes the kernels that stage the token rows by TMA: a length that is no multiple
    of the staged block (8) nor of the segment (128), a last channel tile of 72 of 128 channels, a general decay matrix,
    the fused softplus, the gate on and off, a non-zero initial state; equal to the kernels that load through registers
    (float32 run of the same bf16-rounded inputs) and to the oracle."""
    from oracle.numerics import softplus_stock
    cfg = inputs.selscan1(seed=7, batch=2, seqlen=333, d_inner=200, state_rank=16)
    rng = np.random.default_rng(11)
    a = cfg["a"] if ramp else -np.exp(rng.uniform(-1.0, 2.0, cfg["a"].shape)).astype(np.float32)
    h0 = (0.3 * rng.standard_normal(cfg["h0"].shape)).astype(np.float32)
    u, bb, cc, z = (bf16_round(cfg[k]) for k in ("u", "b", "c", "z"))
    if softplus:
        raw = bf16_round(rng.standard_normal(cfg["delta"].shape).astype(np.float32))
        bias = rng.standard_normal(200).astype(np.float32)
        delta = softplus_stock(raw + bias)
    else:
        raw, bias, delta = bf16_round(cfg["delta"]), None, bf16_round(cfg["delta"])
    want_y, want_h = mamba1.selective_scan(delta, a, bb, cc, cfg["d"], u, h0, dtype=np.float64)
    if gate:
        want_y = want_y * silu(z.astype(np.float64))
    kw = dict(z=dev(z, BF) if gate else None, h0=dev(h0), delta_bias=None if bias is None else dev(bias),
              delta_softplus=softplus)
    y, hf = bm.ops.selscan1_fwd(dev(u, BF), dev(raw, BF), dev(a), dev(bb, BF), dev(cc, BF), dev(cfg["d"]), **kw)
    kw32 = dict(kw, z=dev(z) if gate else None)
    y32, hf32 = bm.ops.selscan1_fwd(dev(u), dev(raw), dev(a), dev(bb), dev(cc), dev(cfg["d"]), **kw32)
    assert rel_l2(host(y), want_y) <= 1e-2 and rel_l2(host(hf), want_h) <= 1e-4
    assert rel_l2(host(y), host(y32)) <= 1e-2 and rel_l2(host(hf), host(hf32)) <= 1e-5


# ------------------------------------------------------------------ Mamba-3 single SSD at its configuration
def _c5(seed, batch, seqlen, nheads):
    cfg = inputs.ssd3_single(seed=seed, batch=batch, seqlen=seqlen, nheads=nheads, headdim=64, state_rank=128,
                             mimo_rank=4)
    cfg["v"], cfg["b"], cfg["c"] = (bf16_round(cfg[k]) for k in ("v", "b", "c"))
    return cfg


@pytest.mark.parametrize("path", ["tensor", "exact"])
def test_ssd3_single_forward_at_the_configured_head_shape_bf16(bm, path):
    """H 32, P 64, N 128, m 4, Q 64, L 2048, bf16, rotation of B / C from the angles; every head runs on the GPU
    (tensor-core kernel and float32 exact path), three of them are checked against the oracle (heads are independent)."""
    cfg = _c5(4, 1, 2048, 32)
    y, hf = bm.ops.ssd3_single_fwd(dev(cfg["v"], BF), dev(cfg["da"]), dev(cfg["b"], BF), dev(cfg["c"], BF),
                                   dev(cfg["gamma"]), dev(cfg["scale"]), None, chunk_len=64,
                                   angles=dev(cfg["angles"]), rope_dim=128, path=path)
    y, hf = host(y), host(hf)
    for h in (0, 13, 31):
        sl = slice(h, h + 1)
        ang = cfg["angles"][:, :, None, sl]
        b_rot = mamba3.apply_rope_partial(cfg["b"][:, :, :, sl], ang, 128, False)
        c_rot = mamba3.apply_rope_partial(cfg["c"][:, :, :, sl], ang, 128, False)
        want_y, want_h = mamba3.single_ssd_serial(cfg["v"][:, :, :, sl], cfg["da"][:, :, sl], b_rot, c_rot,
                                                  cfg["gamma"][:, :, sl], cfg["scale"][:, :, sl], cfg["h0"][:, sl], 64)
        assert rel_l2(y[:, :, :, sl], want_y) <= 2e-2 and rel_l2(hf[:, sl], want_h) <= 2e-2, h


def test_ssd3_double_forward_bf16(bm):
    cfg = _c5(14, 1, 512, 4)
    ang = cfg["angles"][:, :, None]
    b_rot = mamba3.apply_rope_partial(cfg["b"], ang, 128, False)
    c_rot = mamba3.apply_rope_partial(cfg["c"], ang, 128, False)
    want_y, want_h = mamba3.double_ssd_serial(cfg["v"], cfg["da"], b_rot, c_rot, cfg["h0"], 64)
    y, hf = bm.ops.ssd3_double_fwd(dev(cfg["v"], BF), dev(cfg["da"]), dev(cfg["b"], BF), dev(cfg["c"], BF), None,
                                   chunk_len=64, angles=dev(cfg["angles"]), rope_dim=128)
    assert rel_l2(host(y), want_y) <= 2e-2 and rel_l2(host(hf), want_h) <= 2e-2


def test_ssd3_single_forward_backward_chain_bf16(bm):
    """Forward plus recompute backward in bf16 with the configuration's gradient chain: the slot's
    d_da, d_gamma, d_scale become ddt and dA, and dB / dC are pulled back through the rotation
    (ddt_t = A_h d_da_t + lambda_t (d_gamma_t + d_scale_t) + (1 - lambda_t) d_scale_{t-1},
    dA_h = sum d_da dt, gradients of rotated B / C rotated by -theta).  The oracle differentiates the whole
    chain (src/mamba3/single_ssd/single_ssd/mod.rs:111-149 builds the slot inputs this way)."""
    bsz, s, H, m = 1, 512, 2, 4
    cfg = _c5(24, bsz, s, H)
    rng = np.random.default_rng(4)
    x = bf16_round(rng.standard_normal((bsz, s, H, 64)).astype(np.float32))
    dy = bf16_round(rng.standard_normal(cfg["v"].shape).astype(np.float32))
    dhf = rng.standard_normal(cfg["h0"].shape).astype(np.float32)
    want = backward.ssd3_single_chain_grads(x, cfg["b"], cfg["c"], cfg["dt"], cfg["a"], cfg["lam"], cfg["angles"],
                                            cfg["h0"], dy, dhf, 64, mimo_rank=m)
    # device side: the harness builds the slot inputs, the library runs forward and backward
    v = bf16_round(np.repeat(x[:, :, None] / m, m, axis=2))
    ang = cfg["angles"][:, :, None]
    b_rot = bf16_round(mamba3.apply_rope_partial(cfg["b"], ang, 128, False))
    c_rot = bf16_round(mamba3.apply_rope_partial(cfg["c"], ang, 128, False))
    y, hf = bm.ops.ssd3_single_fwd(dev(v, BF), dev(cfg["da"]), dev(b_rot, BF), dev(c_rot, BF), dev(cfg["gamma"]),
                                   dev(cfg["scale"]), None, chunk_len=64)
    assert rel_l2(host(y), want["y"]) <= 2e-2 and rel_l2(host(hf), want["h_final"]) <= 2e-2
    g = bm.ops.ssd3_bwd(dev(v, BF), dev(cfg["da"]), dev(b_rot, BF), dev(c_rot, BF), dev(cfg["gamma"]),
                        dev(cfg["scale"]), None, dev(dy, BF), dev(dhf), chunk_len=64, single=True)
    g = {k: host(t) for k, t in g.items()}
    dx = g["dv"].sum(axis=2) / m
    dsc_prev = np.concatenate([np.zeros_like(g["dscale"][:, :1]), g["dscale"][:, :-1]], axis=1)
    ddt = cfg["a"][None, None] * g["dda"] + cfg["lam"] * (g["dgamma"] + g["dscale"]) + (1.0 - cfg["lam"]) * dsc_prev
    dA = (g["dda"] * cfg["dt"]).sum(axis=(0, 1))
    db = mamba3.apply_rope_partial(g["db"], -ang, 128, False)
    dc = mamba3.apply_rope_partial(g["dc"], -ang, 128, False)
    for name, got in (("dx", dx), ("ddt", ddt), ("dA", dA), ("dB", db), ("dC", dc)):
        assert rel_l2(got, want[name]) <= 2e-2, (name, rel_l2(got, want[name]))


def test_ssd2_backward_bf16_at_the_prefill_head_shape(bm):
    """Mamba-2 recompute backward with bf16 activations at P 64, N 128, G 1, Q 256 over 1024 tokens."""
    cfg = inputs.ssd2_prefill(seed=52, batch=1, seqlen=1024, nheads=3, headdim=64, state_rank=128, ngroups=1, h0_std=0.2)
    x, b, c = (bf16_round(cfg[k]) for k in ("x", "b", "c"))
    rng = np.random.default_rng(6)
    dy = bf16_round(rng.standard_normal(x.shape).astype(np.float32))
    dhf = rng.standard_normal(cfg["h0"].shape).astype(np.float32)
    want = backward.ssd2_grads(x, cfg["dt"], cfg["a"], b, c, cfg["d"], cfg["h0"], dy, dhf, 256)
    got = bm.ops.ssd2_bwd(dev(x, BF), dev(cfg["dt"]), dev(cfg["a"]), dev(b, BF), dev(c, BF), dev(cfg["d"]),
                          dev(cfg["h0"]), dev(dy, BF), dev(dhf), chunk_len=256)
    for k in ("dx", "ddt", "da", "db", "dc", "dd", "dh0"):
        assert rel_l2(host(got[k]), want[k]) <= 2e-2, (k, rel_l2(host(got[k]), want[k]))


# ------------------------------------------------------------------ bounded waits: a wait that runs out
def test_tensor_path_wait_that_runs_out_reports_timeout_and_the_context_stays_usable(bm):
    """The test hook makes the kernel's loader issue nothing: the first wait on a load runs out of its
    (shortened) budget, every role leaves its loop through the abort flag, the status word reads
    BM_ERR_TIMEOUT, and the next ordinary call on the same context is correct."""
    cfg = inputs.ssd2_prefill(seed=61, batch=1, seqlen=512, nheads=4, headdim=64, state_rank=128, ngroups=1)
    x, b, c = (bf16_round(cfg[k]) for k in ("x", "b", "c"))
    args = (dev(x, BF), dev(cfg["dt"]), dev(cfg["a"]), dev(b, BF), dev(c, BF), dev(cfg["d"]), None)
    with pytest.raises(bm.BmError) as e:
        bm.ops.ssd2_fwd(*args, chunk_len=256, path="tensor", check_status=True,
                        debug_reserved=bm._ffi.BM_DEBUG_STALL_LOADS)
    assert e.value.code == bm._ffi.BM_ERR_TIMEOUT
    torch.cuda.synchronize()
    want_y, want_h = mamba2.ssd_serial(x, cfg["dt"], cfg["a"], b, c, cfg["d"], cfg["h0"], 256)
    y, hf = bm.ops.ssd2_fwd(*args, chunk_len=256, path="tensor", check_status=True)
    assert rel_l2(host(y), want_y) <= 2e-2 and rel_l2(host(hf), want_h) <= 2e-2


# ------------------------------------------------------------------ (batch x head) sharding on the device
@pytest.mark.parametrize("world,by_heads", [(2, False), (4, False), (5, True), (8, True)])
def test_sharded_units_give_the_bits_of_the_unsharded_call(bm, world, by_heads):
    """Every rank's share of one problem (shard.partition_units / partition_heads, run here one rank after the
    other through the same library calls a rank makes) put back together equals the single call bit for bit:
    whole rows merged into one call, head ranges cut at group boundaries, partial groups."""
    shard = bm.shard
    cfg = inputs.ssd2_prefill(seed=57, batch=3, seqlen=512, nheads=12, headdim=64, state_rank=128, ngroups=3, h0_std=0.1)
    x, b, c = (dev(cfg[k], BF) for k in ("x", "b", "c"))
    dt, a, d, h0 = dev(cfg["dt"]), dev(cfg["a"]), dev(cfg["d"]), dev(cfg["h0"])
    fwd = lambda *args: bm.ops.ssd2_fwd(*args[:7], chunk_len=args[7], path="tensor", check_status=True)
    want_y, want_h = fwd(x, dt, a, b, c, d, h0, 128)
    parts_of_all = shard.partition_heads(3, 12, world) if by_heads else shard.partition_units(3, 12, 3, world)
    assert sum(p.count for p in parts_of_all) == 36
    got_y, got_h = torch.zeros_like(want_y), torch.zeros_like(want_h)
    for mine in parts_of_all:
        for b_lo, b_hi, h_lo, h_hi, y_p, h_p in shard.ssd2_fwd_local(fwd, x, dt, a, b, c, d, h0, 128, mine):
            got_y[b_lo:b_hi, :, h_lo:h_hi] = y_p
            got_h[b_lo:b_hi, h_lo:h_hi] = h_p
    assert torch.equal(got_y, want_y) and torch.equal(got_h, want_h)
