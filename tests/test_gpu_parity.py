"""GPU parity tests: every C-ABI entry point against the CPU oracle on the same seeded inputs.

Tolerances (rel-L2, stated by the benchmark definition): 1e-4 for float32, 2e-2 for bfloat16, on
outputs and on final states.  The reference's own tolerances at tiny shapes are max-abs 1e-4.
"""
import numpy as np
import pytest
import torch

from oracle import inputs, mamba1, mamba2, mamba3
from oracle.numerics import rel_l2, bf16_round

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    return t.float().cpu().numpy()


def q(x, dtype):
    """The values the kernel actually sees for an activation tensor of `dtype`."""
    return bf16_round(x) if dtype == torch.bfloat16 else x


# ------------------------------------------------------------------ Mamba-2 SSD (exact path)
def _ssd2_case(bm, cfg, chunk_len, dtype, path="exact", use_h0=True, tol=None, **kw):
    x, b, c = (q(cfg[k], dtype) for k in ("x", "b", "c"))
    h0 = cfg["h0"] if use_h0 else None
    want_y, want_h = mamba2.ssd_serial(x, cfg["dt"], cfg["a"], b, c, cfg["d"],
                                       cfg["h0"] if use_h0 else np.zeros_like(cfg["h0"]), chunk_len)
    y, h = bm.ops.ssd2_fwd(dev(x, dtype), dev(cfg["dt"]), dev(cfg["a"]), dev(b, dtype), dev(c, dtype), dev(cfg["d"]),
                           None if h0 is None else dev(h0), chunk_len=chunk_len, path=path, **kw)
    torch.cuda.synchronize()
    tol = tol or TOL[dtype]
    ey, eh = rel_l2(host(y), want_y), rel_l2(host(h), want_h)
    assert ey <= tol and eh <= tol, (ey, eh)
    return y, h


@pytest.mark.parametrize("b,s,h,p,r,g,Q", [
    (2, 4, 2, 8, 8, 1, 4),      # the reference's tiny shapes (src/mamba2/ssd/ssd_path/tests.rs:15-68)
    (2, 12, 4, 8, 8, 2, 4),
    (2, 10, 4, 8, 8, 1, 4),     # ragged tail chunk
    (1, 37, 3, 16, 24, 3, 16),  # odd everything
    (2, 512, 8, 64, 64, 1, 64),  # the CPU-runnable configuration's SSD shape
    (1, 300, 4, 64, 128, 2, 256),
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ssd2_exact_matches_oracle(bm, b, s, h, p, r, g, Q, dtype):
    cfg = inputs.ssd2_prefill(seed=100 + s, batch=b, seqlen=s, nheads=h, headdim=p, state_rank=r, ngroups=g,
                              h0_std=0.1)
    _ssd2_case(bm, cfg, Q, dtype)


def test_ssd2_exact_zero_state_and_chunk_states(bm):
    cfg = inputs.ssd2_prefill(seed=7, batch=2, seqlen=96, nheads=4, headdim=16, state_rank=16)
    _ssd2_case(bm, cfg, 32, torch.float32, use_h0=False)
    t = {k: dev(v) for k, v in cfg.items()}
    y, hf, st = bm.ops.ssd2_fwd(t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], t["h0"], chunk_len=32, path="exact",
                                return_chunk_states=True)
    _, _, want = mamba2.ssd_serial(cfg["x"], cfg["dt"], cfg["a"], cfg["b"], cfg["c"], cfg["d"], cfg["h0"], 32,
                                   return_chunk_states=True)
    assert rel_l2(host(st), want) <= 1e-4


def test_ssd2_fused_dt_bias_and_gate(bm):
    cfg = inputs.ssd2_prefill(seed=8, batch=2, seqlen=70, nheads=4, headdim=16, state_rank=16, h0_std=0.1)
    rng = np.random.default_rng(0)
    raw = rng.standard_normal(cfg["dt"].shape).astype(np.float32)
    z = rng.standard_normal(cfg["x"].shape).astype(np.float32)
    from oracle.numerics import softplus, silu
    dt = np.clip(softplus(raw + cfg["dt_bias"], "f32"), 0.0, 65504.0).astype(np.float32)
    want_y, want_h = mamba2.ssd_serial(cfg["x"], dt, cfg["a"], cfg["b"], cfg["c"], cfg["d"], cfg["h0"], 32)
    y, h = bm.ops.ssd2_fwd(dev(cfg["x"]), dev(raw), dev(cfg["a"]), dev(cfg["b"]), dev(cfg["c"]), dev(cfg["d"]),
                           dev(cfg["h0"]), chunk_len=32, path="exact", dt_bias=dev(cfg["dt_bias"]), z=dev(z))
    assert rel_l2(host(y), want_y * silu(z)) <= 1e-4 and rel_l2(host(h), want_h) <= 1e-4


def test_ssd2_split_prefill_equals_full(bm):
    """split == full (src/mamba2/mamba2/tests.rs:343-392) at the slot level, CUDA vs CUDA."""
    cfg = inputs.ssd2_prefill(seed=9, batch=2, seqlen=200, nheads=4, headdim=32, state_rank=32, h0_std=0.1)
    t = {k: dev(v) for k, v in cfg.items()}
    y, h = bm.ops.ssd2_fwd(t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], t["h0"], chunk_len=64, path="exact")
    cut = 77
    y1, h1 = bm.ops.ssd2_fwd(t["x"][:, :cut].contiguous(), t["dt"][:, :cut].contiguous(), t["a"],
                             t["b"][:, :cut].contiguous(), t["c"][:, :cut].contiguous(), t["d"], t["h0"],
                             chunk_len=64, path="exact")
    y2, h2 = bm.ops.ssd2_fwd(t["x"][:, cut:].contiguous(), t["dt"][:, cut:].contiguous(), t["a"],
                             t["b"][:, cut:].contiguous(), t["c"][:, cut:].contiguous(), t["d"], h1,
                             chunk_len=64, path="exact")
    assert rel_l2(host(torch.cat([y1, y2], 1)), host(y)) <= 1e-5 and rel_l2(host(h2), host(h)) <= 1e-5


def test_ssd2_forward_equals_unrolled_step(bm):
    """forward == unrolled step (src/mamba2/mamba2/tests.rs:202-252), CUDA SSD vs CUDA step kernel."""
    cfg = inputs.ssd2_prefill(seed=10, batch=2, seqlen=48, nheads=4, headdim=32, state_rank=64, ngroups=2, h0_std=0.1)
    t = {k: dev(v) for k, v in cfg.items()}
    y, h = bm.ops.ssd2_fwd(t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], t["h0"], chunk_len=16, path="exact")
    state = t["h0"].clone()
    for s in range(48):
        ys = bm.ops.step2(state, t["x"][:, s].contiguous(), t["dt"][:, s].contiguous(), t["a"],
                          t["b"][:, s].contiguous(), t["c"][:, s].contiguous(), t["d"])
        assert torch.max(torch.abs(ys - y[:, s])).item() <= 1e-4
    assert torch.max(torch.abs(state - h)).item() <= 1e-4


def test_ssd2_rejects_bad_arguments(bm):
    cfg = inputs.ssd2_prefill(seed=1, batch=1, seqlen=8, nheads=2, headdim=8, state_rank=8)
    t = {k: dev(v) for k, v in cfg.items()}
    with pytest.raises(bm.BmError) as e:
        bm.ops.ssd2_fwd(t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], t["h0"], chunk_len=0, path="exact")
    assert e.value.code == bm._ffi.BM_ERR_BAD_SHAPE
    with pytest.raises(bm.BmError) as e:
        bm.ops.ssd2_fwd(t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], t["h0"], chunk_len=4, path="tensor")
    assert e.value.code == bm._ffi.BM_ERR_UNSUPPORTED


# ------------------------------------------------------------------ Mamba-2 step / conv step
@pytest.mark.parametrize("b,h,p,r,g", [(2, 4, 8, 8, 1), (3, 4, 64, 128, 2), (2, 2, 16, 256, 1), (2, 2, 5, 6, 1),
                                       (4, 8, 64, 64, 1), (2, 3, 7, 16, 3)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_step2_matches_oracle(bm, b, h, p, r, g, dtype):
    cfg = inputs.step2_decode(seed=5, batch=b, nheads=h, headdim=p, state_rank=r, ngroups=g, steps=3)
    state = dev(cfg["state"])
    ref = cfg["state"].copy()
    for s in range(3):
        x, bb, cc = (q(cfg[k][s], dtype) for k in ("x", "b", "c"))
        want_y, ref = mamba2.ssm_step(ref, x, cfg["dt"][s], cfg["a"], bb, cc, cfg["d"])
        y = bm.ops.step2(state, dev(x, dtype), dev(cfg["dt"][s]), dev(cfg["a"]), dev(bb, dtype), dev(cc, dtype),
                         dev(cfg["d"]))
        assert rel_l2(host(y), want_y) <= TOL[dtype]
    assert rel_l2(host(state), ref) <= 1e-5


def test_conv_step_matches_oracle(bm):
    rng = np.random.default_rng(3)
    b, v, k = 3, 40, 4
    win = rng.standard_normal((b, v, k)).astype(np.float32)
    w = rng.standard_normal((v, k)).astype(np.float32)
    bias = rng.standard_normal(v).astype(np.float32)
    window = dev(win)
    from oracle.numerics import silu
    for _ in range(3):
        xin = rng.standard_normal((b, v)).astype(np.float32)
        win = np.concatenate([win[:, :, 1:], xin[:, :, None]], axis=2)
        want = silu((win * w[None]).sum(-1) + bias[None])
        out = bm.ops.conv_step(window, dev(xin), dev(w), dev(bias))
        assert rel_l2(host(out), want) <= 1e-5
    assert np.array_equal(host(window), win)


# ------------------------------------------------------------------ Mamba-1
@pytest.mark.parametrize("b,s,i,r", [(2, 9, 24, 4), (2, 200, 64, 16), (1, 130, 96, 8), (2, 33, 10, 3)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selscan1_matches_oracle(bm, b, s, i, r, dtype):
    cfg = inputs.selscan1(seed=1, batch=b, seqlen=s, d_inner=i, state_rank=r)
    rng = np.random.default_rng(2)
    h0 = (0.1 * rng.standard_normal(cfg["h0"].shape)).astype(np.float32)
    u, delta, bb, cc, z = (q(cfg[k], dtype) for k in ("u", "delta", "b", "c", "z"))
    want_y, want_h = mamba1.selective_scan(delta, cfg["a"], bb, cc, cfg["d"], u, h0, dtype=np.float64)
    from oracle.numerics import silu
    want_y = want_y * silu(z.astype(np.float64))
    y, hf = bm.ops.selscan1_fwd(dev(u, dtype), dev(delta, dtype), dev(cfg["a"]), dev(bb, dtype), dev(cc, dtype),
                                dev(cfg["d"]), z=dev(z, dtype), h0=dev(h0))
    assert rel_l2(host(y), want_y) <= TOL[dtype] and rel_l2(host(hf), want_h) <= TOL[dtype]


def test_selscan1_forward_equals_unrolled_step(bm):
    """src/mamba1/mamba1/tests.rs:216-265 at the scan level, CUDA vs CUDA."""
    cfg = inputs.selscan1(seed=4, batch=2, seqlen=40, d_inner=64, state_rank=16)
    t = {k: dev(v) for k, v in cfg.items()}
    y, hf = bm.ops.selscan1_fwd(t["u"], t["delta"], t["a"], t["b"], t["c"], t["d"], h0=t["h0"])
    state = t["h0"].clone()
    for s in range(40):
        ys = bm.ops.step1(state, t["u"][:, s].contiguous(), t["delta"][:, s].contiguous(), t["a"],
                          t["b"][:, s].contiguous(), t["c"][:, s].contiguous(), t["d"])
        assert torch.max(torch.abs(ys - y[:, s])).item() <= 1e-4
    assert torch.max(torch.abs(state - hf)).item() <= 1e-4


def test_selscan1_fused_softplus(bm):
    cfg = inputs.selscan1(seed=6, batch=2, seqlen=70, d_inner=32, state_rank=16)
    rng = np.random.default_rng(1)
    raw = rng.standard_normal(cfg["delta"].shape).astype(np.float32)
    bias = rng.standard_normal(32).astype(np.float32)
    from oracle.numerics import softplus_stock
    delta = softplus_stock(raw + bias)
    want_y, want_h = mamba1.selective_scan(delta, cfg["a"], cfg["b"], cfg["c"], cfg["d"], cfg["u"], cfg["h0"])
    y, hf = bm.ops.selscan1_fwd(dev(cfg["u"]), dev(raw), dev(cfg["a"]), dev(cfg["b"]), dev(cfg["c"]), dev(cfg["d"]),
                                delta_bias=dev(bias), delta_softplus=True)
    assert rel_l2(host(y), want_y) <= 1e-4 and rel_l2(host(hf), want_h) <= 1e-4


# ------------------------------------------------------------------ Mamba-3
@pytest.mark.parametrize("b,s,h,p,r,m,Q", [(2, 12, 2, 8, 8, 1, 4), (2, 12, 4, 8, 8, 2, 4), (2, 10, 2, 8, 8, 2, 4),
                                           (1, 100, 2, 64, 128, 4, 64), (1, 70, 3, 16, 32, 3, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ssd3_single_and_double_match_oracle(bm, b, s, h, p, r, m, Q, dtype):
    cfg = inputs.ssd3_single(seed=40 + s, batch=b, seqlen=s, nheads=h, headdim=p, state_rank=r, mimo_rank=m,
                             h0_std=0.1)
    pairwise = m == 1
    ang = cfg["angles"][:, :, None]
    b_rot = mamba3.apply_rope_partial(q(cfg["b"], dtype), ang, r, pairwise)
    c_rot = mamba3.apply_rope_partial(q(cfg["c"], dtype), ang, r, pairwise)
    v = q(cfg["v"], dtype)
    want_y, want_h = mamba3.single_ssd_serial(v, cfg["da"], b_rot, c_rot, cfg["gamma"], cfg["scale"], cfg["h0"], Q)
    # rotation fused at load: raw B/C + angles
    y, hf = bm.ops.ssd3_single_fwd(dev(v, dtype), dev(cfg["da"]), dev(cfg["b"], dtype), dev(cfg["c"], dtype),
                                   dev(cfg["gamma"]), dev(cfg["scale"]), dev(cfg["h0"]), chunk_len=Q,
                                   angles=dev(cfg["angles"]), rope_dim=r)
    assert rel_l2(host(y), want_y) <= TOL[dtype] and rel_l2(host(hf), want_h) <= TOL[dtype]
    if dtype == torch.float32:
        # pre-rotated B/C, no angles
        y2, hf2 = bm.ops.ssd3_single_fwd(dev(v), dev(cfg["da"]), dev(b_rot), dev(c_rot), dev(cfg["gamma"]),
                                         dev(cfg["scale"]), dev(cfg["h0"]), chunk_len=Q)
        assert rel_l2(host(y2), want_y) <= 1e-4 and rel_l2(host(hf2), want_h) <= 1e-4
        want_yd, want_hd = mamba3.double_ssd_serial(v, cfg["da"], b_rot, c_rot, cfg["h0"], Q)
        y3, hf3 = bm.ops.ssd3_double_fwd(dev(v), dev(cfg["da"]), dev(b_rot), dev(c_rot), dev(cfg["h0"]), chunk_len=Q)
        assert rel_l2(host(y3), want_yd) <= 1e-4 and rel_l2(host(hf3), want_hd) <= 1e-4


@pytest.mark.parametrize("m,rope_fraction", [(1, 1.0), (2, 1.0), (2, 0.5), (1, 0.5), (1, 0.0)])
def test_angle_cumsum_and_step3_match_oracle_block(bm, m, rope_fraction):
    """The oracle's Mamba-3 block supplies slot tensors; the CUDA angle scan and step kernel must
    reproduce its rotation state, state update and readout token by token."""
    rng = np.random.default_rng(12)
    w = mamba3.Mamba3Weights(rng, d_model=16, d_inner=32, nheads=4, state_rank=16, mimo_rank=m,
                             rope_fraction=rope_fraction, dtype=np.float32)
    if m > 1:
        w.mimo_x = (w.mimo_x + 0.2 * rng.standard_normal(w.mimo_x.shape)).astype(np.float32)
    bsz, s = 2, 9
    u = rng.standard_normal((bsz, s, 16)).astype(np.float32)
    cache = {k: (v + 0.1 * rng.standard_normal(v.shape)).astype(np.float32)
             for k, v in mamba3.zero_cache(w, bsz).items()}
    z, x, bm_, cm_, co, rot = mamba3._project(w, u, "f32")
    theta, last = bm.ops.angle_cumsum(dev(rot), dev(co["dt"]), dev(cache["angle"]), rng=w.rotation_range)
    _, _, want_last, want_theta = mamba3.rotate_bc_forward(rot, co["dt"], cache["angle"], bm_, cm_, w.rope_dim,
                                                           w.rotation_range)
    assert np.max(np.abs(host(theta) - want_theta)) <= 1e-4
    assert np.max(np.abs(np.angle(np.exp(1j * (host(last) - want_last))))) <= 1e-4
    state, k_state, v_state, angle = (dev(cache[k]) for k in ("ssm", "k", "v", "angle"))
    c = dict(cache)
    for t in range(s):
        br, cr, new_angle = mamba3.rotate_bc_step(rot[:, t], co["dt"][:, t], c["angle"], bm_[:, t], cm_[:, t],
                                                  w.rope_dim, w.rotation_range)
        want_y, h_new, _ = mamba3.ssm_step3(c["ssm"], x[:, t], c["v"], br, c["k"], cr, co["alpha"][:, t],
                                            co["beta"][:, t], co["gamma"][:, t], w.mimo_x)
        c = dict(ssm=h_new, k=br, v=x[:, t], angle=new_angle)
        y = bm.ops.step3(state, k_state, v_state, angle, dev(x[:, t]), dev(bm_[:, t]), dev(cm_[:, t]),
                         dev(rot[:, t]), dev(co["dt"][:, t]), dev(co["alpha"][:, t]), dev(co["beta"][:, t]),
                         dev(co["gamma"][:, t]), None if w.mimo_x is None else dev(w.mimo_x), rope_dim=w.rope_dim,
                         rng=w.rotation_range)
        assert rel_l2(host(y), want_y) <= 1e-4
    assert rel_l2(host(state), c["ssm"]) <= 1e-4 and rel_l2(host(k_state), c["k"]) <= 1e-4
    assert np.array_equal(host(v_state), c["v"])
    assert np.max(np.abs(np.angle(np.exp(1j * (host(angle) - c["angle"]))))) <= 1e-4


# ------------------------------------------------------------------ Mamba-2 SSD (tensor-core path)
@pytest.mark.parametrize("b,s,h,g,Q", [
    (1, 128, 1, 1, 128),     # one tile
    (1, 256, 2, 1, 256),     # one chunk = two tiles
    (2, 512, 4, 2, 256),     # groups
    (1, 300, 3, 3, 128),     # ragged tail (zero-filled rows, clipped store)
    (1, 100, 2, 1, 64),      # shorter than one tile
    (2, 1024, 8, 1, 256),
    (3, 384, 160, 1, 256),   # more units than SMs: several units per CTA
])
def test_ssd2_tensor_path_matches_oracle(bm, b, s, h, g, Q):
    cfg = inputs.ssd2_prefill(seed=200 + s, batch=b, seqlen=s, nheads=h, headdim=64, state_rank=128, ngroups=g,
                              h0_std=0.1)
    dt = torch.bfloat16
    if b * s * h <= 64 * 1024:
        y, hf = _ssd2_case(bm, cfg, Q, dt, path="tensor", check_status=True)
    else:
        x, bb, cc = (dev(cfg[k], dt) for k in ("x", "b", "c"))
        y, hf = bm.ops.ssd2_fwd(x, dev(cfg["dt"]), dev(cfg["a"]), bb, cc, dev(cfg["d"]), dev(cfg["h0"]), chunk_len=Q,
                                path="tensor", check_status=True)
    # on-device cross-check against the exact path (same bf16 inputs, float32 arithmetic)
    x, bb, cc = (dev(cfg[k], dt) for k in ("x", "b", "c"))
    ye, he = bm.ops.ssd2_fwd(x, dev(cfg["dt"]), dev(cfg["a"]), bb, cc, dev(cfg["d"]), dev(cfg["h0"]), chunk_len=Q,
                             path="exact")
    assert rel_l2(host(y), host(ye)) <= 2e-2 and rel_l2(host(hf), host(he)) <= 2e-2


def test_ssd2_tensor_path_chunk_states_and_fused_dt(bm):
    cfg = inputs.ssd2_prefill(seed=31, batch=2, seqlen=768, nheads=4, headdim=64, state_rank=128, h0_std=0.1)
    dt = torch.bfloat16
    x, bb, cc = (q(cfg[k], dt) for k in ("x", "b", "c"))
    _, _, want = mamba2.ssd_serial(x, cfg["dt"], cfg["a"], bb, cc, cfg["d"], cfg["h0"], 256, return_chunk_states=True)
    y, hf, st = bm.ops.ssd2_fwd(dev(x, dt), dev(cfg["dt"]), dev(cfg["a"]), dev(bb, dt), dev(cc, dt), dev(cfg["d"]),
                                dev(cfg["h0"]), chunk_len=256, path="tensor", return_chunk_states=True,
                                check_status=True)
    assert rel_l2(host(st), want) <= 2e-2
    rng = np.random.default_rng(5)
    raw = rng.standard_normal(cfg["dt"].shape).astype(np.float32)
    from oracle.numerics import softplus
    dtv = np.clip(softplus(raw + cfg["dt_bias"], "f32"), 0.0, 65504.0).astype(np.float32)
    want_y, want_h = mamba2.ssd_serial(x, dtv, cfg["a"], bb, cc, cfg["d"], cfg["h0"], 256)
    y, hf = bm.ops.ssd2_fwd(dev(x, dt), dev(raw), dev(cfg["a"]), dev(bb, dt), dev(cc, dt), dev(cfg["d"]),
                            dev(cfg["h0"]), chunk_len=256, path="tensor", dt_bias=dev(cfg["dt_bias"]),
                            check_status=True)
    assert rel_l2(host(y), want_y) <= 2e-2 and rel_l2(host(hf), want_h) <= 2e-2


def test_ssd2_tensor_path_strong_decay_is_finite(bm):
    """Large dt*|A| (state forgotten within a few tokens): the factored decay mask must not overflow."""
    cfg = inputs.ssd2_prefill(seed=32, batch=1, seqlen=256, nheads=2, headdim=64, state_rank=128, h0_std=0.1)
    cfg["dt"] = (cfg["dt"] * 0 + 3.0).astype(np.float32)
    cfg["a"] = np.float32([-16.0, -0.001])
    y, hf = _ssd2_case(bm, cfg, 256, torch.bfloat16, path="tensor", check_status=True)
    assert torch.isfinite(y.float()).all() and torch.isfinite(hf).all()


def test_ssd2_tensor_path_zero_steps_keep_the_skip_term(bm):
    """Tokens with dt == 0 contribute nothing to the state but still pass D x through; tiles that contain
    one take the exact mask form (the factored form would divide by dt)."""
    cfg = inputs.ssd2_prefill(seed=33, batch=1, seqlen=384, nheads=3, headdim=64, state_rank=128, h0_std=0.1)
    cfg["dt"][:, 5::7, :] = 0.0
    cfg["dt"][:, 200:300, 1] = 0.0
    dt = torch.bfloat16
    x, bb, cc = (q(cfg[k], dt) for k in ("x", "b", "c"))
    want_y, want_h = mamba2.ssd_serial(x, cfg["dt"], cfg["a"], bb, cc, cfg["d"], cfg["h0"], 128)
    y, hf = _ssd2_case(bm, cfg, 128, dt, path="tensor", check_status=True)
    assert rel_l2(host(y), want_y) <= 2e-2 and rel_l2(host(hf), want_h) <= 2e-2
    # the rows of the zero steps themselves: y = C h + D x exactly as the oracle has it
    rows = host(y)[:, 200:300, 1]
    assert rel_l2(rows, want_y[:, 200:300, 1]) <= 2e-2


def test_ssd2_tensor_path_mixed_decay_tiles(bm):
    """Heads with weak and with very strong decay side by side: factored and exact tiles alternate within
    one launch (the X stage is released differently by the two forms)."""
    cfg = inputs.ssd2_prefill(seed=34, batch=2, seqlen=1024, nheads=6, headdim=64, state_rank=128, h0_std=0.1)
    cfg["a"] = np.float32([-0.5, -16.0, -1.0, -12.0, -0.01, -8.0])
    rng = np.random.default_rng(7)
    cfg["dt"] = (rng.random(cfg["dt"].shape) * np.float32([0.01, 0.8, 0.02, 0.5, 0.05, 0.3])).astype(np.float32)
    cfg["dt"][:, 512:640] *= 40.0       # a stretch of large steps in every head
    dt = torch.bfloat16
    x, bb, cc = (q(cfg[k], dt) for k in ("x", "b", "c"))
    want_y, want_h = mamba2.ssd_serial(x, cfg["dt"], cfg["a"], bb, cc, cfg["d"], cfg["h0"], 256)
    y, hf = _ssd2_case(bm, cfg, 256, dt, path="tensor", check_status=True)
    assert rel_l2(host(y), want_y) <= 2e-2 and rel_l2(host(hf), want_h) <= 2e-2


def test_ssd2_tensor_path_units_cut_between_ctas_are_bitwise_equal_to_whole_units(bm):
    """More units than SMs: the tiles of all units are dealt out as one contiguous range per CTA, so units
    straddle CTAs and their state crosses through the workspace.  The same rows launched one at a time (fewer
    units than SMs: nothing is cut) must give the same bits, chunk states included."""
    cfg = inputs.ssd2_prefill(seed=35, batch=3, seqlen=640, nheads=100, headdim=64, state_rank=128, h0_std=0.1)
    dt = torch.bfloat16
    args = [dev(cfg["x"], dt), dev(cfg["dt"]), dev(cfg["a"]), dev(cfg["b"], dt), dev(cfg["c"], dt), dev(cfg["d"]),
            dev(cfg["h0"])]
    y, hf, st = bm.ops.ssd2_fwd(*args, chunk_len=128, path="tensor", return_chunk_states=True, check_status=True)
    for row in range(3):
        sl = lambda t, batched: t[row:row + 1].contiguous() if batched else t
        part = [sl(a, i in (0, 1, 3, 4, 6)) for i, a in enumerate(args)]
        y1, h1, s1 = bm.ops.ssd2_fwd(*part, chunk_len=128, path="tensor", return_chunk_states=True, check_status=True)
        assert torch.equal(y[row:row + 1], y1) and torch.equal(hf[row:row + 1], h1) and torch.equal(st[row:row + 1], s1)
    ye, he = bm.ops.ssd2_fwd(*args, chunk_len=128, path="exact")
    assert rel_l2(host(y), host(ye)) <= 2e-2 and rel_l2(host(hf), host(he)) <= 2e-2


# ------------------------------------------------------------------ backward (recompute) vs autodiff oracle
def _grad_close(got, want, tol=1e-3):
    """The reference's gradient tolerance is max-abs 1e-3 at its tiny shapes; relative-L2 here."""
    return rel_l2(host(got), want) <= tol


@pytest.mark.parametrize("b,s,h,p,r,g,Q", [(2, 12, 4, 8, 8, 1, 4), (2, 10, 4, 8, 8, 2, 4), (1, 70, 2, 16, 32, 1, 32),
                                           (1, 96, 2, 64, 128, 1, 64), (1, 33, 3, 8, 16, 3, 16)])
def test_ssd2_backward_matches_autodiff_oracle(bm, b, s, h, p, r, g, Q):
    """Recompute backward == autodiff of the serial forward
    (src/mamba2/ssd/ssd_path/tests.rs:184-336 asserts the same on all seven inputs)."""
    from oracle import backward
    cfg = inputs.ssd2_prefill(seed=300 + s, batch=b, seqlen=s, nheads=h, headdim=p, state_rank=r, ngroups=g, h0_std=0.2)
    rng = np.random.default_rng(1)
    dy = rng.standard_normal(cfg["x"].shape).astype(np.float32)
    dhf = rng.standard_normal(cfg["h0"].shape).astype(np.float32)
    want = backward.ssd2_grads(cfg["x"], cfg["dt"], cfg["a"], cfg["b"], cfg["c"], cfg["d"], cfg["h0"], dy, dhf, Q)
    got = bm.ops.ssd2_bwd(dev(cfg["x"]), dev(cfg["dt"]), dev(cfg["a"]), dev(cfg["b"]), dev(cfg["c"]), dev(cfg["d"]),
                          dev(cfg["h0"]), dev(dy), dev(dhf), chunk_len=Q)
    torch.cuda.synchronize()
    for k in ("dx", "ddt", "da", "db", "dc", "dd", "dh0"):
        assert _grad_close(got[k], want[k]), (k, rel_l2(host(got[k]), want[k]))


def _bwd_inputs(cfg, seed):
    dt = torch.bfloat16
    x, b, c = (q(cfg[k], dt) for k in ("x", "b", "c"))
    rng = np.random.default_rng(seed)
    dy = q(rng.standard_normal(x.shape).astype(np.float32), dt)
    dhf = rng.standard_normal(cfg["h0"].shape).astype(np.float32)
    args = (dev(x, dt), dev(cfg["dt"]), dev(cfg["a"]), dev(b, dt), dev(c, dt), dev(cfg["d"]), dev(cfg["h0"]), dev(dy, dt),
            dev(dhf))
    return (x, b, c, dy, dhf), args


@pytest.mark.parametrize("b,s,h,g", [(1, 128, 1, 1), (1, 256, 2, 1), (2, 1024, 4, 2), (1, 300, 3, 3), (1, 100, 2, 1)])
def test_ssd2_backward_tensor_path_matches_autodiff_oracle(bm, b, s, h, g):
    """The tcgen05 backward (bf16 operands, float32 accumulation) against autodiff of the serial forward on the
    same bf16-rounded inputs: all seven gradients, ragged lengths, groups, initial state and dh_final."""
    from oracle import backward
    cfg = inputs.ssd2_prefill(seed=310 + s, batch=b, seqlen=s, nheads=h, headdim=64, state_rank=128, ngroups=g, h0_std=0.2)
    (x, bb, cc, dy, dhf), args = _bwd_inputs(cfg, 11)
    want = backward.ssd2_grads(x, cfg["dt"], cfg["a"], bb, cc, cfg["d"], cfg["h0"], dy, dhf, 128)
    got = bm.ops.ssd2_bwd(*args, chunk_len=128, path="tensor", check_status=True)
    for k in ("dx", "ddt", "da", "db", "dc", "dd", "dh0"):
        assert rel_l2(host(got[k]), want[k]) <= 2e-2, (k, rel_l2(host(got[k]), want[k]))


def test_ssd2_backward_tensor_path_cut_units_strong_decay_and_zero_steps(bm):
    """More units than SMs (units straddle CTAs and dh crosses through the workspace), heads whose state is
    forgotten within a few tokens, and steps of exactly zero: the tensor-core backward against the float32
    backward on device, and without dh_final / initial state / skip."""
    cfg = inputs.ssd2_prefill(seed=36, batch=3, seqlen=640, nheads=100, headdim=64, state_rank=128, h0_std=0.1)
    cfg["a"][::7] = -16.0
    cfg["dt"][:, :, ::7] = 3.0
    cfg["dt"][:, 5::9, 1::3] = 0.0
    _, args = _bwd_inputs(cfg, 12)
    got = bm.ops.ssd2_bwd(*args, chunk_len=128, path="tensor", check_status=True)
    want = bm.ops.ssd2_bwd(*args, chunk_len=128, path="exact")
    for k in ("dx", "ddt", "da", "db", "dc", "dd", "dh0"):
        assert torch.isfinite(got[k]).all(), k
        assert rel_l2(host(got[k]), host(want[k])) <= 2e-2, (k, rel_l2(host(got[k]), host(want[k])))
    bare = list(args)
    bare[5] = bare[6] = bare[8] = None
    got = bm.ops.ssd2_bwd(*bare, chunk_len=128, path="tensor", check_status=True)
    want = bm.ops.ssd2_bwd(*bare, chunk_len=128, path="exact")
    for k in ("dx", "ddt", "da", "db", "dc", "dh0"):
        assert rel_l2(host(got[k]), host(want[k])) <= 2e-2, (k, rel_l2(host(got[k]), host(want[k])))


def test_ssd2_backward_tensor_path_refuses_what_it_does_not_cover(bm):
    cfg = inputs.ssd2_prefill(seed=37, batch=1, seqlen=64, nheads=2, headdim=32, state_rank=64, h0_std=0.1)
    _, args = _bwd_inputs(cfg, 13)
    with pytest.raises(RuntimeError):
        bm.ops.ssd2_bwd(*args, chunk_len=64, path="tensor")
    bm.ops.ssd2_bwd(*args, chunk_len=64, path="auto")   # falls back to the exact path


@pytest.mark.parametrize("b,s,h,p,r,m,Q", [(2, 12, 2, 8, 8, 1, 4), (2, 10, 2, 8, 8, 2, 4), (1, 40, 2, 16, 32, 3, 16),
                                           (1, 64, 2, 64, 128, 4, 32)])
def test_ssd3_backward_matches_autodiff_oracle(bm, b, s, h, p, r, m, Q):
    """src/mamba3/single_ssd/ssd/ssd_path/tests.rs:175-339 (incl. d_gamma, d_scale) and the generic core."""
    from oracle import backward
    cfg = inputs.ssd3_single(seed=60 + s, batch=b, seqlen=s, nheads=h, headdim=p, state_rank=r, mimo_rank=m, h0_std=0.2)
    rng = np.random.default_rng(2)
    dy = rng.standard_normal(cfg["v"].shape).astype(np.float32)
    dhf = rng.standard_normal(cfg["h0"].shape).astype(np.float32)
    args = (cfg["v"], cfg["da"], cfg["b"], cfg["c"], cfg["gamma"], cfg["scale"], cfg["h0"])
    want = backward.ssd3_grads(*args, dy, dhf, Q, single=True)
    got = bm.ops.ssd3_bwd(*(dev(t) for t in args), dev(dy), dev(dhf), chunk_len=Q, single=True)
    for k in ("dv", "dda", "db", "dc", "dgamma", "dscale", "dh0"):
        assert _grad_close(got[k], want[k]), ("single", k, rel_l2(host(got[k]), want[k]))
    want = backward.ssd3_grads(*args, dy, dhf, Q, single=False)
    got = bm.ops.ssd3_bwd(*(dev(t) for t in args), dev(dy), dev(dhf), chunk_len=Q, single=False)
    for k in ("dv", "dda", "db", "dc", "dh0"):
        assert _grad_close(got[k], want[k]), ("double", k, rel_l2(host(got[k]), want[k]))


@pytest.mark.parametrize("b,s,h,m", [(1, 128, 1, 1), (1, 64, 2, 2), (2, 160, 2, 4), (1, 75, 3, 4)])
def test_ssd3_backward_tensor_path_matches_autodiff_oracle(bm, b, s, h, m):
    """The tcgen05 backward of the Mamba-3 cores on the fused (time x rank) axis against autodiff of the serial
    forward on the same bf16-rounded inputs: single (with d_gamma, d_scale) and the generic core, MIMO ranks
    1 / 2 / 4, ragged lengths, initial state and dh_final."""
    from oracle import backward
    cfg = inputs.ssd3_single(seed=70 + s, batch=b, seqlen=s, nheads=h, headdim=64, state_rank=128, mimo_rank=m, h0_std=0.2)
    dt = torch.bfloat16
    v, bb, cc = (q(cfg[k], dt) for k in ("v", "b", "c"))
    rng = np.random.default_rng(3)
    dy = q(rng.standard_normal(v.shape).astype(np.float32), dt)
    dhf = rng.standard_normal(cfg["h0"].shape).astype(np.float32)
    args = (dev(v, dt), dev(cfg["da"]), dev(bb, dt), dev(cc, dt), dev(cfg["gamma"]), dev(cfg["scale"]), dev(cfg["h0"]),
            dev(dy, dt), dev(dhf))
    for single, keys in ((True, ("dv", "dda", "db", "dc", "dgamma", "dscale", "dh0")), (False, ("dv", "dda", "db", "dc", "dh0"))):
        want = backward.ssd3_grads(v, cfg["da"], bb, cc, cfg["gamma"], cfg["scale"], cfg["h0"], dy, dhf, 32, single=single)
        got = bm.ops.ssd3_bwd(*args, chunk_len=32, single=single, path="tensor", check_status=True)
        for k in keys:
            assert rel_l2(host(got[k]), want[k]) <= 2e-2, (single, k, rel_l2(host(got[k]), want[k]))


def test_ssd3_backward_tensor_path_cut_units_against_the_float32_backward(bm):
    """More units than SMs with MIMO rank 4: units straddle CTAs, dh crosses through the workspace; every
    gradient against the float32 backward on device."""
    cfg = inputs.ssd3_single(seed=71, batch=2, seqlen=320, nheads=160, headdim=64, state_rank=128, mimo_rank=4, h0_std=0.1)
    dt = torch.bfloat16
    rng = np.random.default_rng(4)
    dy = rng.standard_normal(cfg["v"].shape).astype(np.float32)
    args = (dev(cfg["v"], dt), dev(cfg["da"]), dev(cfg["b"], dt), dev(cfg["c"], dt), dev(cfg["gamma"]), dev(cfg["scale"]),
            dev(cfg["h0"]), dev(dy, dt), None)
    got = bm.ops.ssd3_bwd(*args, chunk_len=64, single=True, path="tensor", check_status=True)
    want = bm.ops.ssd3_bwd(*args, chunk_len=64, single=True, path="exact")
    for k in ("dv", "dda", "db", "dc", "dgamma", "dscale", "dh0"):
        assert rel_l2(host(got[k]), host(want[k])) <= 2e-2, (k, rel_l2(host(got[k]), host(want[k])))


# ------------------------------------------------------------------ Mamba-2 SSD, two heads per CTA (opt-in kernel)
def _pair_case(bm, cfg, Q, oracle=True):
    dt = torch.bfloat16
    x, bb, cc = (q(cfg[k], dt) for k in ("x", "b", "c"))
    args = (dev(x, dt), dev(cfg["dt"]), dev(cfg["a"]), dev(bb, dt), dev(cc, dt), dev(cfg["d"]), dev(cfg["h0"]))
    y, hf = bm.ops.ssd2_fwd(*args, chunk_len=Q, path="tensor_pair", check_status=True)
    ye, he = bm.ops.ssd2_fwd(*args, chunk_len=Q, path="exact")
    assert torch.isfinite(y.float()).all() and torch.isfinite(hf).all()
    assert rel_l2(host(y), host(ye)) <= 2e-2 and rel_l2(host(hf), host(he)) <= 2e-2
    if oracle:
        want_y, want_h = mamba2.ssd_serial(x, cfg["dt"], cfg["a"], bb, cc, cfg["d"], cfg["h0"], Q)
        assert rel_l2(host(y), want_y) <= 2e-2 and rel_l2(host(hf), want_h) <= 2e-2


@pytest.mark.parametrize("b,s,h,g,Q", [
    (1, 128, 2, 1, 128),     # one pair, one tile
    (2, 512, 4, 2, 256),     # two groups
    (1, 300, 2, 1, 128),     # ragged tail (rows past the end are clipped by the store)
    (1, 100, 2, 1, 64),      # shorter than one tile
    (1, 4096, 4, 1, 256),    # long sequence
])
def test_ssd2_pair_kernel_matches_oracle(bm, b, s, h, g, Q):
    cfg = inputs.ssd2_prefill(seed=400 + s, batch=b, seqlen=s, nheads=h, headdim=64, state_rank=128, ngroups=g,
                              h0_std=0.1)
    _pair_case(bm, cfg, Q)


def test_ssd2_pair_kernel_segments_and_many_pairs(bm):
    """More pairs than SMs and a sequence long enough to be cut into segments whose state is handed from CTA to
    CTA through the workspace; every unit against the float32 exact path on device."""
    _pair_case(bm, inputs.ssd2_prefill(seed=41, batch=3, seqlen=384, nheads=160, headdim=64, state_rank=128), 256, oracle=False)
    _pair_case(bm, inputs.ssd2_prefill(seed=42, batch=4, seqlen=4096, nheads=80, headdim=64, state_rank=128), 256, oracle=False)


def test_ssd2_pair_kernel_strong_zero_and_tiny_steps(bm):
    """Decay far beyond what one pass represents (the tile is walked in sub-ranges), steps of exactly zero, and
    steps below the kernel's step floor: results stay finite and within tolerance, D x passes through."""
    cfg = inputs.ssd2_prefill(seed=43, batch=1, seqlen=256, nheads=2, headdim=64, state_rank=128, h0_std=0.1)
    cfg["dt"] = (cfg["dt"] * 0 + 3.0).astype(np.float32)
    cfg["a"] = np.float32([-16.0, -0.001])
    _pair_case(bm, cfg, 256)
    cfg = inputs.ssd2_prefill(seed=44, batch=1, seqlen=384, nheads=4, headdim=64, state_rank=128, h0_std=0.1)
    cfg["dt"][:, 5::7, :] = 0.0
    cfg["dt"][:, 200:300, 1] = 0.0
    _pair_case(bm, cfg, 128)
    cfg = inputs.ssd2_prefill(seed=45, batch=2, seqlen=1024, nheads=6, headdim=64, state_rank=128, h0_std=0.1)
    cfg["a"] = np.float32([-0.5, -16.0, -1.0, -12.0, -0.01, -8.0])
    rng = np.random.default_rng(7)
    cfg["dt"] = (rng.random(cfg["dt"].shape) * np.float32([0.01, 0.8, 0.02, 0.5, 0.05, 0.3])).astype(np.float32)
    cfg["dt"][:, 512:640] *= 40.0
    _pair_case(bm, cfg, 256)
    cfg = inputs.ssd2_prefill(seed=46, batch=1, seqlen=256, nheads=2, headdim=64, state_rank=128, h0_std=0.1)
    cfg["a"] = np.float32([-1.0, -1.0])
    dtv = np.full((1, 256, 2), 95.0 / (128 * 1.4426950408889634), np.float32)
    dtv[0, 0, 0], dtv[0, 128, 1] = 1e-9, 1e-30
    cfg["dt"] = dtv
    _pair_case(bm, cfg, 128)


def test_ssd2_pair_kernel_refuses_odd_heads_per_group(bm):
    cfg = inputs.ssd2_prefill(seed=47, batch=1, seqlen=128, nheads=3, headdim=64, state_rank=128, ngroups=1)
    t = {k: dev(v, torch.bfloat16 if k in ("x", "b", "c") else None) for k, v in cfg.items()}
    with pytest.raises(bm.BmError) as e:
        bm.ops.ssd2_fwd(t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], None, chunk_len=128, path="tensor_pair")
    assert e.value.code == bm._ffi.BM_ERR_UNSUPPORTED


# ------------------------------------------------------------------ Mamba-3 cores, tensor-core path
@pytest.mark.parametrize("b,s,h,m,double,fused,strong", [
    (1, 32, 2, 4, False, True, False),      # one tile of the fused (time x rank) axis
    (1, 100, 2, 4, False, True, False),     # ragged
    (1, 100, 2, 4, False, False, False),    # pre-rotated B / C, no angles
    (2, 300, 2, 1, False, True, False),     # SISO: pairwise rotation, the same-step block is the diagonal
    (1, 130, 3, 2, False, True, False),
    (1, 100, 2, 4, True, True, False),      # generic core (one pass of the double-SSD pathway)
    (1, 200, 2, 1, True, True, False),
    (1, 128, 2, 4, False, True, True),      # decay beyond the factored form's range: exact mask form
    (1, 256, 2, 1, False, True, True),
])
def test_ssd3_tensor_path_matches_oracle(bm, b, s, h, m, double, fused, strong):
    """bm_ssd3_single_fwd / bm_ssd3_double_fwd on the tcgen05 kernel (strict-in-time mask over the fused axis, column
    scale, same-step gamma block; src/mamba3/single_ssd/ssd/serial.rs:156-268, double_ssd/ssd/serial.rs:118-409)."""
    BF = torch.bfloat16
    cfg = inputs.ssd3_single(seed=70 + s, batch=b, seqlen=s, nheads=h, headdim=64, state_rank=128, mimo_rank=m, h0_std=0.1)
    if strong:
        cfg["da"] = (cfg["da"] * 40).astype(np.float32)
    v, bb, cc = (bf16_round(cfg[k]) for k in ("v", "b", "c"))
    ang = cfg["angles"][:, :, None]
    b_rot = mamba3.apply_rope_partial(bb, ang, 128, m == 1)
    c_rot = mamba3.apply_rope_partial(cc, ang, 128, m == 1)
    if double:
        want_y, want_h = mamba3.double_ssd_serial(v, cfg["da"], b_rot, c_rot, cfg["h0"], 64)
    else:
        want_y, want_h = mamba3.single_ssd_serial(v, cfg["da"], b_rot, c_rot, cfg["gamma"], cfg["scale"], cfg["h0"], 64)
    if fused:
        a = (dev(v, BF), dev(cfg["da"]), dev(bb, BF), dev(cc, BF))
        kw = dict(angles=dev(cfg["angles"]), rope_dim=128)
    else:
        a = (dev(v, BF), dev(cfg["da"]), dev(bf16_round(b_rot), BF), dev(bf16_round(c_rot), BF))
        kw = {}
    if double:
        y, hf = bm.ops.ssd3_double_fwd(*a, dev(cfg["h0"]), chunk_len=64, path="tensor", check_status=True, **kw)
    else:
        y, hf = bm.ops.ssd3_single_fwd(*a, dev(cfg["gamma"]), dev(cfg["scale"]), dev(cfg["h0"]), chunk_len=64, path="tensor",
                                       check_status=True, **kw)
    assert torch.isfinite(y.float()).all()
    assert rel_l2(host(y), want_y) <= 2e-2 and rel_l2(host(hf), want_h) <= 2e-2


@pytest.mark.parametrize("m,rope", [(4, 128), (4, 64), (1, 96), (2, 128)])
def test_ssd3_tensor_path_rotation_in_kernel_with_units_cut_between_ctas(bm, m, rope):
    """More units than SMs (tile ranges cut units between CTAs, the rotating warpgroups walk one tile ahead across
    those cuts), full and partial rope_dim, all three MIMO ranks: the in-kernel rotation against the float32 path,
    which rotates at load, on the same raw B / C and angles."""
    BF = torch.bfloat16
    cfg = inputs.ssd3_single(seed=75 + m, batch=2, seqlen=96, nheads=160, headdim=64, state_rank=128, mimo_rank=m, h0_std=0.1)
    ang = dev(np.ascontiguousarray(cfg["angles"][..., :rope // 2]))
    a = (dev(cfg["v"], BF), dev(cfg["da"]), dev(cfg["b"], BF), dev(cfg["c"], BF), dev(cfg["gamma"]), dev(cfg["scale"]),
         dev(cfg["h0"]))
    y, hf = bm.ops.ssd3_single_fwd(*a, chunk_len=32, path="tensor", check_status=True, angles=ang, rope_dim=rope)
    ye, he = bm.ops.ssd3_single_fwd(*a, chunk_len=32, path="exact", angles=ang, rope_dim=rope)
    assert torch.isfinite(y.float()).all()
    assert rel_l2(host(y), host(ye)) <= 2e-2 and rel_l2(host(hf), host(he)) <= 2e-2


def test_ssd3_tensor_path_refuses_what_it_does_not_cover(bm):
    cfg = inputs.ssd3_single(seed=71, batch=1, seqlen=16, nheads=2, headdim=16, state_rank=32, mimo_rank=3)
    t = {k: dev(cfg[k]) for k in ("v", "da", "b", "c", "gamma", "scale")}
    with pytest.raises(bm.BmError) as e:
        bm.ops.ssd3_single_fwd(t["v"], t["da"], t["b"], t["c"], t["gamma"], t["scale"], None, chunk_len=16, path="tensor")
    assert e.value.code == bm._ffi.BM_ERR_UNSUPPORTED
