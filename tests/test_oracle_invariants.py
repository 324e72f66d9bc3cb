"""Oracle self-checks (CPU): the invariants the reference's own tests assert, applied to the oracle.

The reference holds no golden vectors, so these properties -- at the reference's tiny shapes and
tolerances -- are what anchors the restatement (see oracle/__init__.py).
"""
import numpy as np
import pytest

from oracle import mamba1, mamba2, mamba3
from oracle.numerics import softplus, bf16_round, to_bf16_bits, from_bf16_bits


def _m2_inputs(rng, b=2, s=12, h=4, p=8, r=8, g=1, dtype=np.float64):
    # distributions of src/mamba2/ssd/ssd_path/tests.rs:15-68
    x = rng.standard_normal((b, s, h, p)).astype(dtype)
    dt = rng.uniform(0.05, 0.3, (b, s, h)).astype(dtype)
    a = rng.uniform(-1.0, -0.5, h).astype(dtype)
    bm = rng.standard_normal((b, s, g, r)).astype(dtype)
    cm = rng.standard_normal((b, s, g, r)).astype(dtype)
    d = (0.1 * rng.standard_normal(h)).astype(dtype)
    h0 = (0.1 * rng.standard_normal((b, h, p, r))).astype(dtype)
    return x, dt, a, bm, cm, d, h0


@pytest.mark.parametrize("s,q,g", [(4, 4, 1), (12, 4, 1), (12, 4, 2), (10, 4, 1), (7, 16, 4)])
@pytest.mark.parametrize("dtype,tol", [(np.float64, 1e-10), (np.float32, 1e-4)])
def test_m2_minimal_serial_recurrence_agree(s, q, g, dtype, tol):
    """Minimal == Serial (src/mamba2/ssd/ssd_path/tests.rs:184-336), both == step unroll."""
    rng = np.random.default_rng(0)
    args = _m2_inputs(rng, s=s, g=g, dtype=dtype)
    y_s, f_s = mamba2.ssd_serial(*args, chunk_len=q)
    y_m, f_m = mamba2.ssd_minimal(*args, chunk_len=q)
    y_r, f_r = mamba2.ssd_recurrence(*args)
    for a_, b_ in ((y_s, y_m), (f_s, f_m), (y_s, y_r), (f_s, f_r)):
        assert np.max(np.abs(a_ - b_)) < tol


def test_m2_chunk_len_independence():
    rng = np.random.default_rng(1)
    args = _m2_inputs(rng, s=32)
    ref = mamba2.ssd_serial(*args, chunk_len=32)
    for q in (1, 2, 8, 16, 5):
        out = mamba2.ssd_serial(*args, chunk_len=q)
        assert np.max(np.abs(out[0] - ref[0])) < 1e-10 and np.max(np.abs(out[1] - ref[1])) < 1e-10


def test_m2_initial_state_is_consumed():
    """src/mamba2/mamba2/tests.rs:258-271."""
    rng = np.random.default_rng(2)
    x, dt, a, bm, cm, d, h0 = _m2_inputs(rng)
    y1, _ = mamba2.ssd_serial(x, dt, a, bm, cm, d, h0, 4)
    y0, _ = mamba2.ssd_serial(x, dt, a, bm, cm, d, np.zeros_like(h0), 4)
    assert np.max(np.abs(y1 - y0)) > 1e-3


@pytest.mark.parametrize("g", [1, 2])
def test_m2_block_forward_equals_steps_and_split(g):
    """forward == unrolled step (src/mamba2/mamba2/tests.rs:202-252) and split == full (:343-392)."""
    rng = np.random.default_rng(3)
    w = mamba2.Mamba2Weights(rng, d_model=16, d_inner=32, nheads=4, state_rank=8, ngroups=g, dtype=np.float64)
    bsz, s = 2, 11
    u = rng.standard_normal((bsz, s, 16))
    conv0 = 0.1 * rng.standard_normal((bsz, w.conv_dim, 4))
    ssm0 = 0.1 * rng.standard_normal((bsz, 4, 8, 8))
    out, conv, ssm, _ = mamba2.block_forward(w, u, conv0, ssm0, chunk_len=4)
    c, h = conv0, ssm0
    for t in range(s):
        o, c, h = mamba2.block_step(w, u[:, t], c, h)
        assert np.max(np.abs(o - out[:, t])) < 1e-9
    assert np.max(np.abs(c - conv)) < 1e-12 and np.max(np.abs(h - ssm)) < 1e-9
    o1, c1, h1, _ = mamba2.block_forward(w, u[:, :5], conv0, ssm0, chunk_len=4)
    o2, c2, h2, _ = mamba2.block_forward(w, u[:, 5:], c1, h1, chunk_len=4)
    assert np.max(np.abs(np.concatenate([o1, o2], 1) - out)) < 1e-9
    assert np.max(np.abs(c2 - conv)) < 1e-12 and np.max(np.abs(h2 - ssm)) < 1e-9


def test_m2_optimal_chunk_len():
    assert mamba2.optimal_chunk_len(64, 64) == 64
    assert mamba2.optimal_chunk_len(128, 64) == 96
    assert mamba2.optimal_chunk_len(8, 8) == 32


def test_m1_forward_equals_steps_and_split():
    """src/mamba1/mamba1/tests.rs:216-265, :384-427."""
    rng = np.random.default_rng(4)
    w = mamba1.Mamba1Weights(rng, d_model=12, d_inner=24, state_rank=4, dtype=np.float64)
    bsz, s = 2, 9
    x = rng.standard_normal((bsz, s, 12))
    conv0 = 0.1 * rng.standard_normal((bsz, 24, 4))
    ssm0 = 0.1 * rng.standard_normal((bsz, 24, 4))
    out, conv, ssm, _ = mamba1.block_forward(w, x, conv0, ssm0)
    c, h = conv0, ssm0
    for t in range(s):
        o, c, h = mamba1.block_step(w, x[:, t], c, h)
        assert np.max(np.abs(o - out[:, t])) < 1e-10
    assert np.max(np.abs(h - ssm)) < 1e-10 and np.max(np.abs(c - conv)) < 1e-12
    o1, c1, h1, _ = mamba1.block_forward(w, x[:, :4], conv0, ssm0)
    o2, c2, h2, _ = mamba1.block_forward(w, x[:, 4:], c1, h1)
    assert np.max(np.abs(np.concatenate([o1, o2], 1) - out)) < 1e-10


def test_m3_mimo_outer_sum_matches_loops():
    """src/mamba3/helpers/tests.rs:13-72 (tolerance 1e-5)."""
    rng = np.random.default_rng(5)
    v = rng.standard_normal((2, 3, 2, 4)).astype(np.float32)
    k = rng.standard_normal((2, 3, 2, 5)).astype(np.float32)
    assert np.max(np.abs(mamba3.mimo_outer_sum(v, k) - mamba3.mimo_outer_sum_loops(v, k))) < 1e-5


def test_m3_angle_increment_formula():
    """src/mamba3/rotation/tests.rs:1238-1248: at range 1 the increment is dt * pi * tanh(rot)."""
    rng = np.random.default_rng(6)
    rot = rng.standard_normal((2, 5, 3)).astype(np.float32)
    dt = rng.uniform(0.01, 0.2, (2, 5, 4)).astype(np.float32)
    inc = mamba3.angle_increment(rot, dt, 1.0)
    want = dt[..., :, None] * (np.pi * np.tanh(rot))[..., None, :]
    assert inc.shape == (2, 5, 4, 3) and np.max(np.abs(inc - want)) < 1e-6


def test_m3_wrap_angle_range_and_rotation_invariance():
    t = np.linspace(-50, 50, 1001).astype(np.float32)
    w = mamba3.wrap_angle(t)
    assert np.all(np.abs(w) <= np.pi + 1e-5)
    assert np.max(np.abs(np.cos(w) - np.cos(t.astype(np.float64)))) < 1e-4


@pytest.mark.parametrize("m,g,rope_fraction", [(1, 1, 1.0), (2, 1, 1.0), (2, 2, 0.5), (1, 1, 0.5), (1, 1, 0.0)])
def test_m3_forward_single_double_step_agree(m, g, rope_fraction):
    """single == double (src/mamba3/single_ssd/single_ssd/tests.rs:374-428), forward == unrolled step
    (src/mamba3/double_ssd/double_ssd/tests.rs:259-307, + mimo/ngroups2/rope half/zero :380-494),
    split == full (src/mamba3/single_ssd/single_ssd/tests.rs:592-666)."""
    rng = np.random.default_rng(7)
    w = mamba3.Mamba3Weights(rng, d_model=16, d_inner=32, nheads=4, state_rank=8, ngroups=g, mimo_rank=m,
                             rope_fraction=rope_fraction, dtype=np.float64)
    w.b_bias = w.b_bias + 0.3 * rng.standard_normal(w.b_bias.shape)
    w.c_bias = w.c_bias + 0.3 * rng.standard_normal(w.c_bias.shape)
    if m > 1:
        w.mimo_x = w.mimo_x + 0.2 * rng.standard_normal(w.mimo_x.shape)
        w.mimo_z = w.mimo_z + 0.2 * rng.standard_normal(w.mimo_z.shape)
        w.mimo_o = w.mimo_o + 0.2 * rng.standard_normal(w.mimo_o.shape)
    bsz, s = 2, 10
    u = rng.standard_normal((bsz, s, 16))
    cache = mamba3.zero_cache(w, bsz, np.float64)
    cache = {k: v + 0.1 * rng.standard_normal(v.shape) for k, v in cache.items()}
    o_s, c_s, _ = mamba3.block_forward_single(w, u, cache, chunk_len=4)
    o_d, c_d = mamba3.block_forward_double(w, u, cache, chunk_len=4)
    assert np.max(np.abs(o_s - o_d)) < 1e-9
    for k in c_s:
        assert np.max(np.abs(c_s[k] - c_d[k])) < 1e-9, k
    c = cache
    for t in range(s):
        o, c = mamba3.block_step(w, u[:, t], c)
        assert np.max(np.abs(o - o_s[:, t])) < 1e-9
    for k in c_s:
        diff = c[k] - c_s[k]
        if k == "angle":
            diff = np.angle(np.exp(1j * diff))
        assert np.max(np.abs(diff)) < 1e-8, k
    o1, c1, _ = mamba3.block_forward_single(w, u[:, :6], cache, chunk_len=4)
    o2, c2, _ = mamba3.block_forward_single(w, u[:, 6:], c1, chunk_len=4)
    assert np.max(np.abs(np.concatenate([o1, o2], 1) - o_s)) < 1e-9


def test_m3_recurrence_matches_slot():
    rng = np.random.default_rng(8)
    w = mamba3.Mamba3Weights(rng, d_model=16, d_inner=32, nheads=4, state_rank=8, mimo_rank=2, dtype=np.float64)
    u = rng.standard_normal((2, 9, 16))
    cache = {k: v + 0.1 * rng.standard_normal(v.shape) for k, v in mamba3.zero_cache(w, 2, np.float64).items()}
    _, _, slot = mamba3.block_forward_single(w, u, cache, chunk_len=4)
    y, hf = mamba3.recurrence(slot["x"], slot["b"], slot["c"], slot["alpha"], slot["beta"], slot["gamma"],
                              cache["ssm"], cache["v"], cache["k"], w.mimo_x)
    assert np.max(np.abs(y - slot["y"])) < 1e-9 and np.max(np.abs(hf - slot["final"])) < 1e-9


def test_softplus_thresholds_and_bf16_helpers():
    x = np.array([-3.0, 0.0, 6.9, 7.1, 17.9, 18.1], np.float32)
    assert softplus(x, "bf16")[3] == x[3] and softplus(x, "f32")[3] != x[3] and softplus(x, "f32")[5] == x[5]
    v = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.1415927], np.float32)
    assert np.array_equal(from_bf16_bits(to_bf16_bits(v)), bf16_round(v))
    assert bf16_round(np.float32([1.00390625]))[0] == 1.0  # tie rounds to even


def test_c_port_matches_numpy_oracle():
    """The timed CPU baseline (C restatement) agrees with the numpy oracle."""
    from oracle import cport, inputs
    from oracle.numerics import rel_l2
    cfg = inputs.ssd2_prefill(seed=3, batch=2, seqlen=128, nheads=4, headdim=16, state_rank=32, ngroups=2, h0_std=0.1)
    y, hf = cport.ssd2_serial(cfg["x"], cfg["dt"], cfg["a"], cfg["b"], cfg["c"], cfg["d"], cfg["h0"], 32)
    wy, wh = mamba2.ssd_serial(*(cfg[k].astype(np.float64) for k in ("x", "dt", "a", "b", "c", "d", "h0")), 32)
    assert rel_l2(y, wy) < 1e-5 and rel_l2(hf, wh) < 1e-5
    st = inputs.step2_decode(seed=3, batch=3, nheads=4, headdim=8, state_rank=16, steps=1)
    state = st["state"].copy()
    y = cport.step2(state, st["x"][0], st["dt"][0], st["a"], st["b"][0], st["c"][0], st["d"])
    wy, wh = mamba2.ssm_step(st["state"], st["x"][0], st["dt"][0], st["a"], st["b"][0], st["c"][0], st["d"])
    assert rel_l2(y, wy) < 1e-5 and rel_l2(state, wh) < 1e-6
    sc = inputs.selscan1(seed=2, batch=2, seqlen=50, d_inner=12, state_rank=8)
    y, hf = cport.selscan1(sc["u"], sc["delta"], sc["a"], sc["b"], sc["c"], sc["d"], sc["h0"])
    wy, wh = mamba1.selective_scan(sc["delta"], sc["a"], sc["b"], sc["c"], sc["d"], sc["u"], sc["h0"], dtype=np.float64)
    assert rel_l2(y, wy) < 1e-5 and rel_l2(hf, wh) < 1e-5


def test_backward_oracle_forward_matches_numpy_and_finite_differences():
    """The torch restatement used for autodiff equals the numpy oracle, and its gradients equal central
    finite differences of the numpy oracle (an autodiff-free check)."""
    import torch
    from oracle import backward, inputs
    cfg = inputs.ssd2_prefill(seed=9, batch=1, seqlen=10, nheads=2, headdim=3, state_rank=4, ngroups=1, h0_std=0.3)
    arr = {k: cfg[k].astype(np.float64) for k in ("x", "dt", "a", "b", "c", "d", "h0")}
    rng = np.random.default_rng(0)
    dy = rng.standard_normal(arr["x"].shape)
    dhf = rng.standard_normal(arr["h0"].shape)
    y_t, h_t = backward.ssd2_forward_torch(*(torch.tensor(arr[k]) for k in ("x", "dt", "a", "b", "c", "d", "h0")), 4)
    y_n, h_n = mamba2.ssd_serial(arr["x"], arr["dt"], arr["a"], arr["b"], arr["c"], arr["d"], arr["h0"], 4)
    assert np.max(np.abs(y_t.numpy() - y_n)) < 1e-12 and np.max(np.abs(h_t.numpy() - h_n)) < 1e-12
    g = backward.ssd2_grads(arr["x"], arr["dt"], arr["a"], arr["b"], arr["c"], arr["d"], arr["h0"], dy, dhf, 4)

    def loss(**a):
        y, h = mamba2.ssd_serial(a["x"], a["dt"], a["a"], a["b"], a["c"], a["d"], a["h0"], 4)
        return float((y * dy).sum() + (h * dhf).sum())

    for name, key, idx in (("x", "dx", (0, 3, 1, 2)), ("dt", "ddt", (0, 5, 1)), ("a", "da", (1,)), ("b", "db", (0, 2, 0, 3)),
                           ("c", "dc", (0, 7, 0, 1)), ("d", "dd", (0,)), ("h0", "dh0", (0, 1, 2, 3))):
        fd = backward.finite_difference(loss, arr, name, idx)
        assert abs(fd - g[key][idx]) < 1e-6 * max(1.0, abs(fd)), (name, fd, g[key][idx])


def test_backward_oracle_m3_single_equals_double_gradients():
    """single-SSD == double-SSD on gradients (src/mamba3/single_ssd/single_ssd/tests.rs:374-428), at the core
    level: with scale = gamma (no look-ahead term) and a strict mask + gamma diagonal, the single core on v
    equals the generic core on gamma*v, so their gradients with respect to B, C, da, h0 agree."""
    from oracle import backward
    rng = np.random.default_rng(3)
    b, s, m, h, p, r = 1, 9, 2, 2, 3, 4
    v = rng.standard_normal((b, s, m, h, p))
    bm = rng.standard_normal((b, s, m, h, r))
    cm = rng.standard_normal((b, s, m, h, r))
    da = -rng.uniform(0.05, 0.3, (b, s, h))
    gamma = rng.uniform(0.1, 0.5, (b, s, h))
    h0 = 0.1 * rng.standard_normal((b, h, p, r))
    dy = rng.standard_normal(v.shape)
    dhf = rng.standard_normal(h0.shape)
    g1 = backward.ssd3_grads(v, da, bm, cm, gamma, gamma, h0, dy, dhf, 4, single=True)
    g2 = backward.ssd3_grads(v * gamma[:, :, None, :, None], da, bm, cm, None, None, h0, dy, dhf, 4, single=False)
    for k in ("dda", "db", "dc", "dh0"):
        assert np.max(np.abs(g1[k] - g2[k])) < 1e-9, k
    assert np.max(np.abs(g1["dv"] - g2["dv"] * gamma[:, :, None, :, None])) < 1e-9


def test_backward_oracle_m3_chain_agrees_with_finite_differences_and_the_closed_form_chain():
    """The forward + backward configuration's chain (dt, A, lambda, theta -> da, gamma, scale, rotated B / C):
    autodiff of the whole chain == central differences, and == the closed form that the GPU test harness
    applies to the slot's gradients (ddt_t = A d_da_t + lambda_t (d_gamma_t + d_scale_t) + (1 - lambda_t) d_scale_{t-1})."""
    from oracle import backward, mamba3
    rng = np.random.default_rng(8)
    b, s, m, h, p, r, Q = 1, 7, 2, 2, 3, 4, 4
    arr = dict(x=rng.standard_normal((b, s, h, p)), b=rng.standard_normal((b, s, m, h, r)),
               c=rng.standard_normal((b, s, m, h, r)), dt=rng.uniform(0.05, 0.3, (b, s, h)), a=-rng.uniform(1, 4, h))
    lam = rng.uniform(0.2, 0.8, (b, s, h))
    theta = rng.standard_normal((b, s, h, r // 2))
    h0 = 0.1 * rng.standard_normal((b, h, p, r))
    dy = rng.standard_normal((b, s, m, h, p))
    dhf = rng.standard_normal(h0.shape)
    g = backward.ssd3_single_chain_grads(arr["x"], arr["b"], arr["c"], arr["dt"], arr["a"], lam, theta, h0, dy, dhf, Q, m)

    def slot_inputs(a):
        v = np.repeat(a["x"][:, :, None] / m, m, axis=2)
        da = a["dt"] * a["a"][None, None]
        gamma = lam * a["dt"]
        scale = gamma.copy()
        scale[:, :-1] += ((1 - lam) * a["dt"])[:, 1:]
        ang = theta[:, :, None]
        return (v, da, mamba3.apply_rope_partial(a["b"], ang, r, False), mamba3.apply_rope_partial(a["c"], ang, r, False),
                gamma, scale)

    def loss(**a):
        y, hf = mamba3.single_ssd_serial(*slot_inputs(a), h0, Q)
        return float((y * dy).sum() + (hf * dhf).sum())

    for name, key, idx in (("x", "dx", (0, 3, 1, 2)), ("dt", "ddt", (0, 2, 1)), ("dt", "ddt", (0, 6, 0)), ("a", "dA", (1,)),
                           ("b", "dB", (0, 2, 1, 0, 3)), ("c", "dC", (0, 5, 0, 1, 1))):
        fd = backward.finite_difference(loss, arr, name, idx)
        assert abs(fd - g[key][idx]) < 1e-6 * max(1.0, abs(fd)), (name, fd, g[key][idx])
    # closed-form chain on the slot's own gradients
    sg = backward.ssd3_grads(*slot_inputs(arr), h0, dy, dhf, Q, single=True)
    prev = np.concatenate([np.zeros_like(sg["dscale"][:, :1]), sg["dscale"][:, :-1]], axis=1)
    ddt = arr["a"][None, None] * sg["dda"] + lam * (sg["dgamma"] + sg["dscale"]) + (1 - lam) * prev
    assert np.max(np.abs(ddt - g["ddt"])) < 1e-6
    assert np.max(np.abs((sg["dda"] * arr["dt"]).sum((0, 1)) - g["dA"])) < 1e-6
    ang = theta[:, :, None]
    assert np.max(np.abs(mamba3.apply_rope_partial(sg["db"], -ang, r, False) - g["dB"])) < 1e-6
    assert np.max(np.abs(sg["dv"].sum(2) / m - g["dx"])) < 1e-6
