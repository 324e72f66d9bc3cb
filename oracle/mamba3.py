"""Mamba-3 oracle: trapezoid coefficients, QK-norm, Complex2D rotation, single/double SSD, step.

Test infrastructure (see oracle/__init__.py).  Extra shape letters: m mimo rank, a rope angles.
All sequence tensors are flat ``[b, s, ...]``; the reference's ``[b, n, l, ...]`` is a reshape.
"""
import numpy as np

from .numerics import softplus, sigmoid, silu, rms_norm
from .mamba2 import gqa_expand


# ---------------------------------------------------------------------------------------------
# coefficients, QK-norm, rotation
# ---------------------------------------------------------------------------------------------
def trapezoidal_coefficients(dd_dt, dd_a_raw, lambda_raw, dt_bias_h, dt_limit=(0.0, 65504.0), a_floor=1e-4,
                             dtype_name="f32"):
    """src/mamba3/helpers.rs:42-73.  Returns dict(dt, da, alpha, beta, gamma, lam)."""
    dt = np.clip(softplus(dd_dt + dt_bias_h, dtype_name), *dt_limit).astype(dd_dt.dtype)
    a = -np.maximum(softplus(dd_a_raw, dtype_name), a_floor)
    da = dt * a
    lam = sigmoid(lambda_raw)
    alpha = np.exp(da)
    beta = (1.0 - lam) * dt * alpha
    gamma = lam * dt
    return dict(dt=dt, da=da, alpha=alpha, beta=beta, gamma=gamma, lam=lam)


def single_ssd_scale(gamma_bsh, dt_bsh, lam_bsh):
    """scale_t = gamma_t + (1 - lambda_{t+1}) dt_{t+1}; the last position keeps gamma
    (src/mamba3/single_ssd/single_ssd/mod.rs:134-149)."""
    shifted = np.zeros_like(gamma_bsh)
    shifted[:, :-1] = dt_bsh[:, 1:] * (1.0 - lam_bsh[:, 1:])
    return gamma_bsh + shifted


def qk_norm_expand_bias(raw_mgr, gamma_r, bias_hmr, nheads, dtype_name="f32"):
    """RMSNorm over r, group->head expansion, + bias[h, m, r] (src/mamba3/helpers.rs:82-95).
    raw: [..., m, g, r] -> [..., m, h, r]."""
    normed = rms_norm(raw_mgr, gamma_r, dtype_name)
    expanded = gqa_expand(normed, nheads)
    return expanded + bias_hmr.transpose(1, 0, 2)


def wrap_angle(t):
    """theta - round(theta / 2pi) * 2pi in float32 constants (src/modules/misc/rope.rs:23-27)."""
    two_pi = t.dtype.type(2.0 * np.float32(np.pi))
    k = np.round(t * (t.dtype.type(1.0) / two_pi))
    return t - k * two_pi


def angle_increment(rot_a, dt_h, rng):
    """dt[..., h, None] * (range * pi * tanh(rot))[..., None, a] (src/mamba3/rotation/mod.rs:559-567)."""
    bounded = np.tanh(rot_a) * rot_a.dtype.type(rng * np.pi)
    return dt_h[..., :, None] * bounded[..., None, :]


def apply_rope_partial(x, angles, rope_dim, pairwise):
    """Rotate the leading rope_dim entries of the last axis (src/modules/misc/rope.rs:50-170).
    pairwise: pairs (2j, 2j+1); otherwise halves (j, j + r/2) with the first rope_dim/2 of each half.
    ``angles`` has last axis rope_dim/2 and is wrapped before cos/sin."""
    if rope_dim == 0:
        return x
    r = x.shape[-1]
    na = rope_dim // 2
    ang = wrap_angle(angles[..., :na])
    cos, sin = np.cos(ang), np.sin(ang)
    out = x.copy()
    if pairwise:
        x0, x1 = x[..., 0:rope_dim:2], x[..., 1:rope_dim:2]
        out[..., 0:rope_dim:2] = cos * x0 - sin * x1
        out[..., 1:rope_dim:2] = sin * x0 + cos * x1
    else:
        half = r // 2
        x0, x1 = x[..., :na], x[..., half:half + na]
        out[..., :na] = cos * x0 - sin * x1
        out[..., half:half + na] = sin * x0 + cos * x1
    return out


def rotate_bc_forward(rot_bsa, dt_bsh, prev_angle_bha, b_bsmhr, c_bsmhr, rope_dim, rng=2.0):
    """Complex2D branch of rotate_bc_forward (src/mamba3/rotation/mod.rs:653-679).
    Returns (b_rot, c_rot, last_angle_wrapped_bha, cum_angles_bsha)."""
    m = b_bsmhr.shape[2]
    inc = angle_increment(rot_bsa, dt_bsh, rng)  # b s h a
    cum = prev_angle_bha[:, None] + np.cumsum(inc, axis=1)
    pairwise = m == 1
    ang_m = cum[:, :, None]  # broadcast over m
    b_rot = apply_rope_partial(b_bsmhr, ang_m, rope_dim, pairwise)
    c_rot = apply_rope_partial(c_bsmhr, ang_m, rope_dim, pairwise)
    return b_rot, c_rot, wrap_angle(cum[:, -1]), cum


def rotate_bc_step(rot_ba, dt_bh, prev_angle_bha, b_bmhr, c_bmhr, rope_dim, rng=2.0):
    """Complex2D branch of rotate_bc_step (src/mamba3/rotation/mod.rs:729-764)."""
    m = b_bmhr.shape[1]
    new = wrap_angle(prev_angle_bha + angle_increment(rot_ba, dt_bh, rng))
    pairwise = m == 1
    return (apply_rope_partial(b_bmhr, new[:, None], rope_dim, pairwise),
            apply_rope_partial(c_bmhr, new[:, None], rope_dim, pairwise), new)


def mimo_outer_sum(v_bmhp, k_bmhr):
    """sum_m v[b,m,h,p] * k[b,m,h,r] -> [b,h,p,r] (src/mamba3/helpers.rs:113-140)."""
    return np.einsum("bmhp,bmhr->bhpr", v_bmhp, k_bmhr)


def mimo_outer_sum_loops(v_bmhp, k_bmhr):
    """The 5-deep host loop the reference tests mimo_outer_sum against (src/mamba3/helpers/tests.rs:13-72)."""
    bsz, m, h, p = v_bmhp.shape
    r = k_bmhr.shape[-1]
    out = np.zeros((bsz, h, p, r), v_bmhp.dtype)
    for b_ in range(bsz):
        for h_ in range(h):
            for p_ in range(p):
                for r_ in range(r):
                    acc = 0.0
                    for m_ in range(m):
                        acc += v_bmhp[b_, m_, h_, p_] * k_bmhr[b_, m_, h_, r_]
                    out[b_, h_, p_, r_] = acc
    return out


# ---------------------------------------------------------------------------------------------
# SSD cores (slot level).  v: [b,s,m,h,p]; b,c: [b,s,m,h,r] (per head, normed+biased+rotated);
# da, gamma, scale: [b,s,h]; h0: [b,h,p,r].
# ---------------------------------------------------------------------------------------------
def _pad(ts, s, chunk_len):
    pad = (-s) % chunk_len
    if not pad:
        return ts
    return [np.concatenate([t, np.zeros((t.shape[0], pad) + t.shape[2:], t.dtype)], axis=1) for t in ts]


def _mimo_k1_k4(v, da, kmat, h0, chunk_len):
    """K1 (cumsum of da), K3 (chunk state on the given, already scaled K) and K4 (state passing) of
    src/mamba3/double_ssd/ssd/serial.rs:118-303.  Returns (cum_bhnl, h_in_bnhpr, final)."""
    bsz, S, m, H, P = v.shape
    R = kmat.shape[-1]
    n, l = S // chunk_len, chunk_len
    cum = np.cumsum(da.reshape(bsz, n, l, H).transpose(0, 3, 1, 2), axis=3)  # bhnl
    aend = cum[..., -1]
    decay = np.exp(aend[..., None] - cum).transpose(0, 2, 3, 1)  # bnlh
    vc = v.reshape(bsz, n, l, m, H, P)
    kc = kmat.reshape(bsz, n, l, m, H, R)
    s_intra = np.einsum("bnlmhp,bnlmhr,bnlh->bnhpr", vc, kc, decay)
    run = h0.astype(v.dtype).copy()
    entering = []
    for i in range(n):
        entering.append(run)
        run = np.exp(aend[:, :, i])[:, :, None, None] * run + s_intra[:, i]
    return cum, np.stack(entering, axis=1), run


def double_ssd_serial(v_bsmhp, da_bsh, b_bsmhr, c_bsmhr, h0_bhpr, chunk_len):
    """Generic MIMO SSD on pre-scaled v: non-strict causal mask (s <= t), no dt inside
    (src/mamba3/double_ssd/ssd/serial.rs:56-409).  Returns (y_bsmhp, final_state)."""
    s = v_bsmhp.shape[1]
    v, da, bm, cm = _pad([v_bsmhp, da_bsh, b_bsmhr, c_bsmhr], s, chunk_len)
    bsz, S, m, H, P = v.shape
    R = bm.shape[-1]
    n, l = S // chunk_len, chunk_len
    cum, h_in, final = _mimo_k1_k4(v, da, bm, h0_bhpr, chunk_len)
    vc = v.reshape(bsz, n, l, m, H, P)
    bc = bm.reshape(bsz, n, l, m, H, R)
    cc = cm.reshape(bsz, n, l, m, H, R)
    cum_bnhl = cum.transpose(0, 2, 1, 3)
    y_off = np.einsum("bnlmhr,bnhpr->bnlmhp", cc, h_in) * np.exp(cum_bnhl).transpose(0, 1, 3, 2)[:, :, :, None, :, None]
    cb = np.einsum("bntmhr,bnsuhr->bnhtmsu", cc, bc)  # target (t,m), source (s,u)
    diff = cum_bnhl[..., :, None] - cum_bnhl[..., None, :]  # bnh t s
    upper = np.triu(np.ones((l, l), dtype=bool), k=1)
    decay = np.exp(np.where(upper, -np.inf, diff))
    y_in = np.einsum("bnhtmsu,bnhts,bnsuhp->bntmhp", cb, decay, vc)
    y = (y_off + y_in).reshape(bsz, S, m, H, P)[:, :s]
    return y.astype(v_bsmhp.dtype), final.astype(v_bsmhp.dtype)


def single_ssd_serial(v_bsmhp, da_bsh, b_bsmhr, c_bsmhr, gamma_bsh, scale_bsh, h0_bhpr, chunk_len):
    """Single-pass Mamba-3 SSD (src/mamba3/single_ssd/ssd/serial.rs:56-268): K2 on unscaled B, K3 on
    scale*B (:89-95), strictly-lower mask in time (:216-228), source-column scale (:231-241), and the
    same-step correction gamma_t (C_t B_t^T) V_t (src/mamba3/single_ssd/ssd/diag.rs:50-100).
    Returns (y_bsmhp, final_state h')."""
    s = v_bsmhp.shape[1]
    v, da, bm, cm, gam, sc = _pad([v_bsmhp, da_bsh, b_bsmhr, c_bsmhr, gamma_bsh, scale_bsh], s, chunk_len)
    bsz, S, m, H, P = v.shape
    R = bm.shape[-1]
    n, l = S // chunk_len, chunk_len
    kscaled = bm * sc[:, :, None, :, None]
    cum, h_in, final = _mimo_k1_k4(v, da, kscaled, h0_bhpr, chunk_len)
    vc = v.reshape(bsz, n, l, m, H, P)
    bc = bm.reshape(bsz, n, l, m, H, R)
    cc = cm.reshape(bsz, n, l, m, H, R)
    scc = sc.reshape(bsz, n, l, H)
    gc = gam.reshape(bsz, n, l, H)
    cum_bnhl = cum.transpose(0, 2, 1, 3)
    y_off = np.einsum("bnlmhr,bnhpr->bnlmhp", cc, h_in) * np.exp(cum_bnhl).transpose(0, 1, 3, 2)[:, :, :, None, :, None]
    cb = np.einsum("bntmhr,bnsuhr->bnhtmsu", cc, bc)
    diff = cum_bnhl[..., :, None] - cum_bnhl[..., None, :]
    upper_incl = np.triu(np.ones((l, l), dtype=bool), k=0)
    kern = np.exp(np.where(upper_incl, -np.inf, diff)) * scc.transpose(0, 1, 3, 2)[..., None, :]  # bnh t s
    y_lower = np.einsum("bnhtmsu,bnhts,bnsuhp->bntmhp", cb, kern, vc)
    qk = np.einsum("bnlmhr,bnluhr->bnlhmu", cc, bc)
    y_diag = np.einsum("bnlhmu,bnluhp,bnlh->bnlmhp", qk, vc, gc)
    y = (y_off + y_lower + y_diag).reshape(bsz, S, m, H, P)[:, :s]
    return y.astype(v_bsmhp.dtype), final.astype(v_bsmhp.dtype)


def ssm_step3(h_bhpr, x_bhp, xprev_bhp, b_bmhr, bprev_bmhr, c_bmhr, alpha_bh, beta_bh, gamma_bh, mimo_x_hmp=None):
    """State update and readout of step_double_ssd (src/mamba3/double_ssd/double_ssd/mod.rs:672-748):
    h = alpha h + sum_m (gamma x*mx_m) (x) B_m + sum_m (beta x_prev*mx_m) (x) Bprev_m ; y_m = C_m . h.
    Returns (y_bmhp, h_new, x_vals_bmhp)."""
    m = b_bmhr.shape[1]
    if mimo_x_hmp is None:
        mx = np.ones((1, m) + x_bhp.shape[1:], x_bhp.dtype)
    else:
        mx = mimo_x_hmp.transpose(1, 0, 2)[None]
    xv = x_bhp[:, None] * mx
    xs = xprev_bhp[:, None] * mx
    h_new = (alpha_bh[:, :, None, None] * h_bhpr
             + mimo_outer_sum(xv * gamma_bh[:, None, :, None], b_bmhr)
             + mimo_outer_sum(xs * beta_bh[:, None, :, None], bprev_bmhr))
    y = np.einsum("bhpr,bmhr->bmhp", h_new, c_bmhr)
    return y.astype(h_bhpr.dtype), h_new.astype(h_bhpr.dtype), xv


def recurrence(x_bshp, b_bsmhr, c_bsmhr, alpha_bsh, beta_bsh, gamma_bsh, h0, xprev0_bhp, bprev0_bmhr,
               mimo_x_hmp=None, dtype=np.float64):
    """Ground truth for both SSD pathways: ssm_step3 unrolled in float64.  Returns (y_bsmhp, h_final)."""
    f = lambda t: None if t is None else t.astype(dtype)
    x, bm, cm = f(x_bshp), f(b_bsmhr), f(c_bsmhr)
    h, xp, bp = f(h0), f(xprev0_bhp), f(bprev0_bmhr)
    ys = []
    for t in range(x.shape[1]):
        y, h, _ = ssm_step3(h, x[:, t], xp, bm[:, t], bp, cm[:, t], f(alpha_bsh[:, t]), f(beta_bsh[:, t]),
                            f(gamma_bsh[:, t]), f(mimo_x_hmp))
        ys.append(y)
        xp, bp = x[:, t], bm[:, t]
    return np.stack(ys, axis=1), h


# ---------------------------------------------------------------------------------------------
# Block level
# ---------------------------------------------------------------------------------------------
class Mamba3Weights:
    """Random-init block weights (src/mamba3/mamba3.rs:640-790): in_proj split order
    [z | x | B(m g r) | C(m g r) | dd_dt(h) | dd_A(h) | lambda(h) | rot(a)] (single_ssd/mod.rs:89-104),
    B/C bias = 1 (:720), mimo_x = mimo_o = 1/m, mimo_z = 1 (:724-731), D = 1, QK-norm gamma = 1."""

    def __init__(self, rng, d_model, d_inner, nheads, state_rank, ngroups=1, mimo_rank=1, rope_fraction=1.0,
                 rotation_range=2.0, dtype=np.float32):
        self.d_model, self.d_inner, self.nheads = d_model, d_inner, nheads
        self.state_rank, self.ngroups, self.mimo_rank = state_rank, ngroups, mimo_rank
        self.per_head_dim = d_inner // nheads
        rope_dim = int(state_rank * rope_fraction)
        self.rope_dim = rope_dim - rope_dim % 2
        self.num_rope_angles = max(self.rope_dim // 2, 1)
        self.rotation_range = rotation_range
        bc = ngroups * state_rank * mimo_rank
        self.splits = np.cumsum([d_inner, d_inner, bc, bc, nheads, nheads, nheads])
        d_in_proj = int(self.splits[-1]) + self.num_rope_angles
        u = lambda shape, bound: rng.uniform(-bound, bound, size=shape).astype(dtype)
        self.w_in = u((d_model, d_in_proj), 1.0 / np.sqrt(d_model))
        dt = np.maximum(np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=nheads)), 1e-4)
        self.dt_bias = (dt + np.log(-np.expm1(-dt))).astype(dtype)
        self.d = np.ones(nheads, dtype)
        self.b_norm = np.ones(state_rank, dtype)
        self.c_norm = np.ones(state_rank, dtype)
        self.b_bias = np.ones((nheads, mimo_rank, state_rank), dtype)
        self.c_bias = np.ones((nheads, mimo_rank, state_rank), dtype)
        if mimo_rank > 1:
            self.mimo_x = np.full((nheads, mimo_rank, self.per_head_dim), 1.0 / mimo_rank, dtype)
            self.mimo_z = np.ones((nheads, mimo_rank, self.per_head_dim), dtype)
            self.mimo_o = np.full((nheads, mimo_rank, self.per_head_dim), 1.0 / mimo_rank, dtype)
        else:
            self.mimo_x = self.mimo_z = self.mimo_o = None
        self.w_out = u((d_inner, d_model), 1.0 / np.sqrt(d_inner))
        self.dt_limit = (0.0, 65504.0)
        self.a_floor = 1e-4


def zero_cache(w, bsz, dtype=np.float32):
    return dict(ssm=np.zeros((bsz, w.nheads, w.per_head_dim, w.state_rank), dtype),
                k=np.zeros((bsz, w.mimo_rank, w.nheads, w.state_rank), dtype),
                v=np.zeros((bsz, w.nheads, w.per_head_dim), dtype),
                angle=np.zeros((bsz, w.nheads, w.num_rope_angles), dtype))


def _project(w, u, dtype_name):
    proj = u @ w.w_in
    z, x, braw, craw, dd_dt, dd_a, lam_raw, rot = np.split(proj, w.splits.astype(int), axis=-1)
    co = trapezoidal_coefficients(dd_dt, dd_a, lam_raw, w.dt_bias, w.dt_limit, w.a_floor, dtype_name)
    lead = u.shape[:-1]
    braw = braw.reshape(lead + (w.mimo_rank, w.ngroups, w.state_rank))
    craw = craw.reshape(lead + (w.mimo_rank, w.ngroups, w.state_rank))
    bm = qk_norm_expand_bias(braw, w.b_norm, w.b_bias, w.nheads, dtype_name)
    cm = qk_norm_expand_bias(craw, w.c_norm, w.c_bias, w.nheads, dtype_name)
    x = x.reshape(lead + (w.nheads, w.per_head_dim))
    return z, x, bm, cm, co, rot


def _tail(w, y_mhp, xv_mhp, z, m_axis):
    """D skip on the raw v, gate, MIMO down-projection (src/mamba3/single_ssd/single_ssd/mod.rs:291-337,
    src/mamba3/double_ssd/double_ssd/mod.rs:544-614); out_norm is not modelled (default off)."""
    y = y_mhp + w.d[:, None] * xv_mhp
    lead = z.shape[:-1]
    zh = z.reshape(lead + (w.nheads, w.per_head_dim))
    if w.mimo_rank > 1:
        zm = np.expand_dims(zh, m_axis) * w.mimo_z.transpose(1, 0, 2)
        comb = y * silu(zm)
        out = (comb * w.mimo_o.transpose(1, 0, 2)).sum(axis=m_axis)
    else:
        out = np.squeeze(y, axis=m_axis) * silu(zh)
    return out.reshape(lead + (w.d_inner,)) @ w.w_out


def block_forward_single(w, u_bsm, cache, chunk_len, dtype_name="f32"):
    """Mamba3::forward_single_ssd (src/mamba3/single_ssd/single_ssd/mod.rs:44-353).
    Returns (out, new_cache, slot) with ``slot`` holding the tensors at the SSD slot."""
    z, x, bm, cm, co, rot = _project(w, u_bsm, dtype_name)
    dt, gamma, lam = co["dt"], co["gamma"], co["lam"]
    scale = single_ssd_scale(gamma, dt, lam)
    bm, cm, last_angle, cum_angles = rotate_bc_forward(rot, dt, cache["angle"], bm, cm, w.rope_dim, w.rotation_range)
    mx = None if w.mimo_x is None else w.mimo_x
    mxb = np.ones((1, w.mimo_rank, w.nheads, w.per_head_dim), x.dtype) if mx is None else mx.transpose(1, 0, 2)[None]
    seed = mimo_outer_sum(cache["v"][:, None] * mxb, cache["k"])
    h0 = cache["ssm"] + seed * (dt[:, 0] - gamma[:, 0])[:, :, None, None]
    v = x[:, :, None] * mxb[:, None]
    y, final = single_ssd_serial(v, co["da"], bm, cm, gamma, scale, h0, chunk_len)
    out = _tail(w, y, v, z, m_axis=2)
    new_cache = dict(ssm=final, k=bm[:, -1], v=x[:, -1], angle=last_angle)
    slot = dict(v=v, da=co["da"], b=bm, c=cm, gamma=gamma, scale=scale, h0=h0, y=y, final=final,
                angles=cum_angles, x=x, dt=dt, lam=lam, alpha=co["alpha"], beta=co["beta"])
    return out, new_cache, slot


def block_forward_double(w, u_bsm, cache, chunk_len, dtype_name="f32"):
    """Mamba3::forward_double_ssd (src/mamba3/double_ssd/double_ssd/mod.rs:40-369): gamma pass with the
    cached state + beta pass on the shifted x / B with a zero state, summed."""
    z, x, bm, cm, co, rot = _project(w, u_bsm, dtype_name)
    bm, cm, last_angle, _ = rotate_bc_forward(rot, co["dt"], cache["angle"], bm, cm, w.rope_dim, w.rotation_range)
    mxb = (np.ones((1, w.mimo_rank, w.nheads, w.per_head_dim), x.dtype) if w.mimo_x is None
           else w.mimo_x.transpose(1, 0, 2)[None])
    x_prev = np.concatenate([cache["v"][:, None], x[:, :-1]], axis=1)
    b_prev = np.concatenate([cache["k"][:, None], bm[:, :-1]], axis=1)
    v_g = (x * co["gamma"][..., None])[:, :, None] * mxb[:, None]
    v_b = (x_prev * co["beta"][..., None])[:, :, None] * mxb[:, None]
    y_g, f_g = double_ssd_serial(v_g, co["da"], bm, cm, cache["ssm"], chunk_len)
    y_b, f_b = double_ssd_serial(v_b, co["da"], b_prev, cm, np.zeros_like(cache["ssm"]), chunk_len)
    v_raw = x[:, :, None] * mxb[:, None]
    out = _tail(w, y_g + y_b, v_raw, z, m_axis=2)
    return out, dict(ssm=f_g + f_b, k=bm[:, -1], v=x[:, -1], angle=last_angle)


def block_step(w, u_bm, cache, dtype_name="f32"):
    """Mamba3::step_double_ssd (src/mamba3/double_ssd/double_ssd/mod.rs:635-760)."""
    z, x, bm, cm, co, rot = _project(w, u_bm, dtype_name)
    bm, cm, new_angle = rotate_bc_step(rot, co["dt"], cache["angle"], bm, cm, w.rope_dim, w.rotation_range)
    y, h_new, xv = ssm_step3(cache["ssm"], x, cache["v"], bm, cache["k"], cm, co["alpha"], co["beta"], co["gamma"],
                             w.mimo_x)
    out = _tail(w, y, xv, z, m_axis=1)
    return out, dict(ssm=h_new, k=bm, v=x, angle=new_angle)
