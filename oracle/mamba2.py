"""Mamba-2 oracle: chunked SSD (serial, minimal, sequential recurrence), block forward, step.

Test infrastructure (see oracle/__init__.py).  Shape letters follow the reference:
b batch, s sequence, h heads, p per-head dim, r state rank, g groups, n chunks, l chunk length,
v conv_dim, k conv kernel.  All functions take the *flat* sequence layout ``[b, s, ...]``;
the reference's ``[b, n, l, ...]`` is the same memory reshaped (src/mamba2/mamba2.rs:725-731).
"""
import numpy as np

from .numerics import softplus, silu, rms_norm_gated, inv_softplus


def gqa_expand(t_bsgr, nheads):
    """Group -> head broadcast: head h reads group h // (H/G) (src/modules/misc/gqa.rs:30-56)."""
    g = t_bsgr.shape[-2]
    return np.repeat(t_bsgr, nheads // g, axis=-2)


def _pad_to_chunks(x, dt, b, c, chunk_len):
    """Zero-pad the sequence to a multiple of chunk_len; dt = 0 makes a padded step the
    identity on the state (src/mamba2/mamba2.rs:703-722)."""
    s = x.shape[1]
    pad = (-s) % chunk_len
    if pad:
        z = lambda t: np.concatenate([t, np.zeros((t.shape[0], pad) + t.shape[2:], t.dtype)], axis=1)
        x, dt, b, c = z(x), z(dt), z(b), z(c)
    return x, dt, b, c, s


def ssd_serial(x_bshp, dt_bsh, a_h, b_bsgr, c_bsgr, d_h, h0_bhpr, chunk_len, return_chunk_states=False):
    """Serial (K1..K5) chunked SSD, following src/mamba2/ssd/serial.rs:34-506 step by step.

    K1 :138-164  cum = cumsum_l(dt*A_h), Aend = cum[..., -1]
    K2 :170-185  CB = C . B^T
    K3 :192-268  S_n = X^T . (B * dt * exp(Aend - cum))
    K4 :275-343  h_{n+1} = exp(Aend_n) h_n + S_n  (emits the state entering every chunk)
    K5 :349-506  Y = exp(cum) (C . h^T) + ((CB * exp(cum_t - cum_s) [s<=t] * dt_s) . X) + D X
    Returns (y_bshp, final_state_bhpr)."""
    dtype = x_bshp.dtype
    x, dt, bb, cc, s_orig = _pad_to_chunks(x_bshp, dt_bsh, b_bsgr, c_bsgr, chunk_len)
    bsz, S, H, P = x.shape
    R = bb.shape[-1]
    n, l = S // chunk_len, chunk_len
    bh = gqa_expand(bb, H).reshape(bsz, n, l, H, R)
    ch = gqa_expand(cc, H).reshape(bsz, n, l, H, R)
    xc = x.reshape(bsz, n, l, H, P)
    dtc = dt.reshape(bsz, n, l, H).transpose(0, 3, 1, 2)  # bhnl
    # K1
    cum = np.cumsum(dtc * a_h.astype(dtype)[None, :, None, None], axis=3)  # bhnl
    aend = cum[..., -1]  # bhn
    # K2
    cb = np.einsum("bnthr,bnshr->bnhts", ch, bh)  # bnhll
    # K3
    wts = np.exp(aend[..., None] - cum) * dtc  # bhnl
    bscaled = bh * wts.transpose(0, 2, 3, 1)[..., None]  # bnlhr
    s_intra = np.einsum("bnlhp,bnlhr->bnhpr", xc, bscaled)
    # K4
    run = h0_bhpr.astype(dtype).copy()
    entering = []
    for i in range(n):
        entering.append(run)
        run = np.exp(aend[:, :, i])[:, :, None, None] * run + s_intra[:, i]
    final = run
    h_in = np.stack(entering, axis=1)  # bnhpr
    # K5
    cum_bnhl = cum.transpose(0, 2, 1, 3)
    dt_bnhl = dtc.transpose(0, 2, 1, 3)
    blue = np.einsum("bnlhr,bnhpr->bnhlp", ch, h_in) * np.exp(cum_bnhl)[..., None]
    diff = cum_bnhl[..., :, None] - cum_bnhl[..., None, :]  # target - source
    upper = np.triu(np.ones((l, l), dtype=bool), k=1)
    diff = np.where(upper, -np.inf, diff)
    lhs = cb * np.exp(diff) * dt_bnhl[..., None, :]
    orange = np.einsum("bnhts,bnshp->bnhtp", lhs, xc)
    y = (blue + orange).transpose(0, 1, 3, 2, 4) + d_h.astype(dtype)[None, None, None, :, None] * xc
    y = y.reshape(bsz, S, H, P)[:, :s_orig].astype(dtype)
    if return_chunk_states:
        return y, final.astype(dtype), h_in.astype(dtype)
    return y, final.astype(dtype)


def segsum(x):
    """Lower-triangular segment sums with -inf above the diagonal (src/modules/misc/segsum.rs:35-47)."""
    cs = np.cumsum(x, axis=-1)
    diff = cs[..., :, None] - cs[..., None, :]
    l = x.shape[-1]
    return np.where(np.triu(np.ones((l, l), dtype=bool), k=1), -np.inf, diff)


def ssd_minimal(x_bshp, dt_bsh, a_h, b_bsgr, c_bsgr, d_h, h0_bhpr, chunk_len, init_state_hpr=None):
    """Minimal (segsum) SSD, following src/mamba2/ssd/minimal.rs:95-497: B_bar = dt*B folded first,
    L = exp(segsum(dt*A)), inter-chunk recurrence as a (1+n)x(1+n) decay matmul,
    optional learnable init_state_hpr added to the initial state (:317-328)."""
    dtype = x_bshp.dtype
    x, dt, bb, cc, s_orig = _pad_to_chunks(x_bshp, dt_bsh, b_bsgr, c_bsgr, chunk_len)
    bsz, S, H, P = x.shape
    R = bb.shape[-1]
    n, l = S // chunk_len, chunk_len
    bh = gqa_expand(bb, H).reshape(bsz, n, l, H, R)
    ch = gqa_expand(cc, H).reshape(bsz, n, l, H, R)
    xc = x.reshape(bsz, n, l, H, P)
    dtc = dt.reshape(bsz, n, l, H)
    delta_b = dtc[..., None] * bh
    a_bhnl = (dtc * a_h.astype(dtype)[None, None, None, :]).transpose(0, 3, 1, 2)
    cum = np.cumsum(a_bhnl, axis=3)
    cb = np.einsum("bnthr,bnshr->bnhts", ch, delta_b)
    L = np.exp(segsum(a_bhnl)).transpose(0, 2, 1, 3, 4)  # bnhll
    y_diag = np.einsum("bnhts,bnshp->bnthp", cb * L, xc)
    decay_state = np.exp(cum[..., -1:] - cum).transpose(0, 2, 3, 1)[..., None]  # bnlh1
    states = np.einsum("bnlhp,bnlhr->bnhpr", decay_state * xc, delta_b)
    init = h0_bhpr.astype(dtype)
    if init_state_hpr is not None:
        init = init + init_state_hpr[None]
    allst = np.concatenate([init[:, None], states], axis=1)  # bNhpr
    a_pad = np.concatenate([np.zeros((bsz, H, 1), dtype), cum[..., -1]], axis=2)
    decay_chunk = np.exp(segsum(a_pad))  # bhNN
    new_states = np.einsum("bhzn,bnhpr->bzhpr", decay_chunk, allst)
    h_in, final = new_states[:, :n], new_states[:, n]
    y_off = np.einsum("bnlhr,bnhpr->bnlhp", ch, h_in) * np.exp(cum).transpose(0, 2, 3, 1)[..., None]
    y = y_diag + y_off + d_h.astype(dtype)[None, None, None, :, None] * xc
    return y.reshape(bsz, S, H, P)[:, :s_orig].astype(dtype), final.astype(dtype)


def ssd_recurrence(x_bshp, dt_bsh, a_h, b_bsgr, c_bsgr, d_h, h0_bhpr, dtype=np.float64):
    """Ground truth: the step() recurrence unrolled token by token in float64
    (src/mamba2/mamba2.rs:935-991): h = exp(dt A) h + dt B (x) x ; y = C . h + D x."""
    x = x_bshp.astype(dtype)
    dt = dt_bsh.astype(dtype)
    bsz, S, H, P = x.shape
    bh = gqa_expand(b_bsgr.astype(dtype), H)
    ch = gqa_expand(c_bsgr.astype(dtype), H)
    a = a_h.astype(dtype)
    h = h0_bhpr.astype(dtype).copy()
    y = np.empty_like(x)
    for t in range(S):
        da = np.exp(dt[:, t] * a[None, :])  # bh
        h = h * da[:, :, None, None] + (dt[:, t][:, :, None] * x[:, t])[..., None] * bh[:, t][:, :, None, :]
        y[:, t] = np.einsum("bhpr,bhr->bhp", h, ch[:, t]) + d_h.astype(dtype)[None, :, None] * x[:, t]
    return y, h


def ssm_step(h_bhpr, x_bhp, dt_bh, a_h, b_bgr, c_bgr, d_h):
    """One-token state update + readout (src/mamba2/mamba2.rs:935-991).  Returns (y_bhp, h_new)."""
    H = x_bhp.shape[1]
    dtype = h_bhpr.dtype
    bh = gqa_expand(b_bgr, H).astype(dtype)
    ch = gqa_expand(c_bgr, H).astype(dtype)
    da = np.exp(dt_bh * a_h[None, :]).astype(dtype)
    dtbx = (dt_bh[:, :, None, None] * bh[:, :, None, :] * x_bhp[..., None]).astype(dtype)
    h_new = h_bhpr * da[:, :, None, None] + dtbx
    y = (h_new * ch[:, :, None, :]).sum(-1) + d_h[None, :, None] * x_bhp
    return y.astype(dtype), h_new


# ---------------------------------------------------------------------------------------------
# Block level (in_proj -> conv+SiLU -> split -> dt -> SSD -> gated norm -> out_proj)
# ---------------------------------------------------------------------------------------------
class Mamba2Weights:
    """Random-init block weights with the reference's distributions (src/mamba2/mamba2.rs:408-490):
    Linear U(+-1/sqrt(fan_in)), conv U(+-1/sqrt(k)) with bias, dt log-uniform [1e-3,1e-1] floored at
    1e-4 then inverse-softplus, A ~ U[1,16] -> log, D = 1, norm gamma = 1.  Burn's RNG stream is not
    reproducible outside Burn, so identical arrays are fed to both sides instead."""

    def __init__(self, rng, d_model, d_inner, nheads, state_rank, ngroups=1, conv_kernel=4, dtype=np.float32):
        self.d_model, self.d_inner, self.nheads = d_model, d_inner, nheads
        self.state_rank, self.ngroups, self.conv_kernel = state_rank, ngroups, conv_kernel
        self.per_head_dim = d_inner // nheads
        self.conv_dim = d_inner + 2 * ngroups * state_rank
        d_in_proj = d_inner + self.conv_dim + nheads
        u = lambda shape, bound: rng.uniform(-bound, bound, size=shape).astype(dtype)
        self.w_in = u((d_model, d_in_proj), 1.0 / np.sqrt(d_model))
        self.conv_w = u((self.conv_dim, conv_kernel), 1.0 / np.sqrt(conv_kernel))
        self.conv_b = u((self.conv_dim,), 1.0 / np.sqrt(conv_kernel))
        dt = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=nheads))
        self.dt_bias = inv_softplus(np.maximum(dt, 1e-4)).astype(dtype)
        self.a_log = np.log(rng.uniform(1.0, 16.0, size=nheads)).astype(dtype)
        self.d = np.ones(nheads, dtype)
        self.norm_gamma = np.ones(d_inner, dtype)
        self.w_out = u((d_inner, d_model), 1.0 / np.sqrt(d_inner))
        self.dt_limit = (0.0, 65504.0)


def block_pre_ssd(w, u_bsm, conv_bvk, dtype_name="f32"):
    """in_proj, causal depthwise conv + bias + SiLU, split, dt (src/mamba2/mamba2.rs:590-701).
    Returns (z, x_bshp, b_bsgr, c_bsgr, dt_bsh, a_h, new_conv_bvk)."""
    bsz, s, _ = u_bsm.shape
    k = w.conv_kernel
    proj = u_bsm @ w.w_in
    z, xbc, dt_raw = np.split(proj, [w.d_inner, w.d_inner + w.conv_dim], axis=2)
    padded = np.concatenate([conv_bvk[:, :, 1:], xbc.transpose(0, 2, 1)], axis=2)  # b v (k-1+s)
    new_conv = padded[:, :, s - 1:].copy()  # last k columns, raw pre-conv (:640)
    conv = np.zeros((bsz, w.conv_dim, s), u_bsm.dtype)
    for j in range(k):
        conv += padded[:, :, j:j + s] * w.conv_w[None, :, j:j + 1]
    conv = silu(conv + w.conv_b[None, :, None]).transpose(0, 2, 1)
    gr = w.ngroups * w.state_rank
    x, bm, cm = np.split(conv, [w.d_inner, w.d_inner + gr], axis=2)
    x = x.reshape(bsz, s, w.nheads, w.per_head_dim)
    bm = bm.reshape(bsz, s, w.ngroups, w.state_rank)
    cm = cm.reshape(bsz, s, w.ngroups, w.state_rank)
    dt = np.clip(softplus(dt_raw + w.dt_bias[None, None, :], dtype_name), *w.dt_limit).astype(u_bsm.dtype)
    a = -np.exp(w.a_log)
    return z, x, bm, cm, dt, a, new_conv


def block_forward(w, u_bsm, conv_bvk, ssm_bhpr, chunk_len, ssd=ssd_serial, dtype_name="f32"):
    """Mamba2::forward (src/mamba2/mamba2.rs:546-786).  Returns (out_bsm, new_conv_bvk, final_state,
    pre) where ``pre`` holds the tensors at the SSD slot for slot-level parity checks."""
    z, x, bm, cm, dt, a, new_conv = block_pre_ssd(w, u_bsm, conv_bvk, dtype_name)
    y, final = ssd(x, dt, a, bm, cm, w.d, ssm_bhpr, chunk_len)
    bsz, s = u_bsm.shape[:2]
    y_bsi = y.reshape(bsz, s, w.d_inner)
    g = rms_norm_gated(y_bsi, z, w.norm_gamma, norm_before_gate=False, dtype_name=dtype_name)
    out = g @ w.w_out
    pre = dict(z=z, x=x, b=bm, c=cm, dt=dt, a=a, y=y)
    return out, new_conv, final, pre


def block_step(w, u_bm, conv_bvk, ssm_bhpr, dtype_name="f32"):
    """Mamba2::step (src/mamba2/mamba2.rs:820-1004).  Returns (out_bm, new_conv_bvk, new_state)."""
    bsz = u_bm.shape[0]
    proj = u_bm @ w.w_in
    z, xbc, dt_raw = np.split(proj, [w.d_inner, w.d_inner + w.conv_dim], axis=1)
    new_conv = np.concatenate([conv_bvk[:, :, 1:], xbc[:, :, None]], axis=2)
    xbc = silu((new_conv * w.conv_w[None]).sum(-1) + w.conv_b[None])
    gr = w.ngroups * w.state_rank
    x, bm, cm = np.split(xbc, [w.d_inner, w.d_inner + gr], axis=1)
    x = x.reshape(bsz, w.nheads, w.per_head_dim)
    bm = bm.reshape(bsz, w.ngroups, w.state_rank)
    cm = cm.reshape(bsz, w.ngroups, w.state_rank)
    dt = np.clip(softplus(dt_raw + w.dt_bias[None], dtype_name), *w.dt_limit).astype(u_bm.dtype)
    a = -np.exp(w.a_log)
    y, h_new = ssm_step(ssm_bhpr, x, dt, a, bm, cm, w.d)
    g = rms_norm_gated(y.reshape(bsz, w.d_inner), z, w.norm_gamma, norm_before_gate=False, dtype_name=dtype_name)
    return g @ w.w_out, new_conv, h_new


def optimal_chunk_len(state_rank, per_head_dim):
    """ceil32(isqrt(N*P)) capped at 512 (src/mamba2/ssd/ssd_path.rs:109-114)."""
    root = int(np.floor(np.sqrt(state_rank * per_head_dim)))
    return min(((root + 31) // 32) * 32, 512)
