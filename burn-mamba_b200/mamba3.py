"""Host-side mirror of the reference's Mamba-3 block around the SSD slot and the recurrent step.

`Mamba3.forward_single_ssd` (src/mamba3/single_ssd/single_ssd/mod.rs:44-353), `forward_double_ssd`
(src/mamba3/double_ssd/double_ssd/mod.rs:40-369) and `step_double_ssd` (:635-760) with the reference's
parameter set (src/mamba3/mamba3.rs:640-790) and cache layout (ssm [b,h,p,r], k [b,m,h,r] rotated B of the
last token, v [b,h,p] last x, angle [b,h,a] wrapped).  The SSM core runs in libbm_b200: the angle scan
(`bm_angle_cumsum`), the chunked SSD with the rotation of B / C fused into its loads (`bm_ssd3_*_fwd`)
and the step (`bm_step3`).  Projection, trapezoid coefficients, QK-norm, gate and MIMO down-projection
are plain library ops (torch), as they sit outside the hot path in the reference too; `out_norm` is not
modelled (default off).
"""
import math

import torch

from . import ops

DIV_EPS = 8.1584695e-8   # float32 entry of src/utils/mod.rs:50-95


def _silu(t):
    return t / (1.0 + torch.exp(-t))


def _softplus(t):
    return torch.where(t > 18.0, t, torch.log1p(torch.exp(torch.clamp(t, max=18.0))))


def wrap_angle(t):
    """theta - round(theta / 2pi) * 2pi (src/modules/misc/rope.rs:23-27)."""
    two_pi = 2.0 * math.pi
    return t - torch.round(t * (1.0 / two_pi)) * two_pi


def apply_rope_partial(x, angles, rope_dim, pairwise):
    """Rotate the leading rope_dim entries of the last axis (src/modules/misc/rope.rs:50-170); pairs
    (2j, 2j+1) when pairwise, halves (j, j + r/2) otherwise."""
    if rope_dim == 0:
        return x
    na = rope_dim // 2
    ang = wrap_angle(angles[..., :na])
    cos, sin = torch.cos(ang), torch.sin(ang)
    out = x.clone()
    if pairwise:
        x0, x1 = x[..., 0:rope_dim:2], x[..., 1:rope_dim:2]
        out[..., 0:rope_dim:2] = cos * x0 - sin * x1
        out[..., 1:rope_dim:2] = sin * x0 + cos * x1
    else:
        half = x.shape[-1] // 2
        x0, x1 = x[..., :na], x[..., half:half + na]
        out[..., :na] = cos * x0 - sin * x1
        out[..., half:half + na] = sin * x0 + cos * x1
    return out


class Mamba3:
    """One Mamba-3 block.  Weights are float32 tensors on the GPU:
    w_in [d_model, 2 d_inner + 2 m g r + 3 h + a] with the reference's split order
    [z | x | B(m g r) | C(m g r) | dd_dt(h) | dd_A(h) | lambda(h) | rot(a)], dt_bias [h], d [h],
    b_norm / c_norm [r], b_bias / c_bias [h, m, r], mimo_x / mimo_z / mimo_o [h, m, p] (or None when
    m = 1), w_out [d_inner, d_model]."""

    def __init__(self, w_in, dt_bias, d, b_norm, c_norm, b_bias, c_bias, w_out, nheads, state_rank, ngroups=1,
                 mimo_rank=1, rope_dim=None, rotation_range=2.0, mimo_x=None, mimo_z=None, mimo_o=None,
                 dt_limit=(0.0, 65504.0), a_floor=1e-4):
        self.w_in, self.w_out, self.dt_bias, self.d = w_in, w_out, dt_bias, d
        self.b_norm, self.c_norm, self.b_bias, self.c_bias = b_norm, c_norm, b_bias, c_bias
        self.mimo_x, self.mimo_z, self.mimo_o = mimo_x, mimo_z, mimo_o
        self.nheads, self.state_rank, self.ngroups, self.mimo_rank = nheads, state_rank, ngroups, mimo_rank
        self.d_inner = w_out.shape[0]
        self.per_head_dim = self.d_inner // nheads
        self.rope_dim = state_rank if rope_dim is None else rope_dim
        self.num_rope_angles = max(self.rope_dim // 2, 1)
        self.rotation_range, self.dt_limit, self.a_floor = rotation_range, dt_limit, a_floor
        bc = ngroups * state_rank * mimo_rank
        self.splits = [self.d_inner, self.d_inner, bc, bc, nheads, nheads, nheads, self.num_rope_angles]
        assert w_in.shape[1] == sum(self.splits)

    @classmethod
    def from_oracle_weights(cls, w, device):
        """Builds the block from the oracle's random-init weight bundle (tests)."""
        t = lambda a: None if a is None else torch.tensor(a, dtype=torch.float32, device=device)
        return cls(t(w.w_in), t(w.dt_bias), t(w.d), t(w.b_norm), t(w.c_norm), t(w.b_bias), t(w.c_bias), t(w.w_out),
                   w.nheads, w.state_rank, w.ngroups, w.mimo_rank, w.rope_dim, w.rotation_range, t(w.mimo_x),
                   t(w.mimo_z), t(w.mimo_o), w.dt_limit, w.a_floor)

    def zero_cache(self, batch):
        dev, f = self.w_in.device, torch.float32
        return dict(ssm=torch.zeros((batch, self.nheads, self.per_head_dim, self.state_rank), device=dev, dtype=f),
                    k=torch.zeros((batch, self.mimo_rank, self.nheads, self.state_rank), device=dev, dtype=f),
                    v=torch.zeros((batch, self.nheads, self.per_head_dim), device=dev, dtype=f),
                    angle=torch.zeros((batch, self.nheads, self.num_rope_angles), device=dev, dtype=f))

    # -- the glue in front of the core --------------------------------------------------------------
    def _qk(self, raw, gamma_r, bias_hmr):
        """RMSNorm over r, group -> head expansion, + bias[h, m, r] (src/mamba3/helpers.rs:82-95)."""
        normed = raw / torch.sqrt((raw * raw).mean(-1, keepdim=True) + DIV_EPS) * gamma_r
        expanded = normed.repeat_interleave(self.nheads // self.ngroups, dim=-2)
        return expanded + bias_hmr.transpose(0, 1)

    def _project(self, u, qk=True):
        """In-projection and its splits.  qk = True: B / C normed, expanded and biased by torch ops (the step
        pathway, whose kernel rotates them itself); qk = False: the raw B / C columns, for `_bc_prep`."""
        proj = u @ self.w_in
        z, x, braw, craw, dd_dt, dd_a, lam_raw, rot = torch.split(proj, self.splits, dim=-1)
        # trapezoid coefficients (src/mamba3/helpers.rs:42-73)
        dt = torch.clamp(_softplus(dd_dt + self.dt_bias), *self.dt_limit)
        a = -torch.clamp(_softplus(dd_a), min=self.a_floor)
        da = dt * a
        lam = torch.sigmoid(lam_raw)
        alpha = torch.exp(da)
        co = dict(dt=dt, da=da, lam=lam, alpha=alpha, beta=(1.0 - lam) * dt * alpha, gamma=lam * dt)
        lead = u.shape[:-1]
        shape = lead + (self.mimo_rank, self.ngroups, self.state_rank)
        if qk:
            bm = self._qk(braw.reshape(shape), self.b_norm, self.b_bias)
            cm = self._qk(craw.reshape(shape), self.c_norm, self.c_bias)
        else:
            bm, cm = braw, craw
        return z, x.reshape(lead + (self.nheads, self.per_head_dim)), bm, cm, co, rot

    def _bc_prep(self, braw, craw, theta):
        """Raw B / C columns of the projection -> normed, expanded, biased and rotated [b, s, m, h, r] in one
        kernel (helpers.rs:82-95 + rotation/mod.rs:653-679)."""
        f = lambda t: t.float().contiguous()
        return ops.mamba3_bc_prep(braw, craw, f(self.b_norm), f(self.c_norm), f(self.b_bias), f(self.c_bias),
                                  angles=theta if self.rope_dim > 0 else None,
                                  rope_dim=self.rope_dim, pairwise=self.mimo_rank == 1, ngroups=self.ngroups)

    def _mx(self):
        """mimo_x as a broadcastable [1, m, h, p] (ones when m = 1)."""
        if self.mimo_x is None:
            return torch.ones((1, self.mimo_rank, self.nheads, self.per_head_dim), device=self.w_in.device)
        return self.mimo_x.transpose(0, 1).unsqueeze(0)

    def _tail(self, y_mhp, xv_mhp, z, m_axis):
        """D skip on the raw v, gate, MIMO down-projection (single_ssd/mod.rs:291-337, double_ssd/mod.rs:544-614)."""
        y = y_mhp + self.d[:, None] * xv_mhp
        lead = z.shape[:-1]
        zh = z.reshape(lead + (self.nheads, self.per_head_dim))
        if self.mimo_rank > 1:
            zm = zh.unsqueeze(m_axis) * self.mimo_z.transpose(0, 1)
            out = (y * _silu(zm) * self.mimo_o.transpose(0, 1)).sum(dim=m_axis)
        else:
            out = y.squeeze(m_axis) * _silu(zh)
        return out.reshape(lead + (self.d_inner,)) @ self.w_out

    def _angles(self, rot, dt, cache):
        """Cumulative rotation angles of the sequence and the wrapped angle after its last token."""
        return ops.angle_cumsum(rot.contiguous(), dt.contiguous(), cache["angle"].contiguous(), rng=self.rotation_range)

    # -- forward, single-SSD pathway -------------------------------------------------------------------
    def forward_single_ssd(self, u_bsm, cache=None, chunk_len=64):
        """-> (out [b,s,d_model], cache).  One SSD pass with the trapezoid folded into gamma / scale; B / C go
        from the projection's raw columns to the rotated per-head tensors in one kernel."""
        bsz = u_bsm.shape[0]
        cache = cache or self.zero_cache(bsz)
        z, x, braw, craw, co, rot = self._project(u_bsm, qk=False)
        dt, gamma, lam = co["dt"], co["gamma"], co["lam"]
        scale = gamma.clone()
        scale[:, :-1] += dt[:, 1:] * (1.0 - lam[:, 1:])             # single_ssd/mod.rs:134-149
        theta, last_angle = self._angles(rot, dt, cache)
        bm, cm = self._bc_prep(braw, craw, theta)
        mxb = self._mx()
        seed = torch.einsum("bmhp,bmhr->bhpr", cache["v"][:, None] * mxb, cache["k"])
        h0 = cache["ssm"] + seed * (dt[:, 0] - gamma[:, 0])[:, :, None, None]
        v = (x[:, :, None] * mxb[:, None]).contiguous()
        y, final = ops.ssd3_single_fwd(v, co["da"].contiguous(), bm, cm, gamma.contiguous(), scale.contiguous(),
                                       h0.contiguous(), chunk_len=chunk_len)
        out = self._tail(y, v, z, m_axis=2)
        return out, dict(ssm=final, k=bm[:, -1].contiguous(), v=x[:, -1].contiguous(), angle=last_angle)

    # -- forward, double-SSD pathway -------------------------------------------------------------------
    def forward_double_ssd(self, u_bsm, cache=None, chunk_len=64):
        """-> (out, cache).  Gamma pass from the cached state plus beta pass on the shifted x / B from a
        zero state.  The beta pass pairs B of token t-1 (rotated by its own angle) with C of token t, so
        both passes take the rotated tensors, which this pathway materialises once."""
        bsz = u_bsm.shape[0]
        cache = cache or self.zero_cache(bsz)
        z, x, braw, craw, co, rot = self._project(u_bsm, qk=False)
        theta, last_angle = self._angles(rot, co["dt"], cache)
        bm, cm = self._bc_prep(braw, craw, theta)
        mxb = self._mx()
        x_prev = torch.cat([cache["v"][:, None], x[:, :-1]], dim=1)
        b_prev = torch.cat([cache["k"][:, None], bm[:, :-1]], dim=1).contiguous()
        v_g = ((x * co["gamma"][..., None])[:, :, None] * mxb[:, None]).contiguous()
        v_b = ((x_prev * co["beta"][..., None])[:, :, None] * mxb[:, None]).contiguous()
        da = co["da"].contiguous()
        y_g, f_g = ops.ssd3_double_fwd(v_g, da, bm, cm, cache["ssm"].contiguous(), chunk_len=chunk_len)
        y_b, f_b = ops.ssd3_double_fwd(v_b, da, b_prev, cm, None, chunk_len=chunk_len)
        v_raw = x[:, :, None] * mxb[:, None]
        out = self._tail(y_g + y_b, v_raw, z, m_axis=2)
        return out, dict(ssm=f_g + f_b, k=bm[:, -1].contiguous(), v=x[:, -1].contiguous(), angle=last_angle)

    # -- step ---------------------------------------------------------------------------------------------
    def step_double_ssd(self, u_bm, cache=None):
        """-> (out [b,d_model], cache).  The cache tensors are updated in place by `bm_step3` (angle update,
        rotation of B / C, trapezoid state update, readout, cache roll) and returned."""
        bsz = u_bm.shape[0]
        cache = cache or self.zero_cache(bsz)
        z, x, bm, cm, co, rot = self._project(u_bm)
        x = x.contiguous()
        y = ops.step3(cache["ssm"], cache["k"], cache["v"], cache["angle"], x, bm.contiguous(), cm.contiguous(),
                      rot.contiguous(), co["dt"].contiguous(), co["alpha"].contiguous(), co["beta"].contiguous(),
                      co["gamma"].contiguous(), self.mimo_x, rope_dim=self.rope_dim, rng=self.rotation_range)
        xv = x[:, None] * self._mx()
        return self._tail(y, xv, z, m_axis=1), cache
