"""Gradient oracle for the chunked SSD cores (test infrastructure, see oracle/__init__.py).

The reference obtains gradients two ways and tests them against each other
(src/mamba2/ssd/ssd_path/tests.rs:184-336, src/mamba3/single_ssd/ssd/ssd_path/tests.rs:175-339):
autodiff through the Minimal/Serial forward, and the hand-written recompute backward
(src/mamba2/ssd/serial_recalculated/combined_backward.rs:126-590,
src/mamba3/single_ssd/ssd/serial_recalculated/combined_backward.rs:74-536).  This module plays the
autodiff side: the serial forward restated in torch (float64) and differentiated by torch.autograd,
plus a central finite-difference check that does not depend on any autodiff.
"""
import numpy as np
import torch


def _pad(t, pad):
    if pad == 0:
        return t
    return torch.cat([t, torch.zeros((t.shape[0], pad) + tuple(t.shape[2:]), dtype=t.dtype)], dim=1)


def mimo_ssd_forward_torch(v, da, bm, cm, cs, gsame, h0, chunk_len, strict, d=None):
    """General chunked SSD in torch, the common form of the three reference cores:
        y_i = exp(cum_t) C_i h_n + sum_j (C_i . B_j) kern(i, j) v_j (+ D v_i)
        kern = exp(cum_ti - cum_tj) cs_tj for t_j < t_i;  gsame_t for t_j == t_i;  0 otherwise
        S_n = sum_j exp(Aend - cum_tj) cs_tj v_j (x) B_j ;  h_{n+1} = exp(Aend) h_n + S_n
    v [b,s,m,h,p]; bm, cm [b,s,m,h,r]; da, cs, gsame [b,s,h]; h0 [b,h,p,r]; d [h] or None.
    Mamba-2: m = 1, da = dt*A, cs = gsame = dt (src/mamba2/ssd/serial.rs:138-506).
    Mamba-3 single: cs = scale, gsame = gamma, strict mask (src/mamba3/single_ssd/ssd/serial.rs:56-268).
    Mamba-3 double: cs = gsame = 1 (src/mamba3/double_ssd/ssd/serial.rs:56-409).
    `strict` only documents which reference mask is meant; the same-time weight is always gsame."""
    bsz, s, m, H, P = v.shape
    R = bm.shape[-1]
    pad = (-s) % chunk_len
    v, da, bm, cm, cs, gsame = (_pad(t, pad) for t in (v, da, bm, cm, cs, gsame))
    S = s + pad
    n, l = S // chunk_len, chunk_len
    vc = v.reshape(bsz, n, l, m, H, P)
    bc = bm.reshape(bsz, n, l, m, H, R)
    cc = cm.reshape(bsz, n, l, m, H, R)
    cum = torch.cumsum(da.reshape(bsz, n, l, H), dim=2)            # b n l h
    csn = cs.reshape(bsz, n, l, H)
    gsn = gsame.reshape(bsz, n, l, H)
    aend = cum[:, :, -1]                                           # b n h
    w = torch.exp(aend[:, :, None] - cum) * csn                    # b n l h
    s_intra = torch.einsum("bnlmhp,bnlmhr,bnlh->bnhpr", vc, bc, w)
    run = h0
    entering = []
    for i in range(n):
        entering.append(run)
        run = torch.exp(aend[:, i])[:, :, None, None] * run + s_intra[:, i]
    h_in = torch.stack(entering, dim=1)                            # b n h p r
    y_off = torch.einsum("bnlmhr,bnhpr->bnlmhp", cc, h_in) * torch.exp(cum)[:, :, :, None, :, None]
    cb = torch.einsum("bntmhr,bnsuhr->bnhtmsu", cc, bc)
    cum_h = cum.permute(0, 1, 3, 2)                                # b n h l
    diff = cum_h[..., :, None] - cum_h[..., None, :]               # b n h t s
    lower = torch.tril(torch.ones(l, l, dtype=torch.bool), diagonal=-1)
    eye = torch.eye(l, dtype=torch.bool)
    kern = torch.where(lower, torch.exp(torch.where(lower, diff, torch.zeros_like(diff))), torch.zeros_like(diff))
    kern = kern * csn.permute(0, 1, 3, 2)[..., None, :]
    kern = kern + torch.where(eye, gsn.permute(0, 1, 3, 2)[..., :, None].expand_as(diff), torch.zeros_like(diff))
    y_in = torch.einsum("bnhtmsu,bnhts,bnsuhp->bntmhp", cb, kern, vc)
    y = y_off + y_in
    if d is not None:
        y = y + d[None, None, None, None, :, None] * vc
    return y.reshape(bsz, S, m, H, P)[:, :s], run


def ssd2_forward_torch(x, dt, a, b, c, d, h0, chunk_len):
    """Mamba-2 SSD through the general form.  x [b,s,h,p]; b, c [b,s,g,r] (expanded to heads here)."""
    H = x.shape[2]
    rep = H // b.shape[2]
    bh = b.repeat_interleave(rep, dim=2)[:, :, None]
    ch = c.repeat_interleave(rep, dim=2)[:, :, None]
    y, hf = mimo_ssd_forward_torch(x[:, :, None], dt * a[None, None, :], bh, ch, dt, dt, h0, chunk_len, False, d)
    return y[:, :, 0], hf


def ssd2_grads(x, dt, a, b, c, d, h0, dy, dhf, chunk_len):
    """Autodiff gradients of (y, h_final) contracted with (dy, dhf).  numpy in / numpy out (float64).
    Returns dict(dx, ddt, da, db, dc, dd, dh0); db/dc are per group (the head sum the reference leaves
    to the autodiff of its GQA expand, src/modules/misc/gqa.rs:30-56)."""
    t = {k: torch.tensor(np.asarray(v, np.float64), requires_grad=True)
         for k, v in dict(x=x, dt=dt, a=a, b=b, c=c, d=d, h0=h0).items()}
    y, hf = ssd2_forward_torch(t["x"], t["dt"], t["a"], t["b"], t["c"], t["d"], t["h0"], chunk_len)
    loss = (y * torch.tensor(np.asarray(dy, np.float64))).sum() + (hf * torch.tensor(np.asarray(dhf, np.float64))).sum()
    loss.backward()
    return dict(dx=t["x"].grad.numpy(), ddt=t["dt"].grad.numpy(), da=t["a"].grad.numpy(), db=t["b"].grad.numpy(),
                dc=t["c"].grad.numpy(), dd=t["d"].grad.numpy(), dh0=t["h0"].grad.numpy())


def ssd3_grads(v, da, bm, cm, gamma, scale, h0, dy, dhf, chunk_len, single=True):
    """Autodiff gradients of the Mamba-3 cores.  single: d_gamma and d_scale are returned too
    (src/mamba3/single_ssd/ssd/serial_recalculated/combined_backward.rs:34-49)."""
    names = dict(v=v, da=da, b=bm, c=cm, h0=h0)
    if single:
        names.update(gamma=gamma, scale=scale)
    t = {k: torch.tensor(np.asarray(val, np.float64), requires_grad=True) for k, val in names.items()}
    ones = torch.ones_like(t["da"])
    cs = t["scale"] if single else ones
    gs = t["gamma"] if single else ones
    y, hf = mimo_ssd_forward_torch(t["v"], t["da"], t["b"], t["c"], cs, gs, t["h0"], chunk_len, single)
    loss = (y * torch.tensor(np.asarray(dy, np.float64))).sum() + (hf * torch.tensor(np.asarray(dhf, np.float64))).sum()
    loss.backward()
    out = dict(dv=t["v"].grad.numpy(), dda=t["da"].grad.numpy(), db=t["b"].grad.numpy(), dc=t["c"].grad.numpy(),
               dh0=t["h0"].grad.numpy())
    if single:
        out.update(dgamma=t["gamma"].grad.numpy(), dscale=t["scale"].grad.numpy())
    return out


def finite_difference(fn, arrays, name, index, eps=1e-6):
    """Central difference of the scalar fn(**arrays) with respect to arrays[name][index]."""
    hi = {k: v.copy() for k, v in arrays.items()}
    lo = {k: v.copy() for k, v in arrays.items()}
    hi[name][index] += eps
    lo[name][index] -= eps
    return (fn(**hi) - fn(**lo)) / (2 * eps)


def rope_halves_torch(x, angles):
    """Half-and-half rotation (pairs (j, j + r/2)) of the last axis of x by `angles` (last axis r/2), as the
    reference applies it when the MIMO rank is above one (src/mamba3/rotation/mod.rs:665,
    src/modules/misc/rope.rs:112-170 with the full width rotated)."""
    half = x.shape[-1] // 2
    cos, sin = torch.cos(angles), torch.sin(angles)
    x0, x1 = x[..., :half], x[..., half:]
    return torch.cat([cos * x0 - sin * x1, sin * x0 + cos * x1], dim=-1)


def ssd3_single_chain_grads(x, b_raw, c_raw, dt, a, lam, theta, h0, dy, dhf, chunk_len, mimo_rank):
    """The Mamba-3 forward + backward configuration as one differentiable chain (float64 autodiff):
    v_m = x / m;  da = dt A_h;  gamma = lambda dt;  scale_t = gamma_t + (1 - lambda_{t+1}) dt_{t+1} (last: gamma)
    (src/mamba3/single_ssd/single_ssd/mod.rs:111-149, src/mamba3/helpers.rs:42-73); B, C rotated by the given
    angles theta [b,s,h,r/2]; then the single-SSD core.  lambda and theta are inputs, not differentiated.
    Returns y, h_final and dx, dB, dC (w.r.t. the un-rotated tensors), ddt, dA."""
    f64 = lambda v, g=True: torch.tensor(np.asarray(v, np.float64), requires_grad=g)
    t = dict(x=f64(x), b=f64(b_raw), c=f64(c_raw), dt=f64(dt), a=f64(a))
    lam_t, th = f64(lam, False), f64(theta, False)
    v = (t["x"] / mimo_rank)[:, :, None].expand(-1, -1, mimo_rank, -1, -1)
    da = t["dt"] * t["a"][None, None]
    gamma = lam_t * t["dt"]
    nxt = torch.cat([((1.0 - lam_t) * t["dt"])[:, 1:], torch.zeros_like(gamma[:, :1])], dim=1)
    scale = gamma + nxt
    b_rot = rope_halves_torch(t["b"], th[:, :, None])
    c_rot = rope_halves_torch(t["c"], th[:, :, None])
    y, hf = mimo_ssd_forward_torch(v, da, b_rot, c_rot, scale, gamma, f64(h0, False), chunk_len, True)
    loss = (y * f64(dy, False)).sum() + (hf * f64(dhf, False)).sum()
    loss.backward()
    return dict(y=y.detach().numpy(), h_final=hf.detach().numpy(), dx=t["x"].grad.numpy(), dB=t["b"].grad.numpy(),
                dC=t["c"].grad.numpy(), ddt=t["dt"].grad.numpy(), dA=t["a"].grad.numpy())
