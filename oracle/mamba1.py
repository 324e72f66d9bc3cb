"""Mamba-1 oracle: sequential selective scan, single-token step, block forward/step.

Test infrastructure (see oracle/__init__.py).  b batch, s sequence, i d_inner, r state rank.
The reference feeds ``delta`` and ``c`` sequence-major (src/mamba1/mamba1.rs:396-400); that is an
internal artefact of its op loop -- here every tensor is batch-major ``[b, s, ...]``.
"""
import numpy as np

from .numerics import softplus_stock, silu


def selective_scan(delta_bsi, a_ir, b_bsr, c_bsr, d_i, u_bsi, h0_bir, dtype=None):
    """Mamba1::selective_scan (src/mamba1/mamba1.rs:422-523), token by token:
    h = h * exp(delta (x) A) + delta * B * u ; y_t = h . C_t ; y += D * u.
    Returns (y_bsi, h_final_bir)."""
    dtype = dtype or delta_bsi.dtype
    delta = delta_bsi.astype(dtype)
    u = u_bsi.astype(dtype)
    a = a_ir.astype(dtype)
    bsz, s, di = delta.shape
    h = h0_bir.astype(dtype).copy()
    y = np.empty((bsz, s, di), dtype)
    for t in range(s):
        d_a = np.exp(delta[:, t, :, None] * a[None])
        d_bu = delta[:, t, :, None] * b_bsr[:, t, None, :].astype(dtype) * u[:, t, :, None]
        h = h * d_a + d_bu
        y[:, t] = np.einsum("bir,br->bi", h, c_bsr[:, t].astype(dtype))
    y = y + d_i.astype(dtype)[None, None, :] * u
    return y, h


def selective_scan_step(delta_bi, a_ir, b_br, c_br, d_i, u_bi, h_bir):
    """Mamba1::selective_scan_step (src/mamba1/mamba1.rs:666-733).  Returns (y_bi, h_new)."""
    d_a = np.exp(delta_bi[:, :, None] * a_ir[None])
    d_bu = delta_bi[:, :, None] * b_br[:, None, :] * u_bi[:, :, None]
    h_new = h_bir * d_a + d_bu
    y = np.einsum("bir,br->bi", h_new, c_br) + d_i[None] * u_bi
    return y.astype(h_bir.dtype), h_new.astype(h_bir.dtype)


class Mamba1Weights:
    """Random-init block weights (src/mamba1/mamba1.rs:137-240): A[i, n] = n + 1 (S4D-real, :184-194),
    D = 1, Linear U(+-1/sqrt(fan_in)), dt bias = inverse softplus of log-uniform [1e-3, 1e-1]."""

    def __init__(self, rng, d_model, d_inner, state_rank=16, dt_rank=None, conv_kernel=4, dtype=np.float32):
        self.d_model, self.d_inner, self.state_rank = d_model, d_inner, state_rank
        self.dt_rank = dt_rank or -(-d_model // state_rank)  # d_model.div_ceil(state_rank), mamba1.rs:236-239
        self.conv_kernel = conv_kernel
        u = lambda shape, bound: rng.uniform(-bound, bound, size=shape).astype(dtype)
        self.w_in = u((d_model, 2 * d_inner), 1.0 / np.sqrt(d_model))
        self.conv_w = u((d_inner, conv_kernel), 1.0 / np.sqrt(conv_kernel))
        self.conv_b = u((d_inner,), 1.0 / np.sqrt(conv_kernel))
        self.w_x = u((d_inner, self.dt_rank + 2 * state_rank), 1.0 / np.sqrt(d_inner))
        self.w_dt = u((self.dt_rank, d_inner), self.dt_rank ** -0.5)
        dt = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), size=d_inner))
        dt = np.maximum(dt, 1e-4)
        self.b_dt = (dt + np.log(-np.expm1(-dt))).astype(dtype)
        self.a_log = np.log(np.tile(np.arange(1, state_rank + 1, dtype=np.float64), (d_inner, 1))).astype(dtype)
        self.d = np.ones(d_inner, dtype)
        self.w_out = u((d_inner, d_model), 1.0 / np.sqrt(d_inner))


def ssm_params(w, u):
    """x_proj / dt_proj / softplus part of Mamba1::ssm (src/mamba1/mamba1.rs:366-394)."""
    x_dbl = u @ w.w_x
    dr, bm, cm = np.split(x_dbl, [w.dt_rank, w.dt_rank + w.state_rank], axis=-1)
    delta = softplus_stock(dr @ w.w_dt + w.b_dt)
    return delta, -np.exp(w.a_log), bm, cm


def block_forward(w, x_bsm, conv_bik, ssm_bir):
    """Mamba1::forward (src/mamba1/mamba1.rs:278-352).  Returns (out, new_conv_bik, new_state, pre)."""
    bsz, s, _ = x_bsm.shape
    k = w.conv_kernel
    xs, res = np.split(x_bsm @ w.w_in, 2, axis=2)
    padded = np.concatenate([conv_bik[:, :, 1:], xs.transpose(0, 2, 1)], axis=2)
    new_conv = padded[:, :, s - 1:].copy()
    conv = np.zeros((bsz, w.d_inner, s), x_bsm.dtype)
    for j in range(k):
        conv += padded[:, :, j:j + s] * w.conv_w[None, :, j:j + 1]
    u = silu(conv + w.conv_b[None, :, None]).transpose(0, 2, 1)
    delta, a, bm, cm = ssm_params(w, u)
    y, h = selective_scan(delta, a, bm, cm, w.d, u, ssm_bir)
    out = (y * silu(res)) @ w.w_out
    return out, new_conv, h, dict(delta=delta, a=a, b=bm, c=cm, u=u, res=res, y=y)


def block_step(w, x_bm, conv_bik, ssm_bir):
    """Mamba1::step (src/mamba1/mamba1.rs:533-611)."""
    xs, res = np.split(x_bm @ w.w_in, 2, axis=1)
    new_conv = np.concatenate([conv_bik[:, :, 1:], xs[:, :, None]], axis=2)
    u = silu((new_conv * w.conv_w[None]).sum(-1) + w.conv_b[None])
    delta, a, bm, cm = ssm_params(w, u)
    y, h = selective_scan_step(delta, a, bm, cm, w.d, u, ssm_bir)
    return (y * silu(res)) @ w.w_out, new_conv, h
