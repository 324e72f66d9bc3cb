"""Seeded synthetic inputs for the benchmark configurations (test infrastructure, see oracle/__init__.py).

The reference uses no dataset on this path; the configurations are defined by shapes and value
distributions only, reproduced here with numpy's PCG64.  Every generator takes shape overrides so the
same distributions can be drawn at sizes the oracle finishes in seconds.
"""
import numpy as np

from .numerics import softplus, inv_softplus


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def log_uniform(rng, lo, hi, size):
    return np.exp(rng.uniform(np.log(lo), np.log(hi), size=size))


def ssd2_prefill(seed=2, batch=8, seqlen=4096, nheads=80, headdim=64, state_rank=128, ngroups=1, h0_std=0.0):
    """Configuration "Mamba-2 SSD prefill at the 2.7B layer shape": x ~ N(0,1); dt = softplus(N(0,1) + dt_bias)
    with dt_bias = inverse-softplus of log-uniform [1e-3, 1e-1]; A = -U[1,16] per head; B, C ~ N(0,1)/sqrt(N);
    D ~ U[0,1]; zero initial state unless h0_std > 0.  All float32 (cast by the caller)."""
    rng = _rng(seed)
    f = np.float32
    x = rng.standard_normal((batch, seqlen, nheads, headdim), dtype=f)
    dt_bias = inv_softplus(log_uniform(rng, 1e-3, 1e-1, nheads)).astype(f)
    dt = softplus(rng.standard_normal((batch, seqlen, nheads), dtype=f) + dt_bias, "f32").astype(f)
    a = (-rng.uniform(1.0, 16.0, nheads)).astype(f)
    b = (rng.standard_normal((batch, seqlen, ngroups, state_rank), dtype=f) / np.sqrt(state_rank)).astype(f)
    c = (rng.standard_normal((batch, seqlen, ngroups, state_rank), dtype=f) / np.sqrt(state_rank)).astype(f)
    d = rng.uniform(0.0, 1.0, nheads).astype(f)
    h0 = (h0_std * rng.standard_normal((batch, nheads, headdim, state_rank), dtype=f)).astype(f)
    return dict(x=x, dt=dt, a=a, b=b, c=c, d=d, h0=h0, dt_bias=dt_bias)


def selscan1(seed=1, batch=4, seqlen=2048, d_inner=1536, state_rank=16):
    """Configuration "Mamba-1 selective scan": delta log-uniform [1e-3, 1e-1]; A[i, n] = -(n+1);
    B, C, u, z ~ N(0,1); D = 1; zero initial state."""
    rng = _rng(seed)
    f = np.float32
    u = rng.standard_normal((batch, seqlen, d_inner), dtype=f)
    delta = log_uniform(rng, 1e-3, 1e-1, (batch, seqlen, d_inner)).astype(f)
    a = -np.tile(np.arange(1, state_rank + 1, dtype=f), (d_inner, 1))
    b = rng.standard_normal((batch, seqlen, state_rank), dtype=f)
    c = rng.standard_normal((batch, seqlen, state_rank), dtype=f)
    d = np.ones(d_inner, f)
    z = rng.standard_normal((batch, seqlen, d_inner), dtype=f)
    h0 = np.zeros((batch, d_inner, state_rank), f)
    return dict(u=u, delta=delta, a=a, b=b, c=c, d=d, z=z, h0=h0)


def step2_decode(seed=3, batch=256, nheads=80, headdim=64, state_rank=128, ngroups=1, steps=4):
    """Per-layer tensors of configuration "Mamba-2 recurrent step() decode": fp32 state ~ N(0, 0.1) and
    `steps` tokens of post-conv x, B, C, dt drawn as in ssd2_prefill."""
    rng = _rng(seed)
    f = np.float32
    state = (0.1 * rng.standard_normal((batch, nheads, headdim, state_rank), dtype=f)).astype(f)
    x = rng.standard_normal((steps, batch, nheads, headdim), dtype=f)
    dt_bias = inv_softplus(log_uniform(rng, 1e-3, 1e-1, nheads)).astype(f)
    dt = softplus(rng.standard_normal((steps, batch, nheads), dtype=f) + dt_bias, "f32").astype(f)
    a = (-rng.uniform(1.0, 16.0, nheads)).astype(f)
    b = (rng.standard_normal((steps, batch, ngroups, state_rank), dtype=f) / np.sqrt(state_rank)).astype(f)
    c = (rng.standard_normal((steps, batch, ngroups, state_rank), dtype=f) / np.sqrt(state_rank)).astype(f)
    d = rng.uniform(0.0, 1.0, nheads).astype(f)
    return dict(state=state, x=x, dt=dt, a=a, b=b, c=c, d=d)


def ssd3_single(seed=4, batch=16, seqlen=2048, nheads=32, headdim=64, state_rank=128, mimo_rank=4, h0_std=0.0):
    """Configuration "Mamba-3 SSD forward": x ~ N(0,1) with v = x * mimo_x (mimo_x = 1/m); B, C ~ N(0,1)/sqrt(N)
    per (m, head) (un-rotated); angles theta = cumsum(dt * omega), omega ~ N(0,1); lambda = sigmoid(N(0,1));
    dt and A as in ssd2_prefill -> da = dt A_h, gamma = lambda dt, scale_t = gamma_t + (1 - lambda_{t+1}) dt_{t+1}."""
    rng = _rng(seed)
    f = np.float32
    x = rng.standard_normal((batch, seqlen, nheads, headdim), dtype=f)
    v = np.repeat(x[:, :, None] / mimo_rank, mimo_rank, axis=2).astype(f)
    b = (rng.standard_normal((batch, seqlen, mimo_rank, nheads, state_rank), dtype=f) / np.sqrt(state_rank)).astype(f)
    c = (rng.standard_normal((batch, seqlen, mimo_rank, nheads, state_rank), dtype=f) / np.sqrt(state_rank)).astype(f)
    dt_bias = inv_softplus(log_uniform(rng, 1e-3, 1e-1, nheads)).astype(f)
    dt = softplus(rng.standard_normal((batch, seqlen, nheads), dtype=f) + dt_bias, "f32").astype(f)
    a = (-rng.uniform(1.0, 16.0, nheads)).astype(f)
    omega = rng.standard_normal((batch, seqlen, nheads, state_rank // 2), dtype=f)
    angles = np.cumsum(dt[..., None] * omega, axis=1, dtype=np.float64).astype(f)
    lam = (1.0 / (1.0 + np.exp(-rng.standard_normal((batch, seqlen, nheads), dtype=f)))).astype(f)
    da = (dt * a).astype(f)
    gamma = (lam * dt).astype(f)
    scale = gamma.copy()
    scale[:, :-1] += dt[:, 1:] * (1.0 - lam[:, 1:])
    h0 = (h0_std * rng.standard_normal((batch, nheads, headdim, state_rank), dtype=f)).astype(f)
    return dict(v=v, b=b, c=c, da=da, gamma=gamma, scale=scale.astype(f), angles=angles, h0=h0, dt=dt, lam=lam, a=a,
                rope_dim=state_rank)
