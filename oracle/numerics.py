"""Elementwise numerics shared by the oracle (test infrastructure, see oracle/__init__.py)."""
import numpy as np

# src/utils/mod.rs:50-95 -- div_eps(dtype); the reference notes the constants inline.
DIV_EPS = {"f64": 4.0693917e-16, "f32": 8.1584695e-8, "f16": 7.1209995e-4, "bf16": 2.0885676e-5}
# src/modules/activation/softplus.rs:17-48 -- identity above a dtype-specific threshold.
SOFTPLUS_THRESHOLD = {"f64": 38.0, "f32": 18.0, "bf16": 7.0, "f16": 9.0}


def softplus(x, dtype_name="f32"):
    """softplus with the reference's dtype threshold (src/modules/activation/softplus.rs:17-48):
    ``log1p(exp(min(x, thr)))`` below the threshold, ``x`` above it."""
    thr = SOFTPLUS_THRESHOLD[dtype_name]
    below = np.minimum(x, thr)
    return np.where(x > thr, x, np.log1p(np.exp(below))).astype(x.dtype)


def softplus_stock(x):
    """Burn's stock ``activation::softplus(x, beta=1)`` used by Mamba-1
    (src/mamba1/mamba1.rs:394,646): ``log(1 + exp(x))`` with no dtype threshold.
    Evaluated in the overflow-safe form max(x,0) + log1p(exp(-|x|)), equal in exact arithmetic."""
    return (np.maximum(x, 0) + np.log1p(np.exp(-np.abs(x)))).astype(x.dtype)


def inv_softplus(y):
    """dt_bias initialisation: y + ln(1 - exp(-y)) (src/mamba2/mamba2.rs:452)."""
    return y + np.log(-np.expm1(-y))


def silu(x):
    """x / (1 + exp(-x)) (src/modules/activation/silu.rs:24-27)."""
    return (x / (1.0 + np.exp(-x))).astype(x.dtype)


def sigmoid(x):
    return (1.0 / (1.0 + np.exp(-x))).astype(x.dtype)


def rms_norm(x, gamma, dtype_name="f32"):
    """x / sqrt(mean(x^2) + eps) * gamma over the last axis (src/modules/norm/rms_norm.rs:53-98)."""
    eps = x.dtype.type(DIV_EPS[dtype_name])
    rms = np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return (x / rms) * gamma


def rms_norm_gated(x, z, gamma, norm_before_gate=False, dtype_name="f32"):
    """Gated RMSNorm (src/modules/norm/rms_norm_gated.rs:70-135).
    ``norm_before_gate=False`` (the Mamba-2 block's setting): norm(x * silu(z)) * gamma;
    ``True``: norm(x) * gamma * silu(z)."""
    if not norm_before_gate:
        x = x * silu(z)
    out = rms_norm(x, gamma, dtype_name)
    if norm_before_gate:
        out = out * silu(z)
    return out


def bf16_round(x):
    """Round float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    out = rounded.view(np.float32).reshape(x.shape)
    return np.where(np.isfinite(x), out, x)


def to_bf16_bits(x):
    """float32 -> uint16 bfloat16 bit pattern (round to nearest even)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16).reshape(x.shape)


def from_bf16_bits(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(b.shape)


def rel_l2(a, b):
    """||a - b||_2 / ||b||_2 computed in float64 (the tolerance metric of the parity tests)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b.ravel())
    return float(np.linalg.norm((a - b).ravel()) / (den if den > 0 else 1.0))
