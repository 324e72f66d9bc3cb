"""Tensor-level calls into libbm_b200 (torch supplies device memory and the CUDA stream only).

Every function validates dtypes/contiguity on the host, fills the C args struct with raw device
pointers and launches on torch's current stream.  Outputs are freshly allocated, like the tensors a
Burn backend returns from the reference's slot (src/mamba2/ssd/serial_recalculated/serial_recalculated.rs:86-98).
"""
import ctypes as C

import torch

from . import _ffi
from ._ffi import lib, check

_DT = {torch.float32: _ffi.BM_DTYPE_F32, torch.bfloat16: _ffi.BM_DTYPE_BF16}
PATHS = {"auto": _ffi.BM_PATH_AUTO, "exact": _ffi.BM_PATH_EXACT, "tensor": _ffi.BM_PATH_TENSOR,
         "tensor_single": _ffi.BM_PATH_TENSOR_SINGLE, "tensor_pair": _ffi.BM_PATH_TENSOR_PAIR}


def _ptr(t):
    return None if t is None else t.data_ptr()


def _chk(t, name, dtype=None, shape=None, optional=False):
    if t is None:
        if optional:
            return None
        raise ValueError(f"{name} is required")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")
    return t


def _stream():
    return torch.cuda.current_stream().cuda_stream


_ws_cache = {}


def _workspace(nbytes, device):
    """Grow-only per-device scratch buffer (the C ABI never allocates; the caller -- this wrapper -- does)."""
    key = (device.index, torch.cuda.current_stream().cuda_stream)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        _ws_cache[key] = buf
    return buf


def last_workspace_status():
    """Device status word left by the most recent SSD launch on the current device and stream (synchronises);
    0 when no launch has used a workspace yet."""
    key = (torch.cuda.current_device(), torch.cuda.current_stream().cuda_stream)
    ws = _ws_cache.get(key)
    return 0 if ws is None else int(lib.bm_workspace_status(ws.data_ptr(), _stream()))


def ssd2_fwd(x, dt, a, b, c, d=None, h0=None, chunk_len=256, path="auto", dt_bias=None, dt_limit=(0.0, 65504.0),
             z=None, return_chunk_states=False, check_status=False, debug_reserved=0):
    """Mamba-2 chunked SSD forward.  x [b,s,h,p], dt [b,s,h] f32, a [h] f32, b/c [b,s,g,r], d [h] f32,
    h0 [b,h,p,r] f32 -> (y [b,s,h,p], h_final [b,h,p,r] f32[, chunk_states [b,n,h,p,r]]).
    `debug_reserved` goes into the args struct's `reserved` field (0 in production)."""
    bsz, s, h, p = x.shape
    g, r = b.shape[2], b.shape[3]
    act = x.dtype
    if act not in _DT:
        raise ValueError(f"unsupported activation dtype {act}")
    _chk(x, "x"); _chk(dt, "dt", torch.float32, (bsz, s, h)); _chk(a, "a", torch.float32, (h,))
    _chk(b, "b", act, (bsz, s, g, r)); _chk(c, "c", act, (bsz, s, g, r))
    _chk(d, "d", torch.float32, (h,), optional=True); _chk(h0, "h0", torch.float32, (bsz, h, p, r), optional=True)
    _chk(dt_bias, "dt_bias", torch.float32, (h,), optional=True); _chk(z, "z", act, x.shape, optional=True)
    y = torch.empty_like(x)
    h_final = torch.empty((bsz, h, p, r), dtype=torch.float32, device=x.device)
    nchunks = -(-s // max(chunk_len, 1))
    states = torch.empty((bsz, nchunks, h, p, r), dtype=torch.float32, device=x.device) if return_chunk_states else None
    args = _ffi.Ssd2FwdArgs(batch=bsz, seqlen=s, nheads=h, headdim=p, state_rank=r, ngroups=g, chunk_len=chunk_len,
                            dtype=_DT[act], path=PATHS[path], reserved=debug_reserved, x=_ptr(x), dt=_ptr(dt),
                            a=_ptr(a), b=_ptr(b), c=_ptr(c), d=_ptr(d), h0=_ptr(h0), dt_bias=_ptr(dt_bias),
                            dt_min=dt_limit[0], dt_max=dt_limit[1], z=_ptr(z), y=_ptr(y), h_final=_ptr(h_final),
                            chunk_states=_ptr(states))
    nbytes = lib.bm_ssd2_fwd_workspace_bytes(C.byref(args))
    ws = _workspace(nbytes, x.device)
    check(lib.bm_ssd2_fwd(C.byref(args), ws.data_ptr(), ws.numel(), _stream()), "bm_ssd2_fwd")
    if check_status:  # synchronises: the tensor-core kernel's bounded waits report through the workspace
        check(lib.bm_workspace_status(ws.data_ptr(), _stream()), "bm_ssd2_fwd (device status)")
    return (y, h_final, states) if return_chunk_states else (y, h_final)


def step2(state, x, dt, a, b, c, d=None, dt_bias=None, dt_limit=(0.0, 65504.0), z=None):
    """Mamba-2 recurrent step; `state` [b,h,p,r] f32 is updated in place.  Returns y [b,h,p]."""
    bsz, h, p, r = state.shape
    g = b.shape[1]
    act = x.dtype
    _chk(state, "state", torch.float32); _chk(x, "x", act, (bsz, h, p)); _chk(dt, "dt", torch.float32, (bsz, h))
    _chk(a, "a", torch.float32, (h,)); _chk(b, "b", act, (bsz, g, r)); _chk(c, "c", act, (bsz, g, r))
    _chk(d, "d", torch.float32, (h,), optional=True); _chk(dt_bias, "dt_bias", torch.float32, (h,), optional=True)
    _chk(z, "z", act, (bsz, h, p), optional=True)
    y = torch.empty_like(x)
    args = _ffi.Step2Args(batch=bsz, nheads=h, headdim=p, state_rank=r, ngroups=g, dtype=_DT[act], state=_ptr(state),
                          x=_ptr(x), dt=_ptr(dt), a=_ptr(a), b=_ptr(b), c=_ptr(c), d=_ptr(d), dt_bias=_ptr(dt_bias),
                          dt_min=dt_limit[0], dt_max=dt_limit[1], z=_ptr(z), y=_ptr(y))
    check(lib.bm_step2(C.byref(args), _stream()), "bm_step2")
    return y


def conv_step(window, xin, weight, bias=None, splits=None):
    """Causal depthwise conv, one token: slides `window` [b,v,k] f32 in place, returns silu(conv) [b,v] -- or, with
    splits = (split_x, split_bc, split_bc), the three tensors (x [b,split_x], B, C [b,split_bc]).  `xin` [b,v] may be
    a column slice of a wider row."""
    bsz, v, k = window.shape
    _chk(window, "window", torch.float32)
    if not xin.is_cuda or tuple(xin.shape) != (bsz, v) or xin.stride(1) != 1:
        raise ValueError("xin must be a CUDA tensor [b, v] with a contiguous last axis")
    _chk(weight, "weight", torch.float32, (v, k)); _chk(bias, "bias", torch.float32, (v,), optional=True)
    act = xin.dtype
    if splits is None:
        outs, sx, sbc = (torch.empty((bsz, v), dtype=act, device=xin.device), None, None), 0, 0
    else:
        sx, sbc, sbc2 = splits
        if sbc != sbc2 or sx + 2 * sbc != v:
            raise ValueError("splits must be (split_x, split_bc, split_bc) summing to the channel count")
        outs = tuple(torch.empty((bsz, n), dtype=act, device=xin.device) for n in (sx, sbc, sbc))
    args = _ffi.ConvStepArgs(batch=bsz, channels=v, kernel=k, dtype=_DT[act], window=_ptr(window), xin=xin.data_ptr(),
                             weight=_ptr(weight), bias=_ptr(bias), out=_ptr(outs[0]), out_b=_ptr(outs[1]),
                             out_c=_ptr(outs[2]), xin_stride=xin.stride(0), split_x=sx, split_bc=sbc, reserved=0)
    check(lib.bm_conv_step(C.byref(args), _stream()), "bm_conv_step")
    return outs[0] if splits is None else outs


DIV_EPS = {torch.float32: 8.1584695e-8, torch.bfloat16: 2.0885676e-5}   # src/utils/mod.rs:50-95


_keepalive = []   # dense copies made by _rows stay referenced until the next call has been enqueued


def _rows(t, name):
    """(data_ptr, row stride) of a 2-D+ tensor whose last axis is contiguous and whose leading axes collapse
    into rows of one stride (a dense tensor, or a column slice of one)."""
    if t.stride(-1) != 1:
        raise ValueError(f"{name}: last axis must be contiguous")
    stride = t.stride(-2) if t.dim() >= 2 else t.shape[-1]
    if (stride * t.element_size()) % 16 or t.data_ptr() % 16:
        t = t.contiguous()     # rows of a slice that do not start 16-byte aligned: fall back to a dense copy
        stride = t.shape[-1]
        _keepalive.append(t)
    for d in range(t.dim() - 2):
        if t.stride(d) != t.stride(d + 1) * t.shape[d + 1]:
            raise ValueError(f"{name}: leading axes must collapse into rows of one stride")
    return t.data_ptr(), stride


def conv1d_silu_fwd(xbc, weight, bias=None, window=None, splits=None, want_window=True):
    """Prefill causal depthwise conv + bias + SiLU.  xbc [b, s, v] (may be a column slice), weight [v, k] f32,
    window [b, v, k] f32 or None -> (out [b,s,v] or (x, B, C) when splits = (split_x, split_bc, split_bc), new_window)."""
    bsz, s, v = xbc.shape
    k = weight.shape[1]
    act = xbc.dtype
    if not xbc.is_cuda:
        raise ValueError("xbc must be a CUDA tensor (this library has no CPU path)")
    del _keepalive[:]
    ptr, stride = _rows(xbc, "xbc")
    _chk(weight, "weight", torch.float32, (v, k)); _chk(bias, "bias", torch.float32, (v,), optional=True)
    _chk(window, "window", torch.float32, (bsz, v, k), optional=True)
    new_window = torch.empty((bsz, v, k), dtype=torch.float32, device=xbc.device) if want_window else None
    if splits is None:
        outs = (torch.empty((bsz, s, v), dtype=act, device=xbc.device), None, None)
        sx = sbc = 0
    else:
        sx, sbc, sbc2 = splits
        if sbc != sbc2 or sx + 2 * sbc != v:
            raise ValueError("splits must be (split_x, split_bc, split_bc) summing to the channel count")
        outs = tuple(torch.empty((bsz, s, n), dtype=act, device=xbc.device) for n in (sx, sbc, sbc))
    args = _ffi.Conv1dSiluArgs(batch=bsz, seqlen=s, channels=v, kernel=k, dtype=_DT[act], xin_stride=stride, split_x=sx,
                               split_bc=sbc, xin=ptr, weight=_ptr(weight), bias=_ptr(bias), window=_ptr(window),
                               new_window=_ptr(new_window), out_x=_ptr(outs[0]), out_b=_ptr(outs[1]), out_c=_ptr(outs[2]))
    check(lib.bm_conv1d_silu_fwd(C.byref(args), _stream()), "bm_conv1d_silu_fwd")
    return (outs[0] if splits is None else outs), new_window


def rmsnorm_gated(x, z, gamma, norm_before_gate=False, eps=None):
    """RmsNormGated over the last axis (z = None: plain RmsNorm).  x / z [..., d] (may be column slices), gamma [d]."""
    d = x.shape[-1]
    act = x.dtype
    if not x.is_cuda:
        raise ValueError("x must be a CUDA tensor (this library has no CPU path)")
    del _keepalive[:]
    xp, xs = _rows(x, "x")
    zp, zs = (None, 0) if z is None else _rows(z, "z")
    _chk(gamma, "gamma", act, (d,))
    out = torch.empty(tuple(x.shape), dtype=act, device=x.device)
    rows = out.numel() // d
    args = _ffi.RmsnormGatedArgs(rows=rows, width=d, dtype=_DT[act], norm_before_gate=int(norm_before_gate), x_stride=xs,
                                 z_stride=zs, eps=DIV_EPS[act] if eps is None else eps, x=xp, z=zp, gamma=_ptr(gamma),
                                 out=_ptr(out))
    check(lib.bm_rmsnorm_gated(C.byref(args), _stream()), "bm_rmsnorm_gated")
    return out


def mamba3_bc_prep(b_raw, c_raw, b_gamma, c_gamma, b_bias, c_bias, angles=None, rope_dim=None, pairwise=None, ngroups=1,
                   eps=None):
    """Mamba-3 B / C from the raw projection columns to what the SSD slot takes: RMS norm over r, group -> head
    expansion, + bias[h, m, r], rotation by the cumulative angles.  b_raw / c_raw [b, s, m * g * r] (may be column
    slices of the projection output), gammas [r] f32, biases [h, m, r] f32, angles [b, s, h, rope_dim / 2] f32 or
    None -> (B, C) [b, s, m, h, r] in the activations' dtype."""
    bsz, s, mgr = b_raw.shape
    h, m, r = b_bias.shape
    act = b_raw.dtype
    if not b_raw.is_cuda:
        raise ValueError("b_raw must be a CUDA tensor (this library has no CPU path)")
    if mgr != m * ngroups * r or tuple(c_raw.shape) != (bsz, s, mgr):
        raise ValueError("raw rows must hold m * g * r entries")
    rope_dim = r if rope_dim is None else rope_dim
    pairwise = (m == 1) if pairwise is None else pairwise
    del _keepalive[:]
    bp, bs = _rows(b_raw, "b_raw")
    cp, cs = _rows(c_raw, "c_raw")
    if bs != cs:
        raise ValueError("b_raw and c_raw must have the same row stride")
    for t, name in ((b_gamma, "b_gamma"), (c_gamma, "c_gamma")):
        _chk(t, name, torch.float32, (r,))
    _chk(b_bias, "b_bias", torch.float32, (h, m, r)); _chk(c_bias, "c_bias", torch.float32, (h, m, r))
    _chk(angles, "angles", torch.float32, (bsz, s, h, max(rope_dim // 2, 0)), optional=True)
    outs = [torch.empty((bsz, s, m, h, r), dtype=act, device=b_raw.device) for _ in range(2)]
    args = _ffi.Mamba3BcPrepArgs(batch=bsz, seqlen=s, mimo_rank=m, ngroups=ngroups, nheads=h, state_rank=r, dtype=_DT[act],
                                 raw_stride=bs, rope_dim=rope_dim, pairwise=int(pairwise),
                                 eps=DIV_EPS[act] if eps is None else eps, b_raw=bp, c_raw=cp, b_gamma=_ptr(b_gamma),
                                 c_gamma=_ptr(c_gamma), b_bias=_ptr(b_bias), c_bias=_ptr(c_bias), angles=_ptr(angles),
                                 b_out=_ptr(outs[0]), c_out=_ptr(outs[1]))
    check(lib.bm_mamba3_bc_prep(C.byref(args), _stream()), "bm_mamba3_bc_prep")
    return outs[0], outs[1]


def selscan1_fwd(u, delta, a, b, c, d=None, z=None, h0=None, delta_bias=None, delta_softplus=False, serial=False):
    """Mamba-1 selective scan.  u/delta/z [b,s,i], a [i,r] f32, b/c [b,s,r] -> (y [b,s,i], h_final [b,i,r] f32).
    The sequence-parallel kernels (bm_selscan1_fwd_ws) are used unless `serial` asks for the kernels that walk
    the sequence in order and need no workspace (bm_selscan1_fwd)."""
    bsz, s, di = u.shape
    r = a.shape[1]
    act = u.dtype
    _chk(u, "u"); _chk(delta, "delta", act, (bsz, s, di)); _chk(a, "a", torch.float32, (di, r))
    _chk(b, "b", act, (bsz, s, r)); _chk(c, "c", act, (bsz, s, r)); _chk(d, "d", torch.float32, (di,), optional=True)
    _chk(z, "z", act, (bsz, s, di), optional=True); _chk(h0, "h0", torch.float32, (bsz, di, r), optional=True)
    _chk(delta_bias, "delta_bias", torch.float32, (di,), optional=True)
    y = torch.empty_like(u)
    h_final = torch.empty((bsz, di, r), dtype=torch.float32, device=u.device)
    args = _ffi.Selscan1Args(batch=bsz, seqlen=s, d_inner=di, state_rank=r, dtype=_DT[act],
                             delta_softplus=int(delta_softplus), u=_ptr(u), delta=_ptr(delta), a=_ptr(a), b=_ptr(b),
                             c=_ptr(c), d=_ptr(d), delta_bias=_ptr(delta_bias), z=_ptr(z), h0=_ptr(h0), y=_ptr(y),
                             h_final=_ptr(h_final))
    if serial:
        check(lib.bm_selscan1_fwd(C.byref(args), _stream()), "bm_selscan1_fwd")
    else:
        ws = _workspace(lib.bm_selscan1_fwd_workspace_bytes(C.byref(args)), u.device)
        check(lib.bm_selscan1_fwd_ws(C.byref(args), ws.data_ptr(), ws.numel(), _stream()), "bm_selscan1_fwd_ws")
    return y, h_final


def step1(state, u, delta, a, b, c, d=None, z=None, delta_bias=None, delta_softplus=False):
    """Mamba-1 recurrent step; `state` [b,i,r] f32 updated in place.  Returns y [b,i]."""
    bsz, di, r = state.shape
    act = u.dtype
    _chk(state, "state", torch.float32); _chk(u, "u", act, (bsz, di)); _chk(delta, "delta", act, (bsz, di))
    _chk(a, "a", torch.float32, (di, r)); _chk(b, "b", act, (bsz, r)); _chk(c, "c", act, (bsz, r))
    _chk(d, "d", torch.float32, (di,), optional=True); _chk(z, "z", act, (bsz, di), optional=True)
    _chk(delta_bias, "delta_bias", torch.float32, (di,), optional=True)
    y = torch.empty_like(u)
    args = _ffi.Step1Args(batch=bsz, d_inner=di, state_rank=r, dtype=_DT[act], delta_softplus=int(delta_softplus),
                          state=_ptr(state), u=_ptr(u), delta=_ptr(delta), a=_ptr(a), b=_ptr(b), c=_ptr(c), d=_ptr(d),
                          delta_bias=_ptr(delta_bias), z=_ptr(z), y=_ptr(y))
    check(lib.bm_step1(C.byref(args), _stream()), "bm_step1")
    return y


SSD3_TENSOR_PATH = True   # bm_ssd3_*_fwd have a tensor-core path (bf16, P 64, N 128, MIMO rank 1 / 2 / 4)


def _ssd3(fn_name, v, da, b, c, gamma, scale, h0, chunk_len, angles, rope_dim, path, check_status=False):
    bsz, s, m, h, p = v.shape
    r = b.shape[-1]
    act = v.dtype
    _chk(v, "v"); _chk(da, "da", torch.float32, (bsz, s, h)); _chk(b, "b", act, (bsz, s, m, h, r))
    _chk(c, "c", act, (bsz, s, m, h, r)); _chk(gamma, "gamma", torch.float32, (bsz, s, h), optional=True)
    _chk(scale, "scale", torch.float32, (bsz, s, h), optional=True)
    _chk(h0, "h0", torch.float32, (bsz, h, p, r), optional=True)
    if angles is not None:
        _chk(angles, "angles", torch.float32, (bsz, s, h, max(rope_dim // 2, 1)))
    y = torch.empty_like(v)
    h_final = torch.empty((bsz, h, p, r), dtype=torch.float32, device=v.device)
    args = _ffi.Ssd3FwdArgs(batch=bsz, seqlen=s, nheads=h, headdim=p, state_rank=r, mimo_rank=m, chunk_len=chunk_len,
                            dtype=_DT[act], path=PATHS[path], rope_dim=rope_dim, v=_ptr(v), da=_ptr(da), b=_ptr(b),
                            c=_ptr(c), gamma=_ptr(gamma), scale=_ptr(scale), h0=_ptr(h0), angles=_ptr(angles),
                            y=_ptr(y), h_final=_ptr(h_final))
    nbytes = lib.bm_ssd3_fwd_workspace_bytes(C.byref(args))
    ws = _workspace(nbytes, v.device)
    check(getattr(lib, fn_name)(C.byref(args), ws.data_ptr(), ws.numel(), _stream()), fn_name)
    if check_status:
        check(lib.bm_workspace_status(ws.data_ptr(), _stream()), fn_name + " (device status)")
    return y, h_final


def ssd3_single_fwd(v, da, b, c, gamma, scale, h0=None, chunk_len=64, angles=None, rope_dim=0, path="auto", check_status=False):
    """Mamba-3 single-pass SSD.  v [b,s,m,h,p], da/gamma/scale [b,s,h] f32, b/c [b,s,m,h,r]."""
    return _ssd3("bm_ssd3_single_fwd", v, da, b, c, gamma, scale, h0, chunk_len, angles, rope_dim, path, check_status)


def ssd3_double_fwd(v, da, b, c, h0=None, chunk_len=64, angles=None, rope_dim=0, path="auto", check_status=False):
    """Generic MIMO SSD on pre-scaled v (one pass of Mamba-3's double-SSD pathway)."""
    return _ssd3("bm_ssd3_double_fwd", v, da, b, c, None, None, h0, chunk_len, angles, rope_dim, path, check_status)


def angle_cumsum(rot, dt, prev=None, rng=2.0):
    """theta [b,s,h,a] = prev + cumsum_s(dt * range * pi * tanh(rot)); also returns wrap(theta[:, -1])."""
    bsz, s, na = rot.shape
    h = dt.shape[2]
    _chk(rot, "rot", torch.float32); _chk(dt, "dt", torch.float32, (bsz, s, h))
    _chk(prev, "prev", torch.float32, (bsz, h, na), optional=True)
    theta = torch.empty((bsz, s, h, na), dtype=torch.float32, device=rot.device)
    last = torch.empty((bsz, h, na), dtype=torch.float32, device=rot.device)
    args = _ffi.AngleCumsumArgs(batch=bsz, seqlen=s, nheads=h, nangles=na, range=rng, rot=_ptr(rot), dt=_ptr(dt),
                                prev=_ptr(prev), theta=_ptr(theta), last=_ptr(last))
    check(lib.bm_angle_cumsum(C.byref(args), _stream()), "bm_angle_cumsum")
    return theta, last


def step3(state, k_state, v_state, angle, x, b, c, rot, dt, alpha, beta, gamma, mimo_x=None, rope_dim=None, rng=2.0):
    """Mamba-3 recurrent step; state / k_state / v_state / angle are updated in place.  Returns y [b,m,h,p]."""
    bsz, h, p, r = state.shape
    m = b.shape[1]
    if rope_dim is None:
        rope_dim = r
    na = max(rope_dim // 2, 1)
    f = torch.float32
    _chk(state, "state", f); _chk(k_state, "k_state", f, (bsz, m, h, r)); _chk(v_state, "v_state", f, (bsz, h, p))
    _chk(angle, "angle", f, (bsz, h, na)); _chk(x, "x", f, (bsz, h, p)); _chk(b, "b", f, (bsz, m, h, r))
    _chk(c, "c", f, (bsz, m, h, r)); _chk(rot, "rot", f, (bsz, na))
    for n_, t_ in (("dt", dt), ("alpha", alpha), ("beta", beta), ("gamma", gamma)):
        _chk(t_, n_, f, (bsz, h))
    _chk(mimo_x, "mimo_x", f, (h, m, p), optional=True)
    y = torch.empty((bsz, m, h, p), dtype=f, device=state.device)
    args = _ffi.Step3Args(batch=bsz, nheads=h, headdim=p, state_rank=r, mimo_rank=m, rope_dim=rope_dim, range=rng,
                          state=_ptr(state), k_state=_ptr(k_state), v_state=_ptr(v_state), angle=_ptr(angle),
                          x=_ptr(x), b=_ptr(b), c=_ptr(c), rot=_ptr(rot), dt=_ptr(dt), alpha=_ptr(alpha),
                          beta=_ptr(beta), gamma=_ptr(gamma), mimo_x=_ptr(mimo_x), y=_ptr(y))
    check(lib.bm_step3(C.byref(args), _stream()), "bm_step3")
    return y


def ssd2_fwd_noalloc(x, dt, a, b, c, d=None, h0=None, chunk_len=256, dt_bias=None, dt_limit=(0.0, 65504.0), z=None):
    """bm_ssd2_fwd_noalloc: the exact Mamba-2 SSD forward with the library's built-in scratch instead of
    a workspace -- this wrapper still allocates the outputs, the library call itself allocates nothing.
    Raises BmError(BM_ERR_WORKSPACE_TOO_SMALL) when the problem needs more scratch than the built-in
    array holds.  Calls share that array: do not overlap them on different streams."""
    bsz, s, h, p = x.shape
    g, r = b.shape[2], b.shape[3]
    act = x.dtype
    if act not in _DT:
        raise ValueError(f"unsupported activation dtype {act}")
    _chk(x, "x"); _chk(dt, "dt", torch.float32, (bsz, s, h)); _chk(a, "a", torch.float32, (h,))
    _chk(b, "b", act, (bsz, s, g, r)); _chk(c, "c", act, (bsz, s, g, r))
    _chk(d, "d", torch.float32, (h,), optional=True); _chk(h0, "h0", torch.float32, (bsz, h, p, r), optional=True)
    _chk(dt_bias, "dt_bias", torch.float32, (h,), optional=True); _chk(z, "z", act, x.shape, optional=True)
    y = torch.empty_like(x)
    h_final = torch.empty((bsz, h, p, r), dtype=torch.float32, device=x.device)
    args = _ffi.Ssd2FwdArgs(batch=bsz, seqlen=s, nheads=h, headdim=p, state_rank=r, ngroups=g, chunk_len=chunk_len,
                            dtype=_DT[act], path=_ffi.BM_PATH_EXACT, reserved=0, x=_ptr(x), dt=_ptr(dt), a=_ptr(a),
                            b=_ptr(b), c=_ptr(c), d=_ptr(d), h0=_ptr(h0), dt_bias=_ptr(dt_bias),
                            dt_min=dt_limit[0], dt_max=dt_limit[1], z=_ptr(z), y=_ptr(y), h_final=_ptr(h_final),
                            chunk_states=None)
    check(lib.bm_ssd2_fwd_noalloc(C.byref(args), _stream()), "bm_ssd2_fwd_noalloc")
    return y, h_final


def ssd2_bwd(x, dt, a, b, c, d, h0, dy, dh_final=None, chunk_len=256, path="auto", check_status=False):
    """Mamba-2 SSD backward (recompute).  Returns dict(dx, ddt, da, db, dc, dd, dh0), all float32;
    db / dc are per group.  path: "auto" (tensor-core kernel for bf16, headdim 64, state_rank 128), "exact", "tensor"."""
    bsz, s, h, p = x.shape
    g, r = b.shape[2], b.shape[3]
    act = x.dtype
    _chk(x, "x"); _chk(dt, "dt", torch.float32, (bsz, s, h)); _chk(a, "a", torch.float32, (h,))
    _chk(b, "b", act, (bsz, s, g, r)); _chk(c, "c", act, (bsz, s, g, r)); _chk(dy, "dy", act, x.shape)
    _chk(d, "d", torch.float32, (h,), optional=True); _chk(h0, "h0", torch.float32, (bsz, h, p, r), optional=True)
    _chk(dh_final, "dh_final", torch.float32, (bsz, h, p, r), optional=True)
    f = dict(dtype=torch.float32, device=x.device)
    out = dict(dx=torch.empty((bsz, s, h, p), **f), ddt=torch.empty((bsz, s, h), **f), da=torch.empty((h,), **f),
               db=torch.empty((bsz, s, g, r), **f), dc=torch.empty((bsz, s, g, r), **f),
               dd=None if d is None else torch.empty((h,), **f), dh0=torch.empty((bsz, h, p, r), **f))
    args = _ffi.Ssd2BwdArgs(batch=bsz, seqlen=s, nheads=h, headdim=p, state_rank=r, ngroups=g, chunk_len=chunk_len,
                            dtype=_DT[act], x=_ptr(x), dt=_ptr(dt), a=_ptr(a), b=_ptr(b), c=_ptr(c), d=_ptr(d),
                            h0=_ptr(h0), dy=_ptr(dy), dh_final=_ptr(dh_final), dx=_ptr(out["dx"]), ddt=_ptr(out["ddt"]),
                            da=_ptr(out["da"]), db=_ptr(out["db"]), dc=_ptr(out["dc"]), dd=_ptr(out["dd"]),
                            dh0=_ptr(out["dh0"]), path=PATHS[path])
    ws = _workspace(lib.bm_ssd2_bwd_workspace_bytes(C.byref(args)), x.device)
    check(lib.bm_ssd2_bwd(C.byref(args), ws.data_ptr(), ws.numel(), _stream()), "bm_ssd2_bwd")
    if check_status:
        check(lib.bm_workspace_status(ws.data_ptr(), _stream()), "bm_workspace_status")
    return out


def ssd3_bwd(v, da, b, c, gamma, scale, h0, dy, dh_final=None, chunk_len=64, single=True, path="auto", check_status=False):
    """Mamba-3 SSD backward.  single: returns also dgamma / dscale.  All gradients float32.
    path: "auto" (tensor-core kernel for bf16, headdim 64, state_rank 128, MIMO rank 1 / 2 / 4), "exact", "tensor"."""
    bsz, s, m, h, p = v.shape
    r = b.shape[-1]
    act = v.dtype
    _chk(v, "v"); _chk(da, "da", torch.float32, (bsz, s, h)); _chk(b, "b", act, (bsz, s, m, h, r))
    _chk(c, "c", act, (bsz, s, m, h, r)); _chk(dy, "dy", act, v.shape)
    _chk(h0, "h0", torch.float32, (bsz, h, p, r), optional=True)
    _chk(dh_final, "dh_final", torch.float32, (bsz, h, p, r), optional=True)
    f = dict(dtype=torch.float32, device=v.device)
    out = dict(dv=torch.empty((bsz, s, m, h, p), **f), dda=torch.empty((bsz, s, h), **f),
               db=torch.empty((bsz, s, m, h, r), **f), dc=torch.empty((bsz, s, m, h, r), **f),
               dh0=torch.empty((bsz, h, p, r), **f))
    if single:
        _chk(gamma, "gamma", torch.float32, (bsz, s, h)); _chk(scale, "scale", torch.float32, (bsz, s, h))
        out.update(dgamma=torch.empty((bsz, s, h), **f), dscale=torch.empty((bsz, s, h), **f))
    args = _ffi.Ssd3BwdArgs(batch=bsz, seqlen=s, nheads=h, headdim=p, state_rank=r, mimo_rank=m, chunk_len=chunk_len,
                            dtype=_DT[act], v=_ptr(v), da=_ptr(da), b=_ptr(b), c=_ptr(c),
                            gamma=_ptr(gamma) if single else None, scale=_ptr(scale) if single else None, h0=_ptr(h0),
                            dy=_ptr(dy), dh_final=_ptr(dh_final), dv=_ptr(out["dv"]), dda=_ptr(out["dda"]),
                            db=_ptr(out["db"]), dc=_ptr(out["dc"]), dgamma=_ptr(out.get("dgamma")),
                            dscale=_ptr(out.get("dscale")), dh0=_ptr(out["dh0"]), path=PATHS[path])
    ws = _workspace(lib.bm_ssd3_bwd_workspace_bytes(C.byref(args)), v.device)
    fn = lib.bm_ssd3_single_bwd if single else lib.bm_ssd3_double_bwd
    check(fn(C.byref(args), ws.data_ptr(), ws.numel(), _stream()), "bm_ssd3_bwd")
    if check_status:
        check(lib.bm_workspace_status(ws.data_ptr(), _stream()), "bm_workspace_status")
    return out
