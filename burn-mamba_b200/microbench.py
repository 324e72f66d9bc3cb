"""Device-time microbenchmarks of the bandwidth-bound kernels at the benchmark shapes:
Mamba-2 decode step (batch 256, 2.7B head shape), Mamba-1 selective scan (b4 L2048 i1536 N16),
Mamba-3 step, conv step, angle scan.  Prints one JSON line per kernel with the achieved GB/s on the
kernel's algorithmic bytes and the fraction of the measured HBM peak.

    python burn-mamba_b200/microbench.py [--iters 20]
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()  # evict L2 between timed launches (buffer larger than the 126 MB L2)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def main():
    import __graft_entry__ as ge
    bm = ge.load_package()
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    peak, src = _peak()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(3)
    rn = lambda *s, dt=torch.float32: torch.randn(*s, generator=g, device=dev).to(dt)
    out = []

    # Mamba-2 decode step, one layer of the 64-layer stack: state R+W dominates
    B, H, P, R = 256, 80, 64, 128
    state = 0.1 * rn(B, H, P, R)
    x, dt, a = rn(B, H, P, dt=torch.bfloat16), torch.rand(B, H, device=dev) * 0.1, -torch.rand(H, device=dev) * 15 - 1
    bb, cc, d = rn(B, 1, R, dt=torch.bfloat16) / 11, rn(B, 1, R, dt=torch.bfloat16) / 11, torch.rand(H, device=dev)
    ms = _time(lambda: bm.ops.step2(state, x, dt, a, bb, cc, d), args.iters, flush)
    nbytes = 2 * state.numel() * 4 + 2 * x.numel() * 2 + dt.numel() * 4 + 2 * bb.numel() * 2
    out.append(dict(kernel="step2 (Mamba-2 decode, b256 H80 P64 N128, one layer)", ms=ms, bytes=nbytes))

    # Mamba-1 selective scan
    b1, L, I, N = 4, 2048, 1536, 16
    u, delta, z = rn(b1, L, I, dt=torch.bfloat16), (torch.rand(b1, L, I, device=dev) * 0.1).bfloat16(), rn(b1, L, I, dt=torch.bfloat16)
    a1 = -torch.arange(1, N + 1, device=dev, dtype=torch.float32).repeat(I, 1).contiguous()
    b_, c_, d1 = rn(b1, L, N, dt=torch.bfloat16), rn(b1, L, N, dt=torch.bfloat16), torch.ones(I, device=dev)
    ms = _time(lambda: bm.ops.selscan1_fwd(u, delta, a1, b_, c_, d1, z=z), args.iters, flush)
    nbytes = 4 * u.numel() * 2 + 2 * b_.numel() * 2 + a1.numel() * 4 + 2 * b1 * I * N * 4
    out.append(dict(kernel="selscan1 (Mamba-1 scan, b4 L2048 i1536 N16, bf16)", ms=ms, bytes=nbytes))

    # Mamba-3 step (b256 H32 P64 N128 m4)
    B3, H3, M3 = 256, 32, 4
    st3, ks, vs_, ang = 0.1 * rn(B3, H3, P, R), rn(B3, M3, H3, R), rn(B3, H3, P), rn(B3, H3, R // 2)
    x3, b3, c3, rot = rn(B3, H3, P), rn(B3, M3, H3, R), rn(B3, M3, H3, R), rn(B3, R // 2)
    sc = lambda: torch.rand(B3, H3, device=dev) * 0.1
    dt3, al, be, ga = sc(), 1 - sc(), sc(), sc()
    mx = torch.full((H3, M3, P), 0.25, device=dev)
    ms = _time(lambda: bm.ops.step3(st3, ks, vs_, ang, x3, b3, c3, rot, dt3, al, be, ga, mx), args.iters, flush)
    nbytes = 2 * st3.numel() * 4 + 4 * ks.numel() * 4 + 3 * vs_.numel() * 4 + M3 * vs_.numel() * 4
    out.append(dict(kernel="step3 (Mamba-3 decode, b256 H32 P64 N128 m4)", ms=ms, bytes=nbytes))

    # conv step (b256, 5376 channels, k4)
    V = 5376
    win, xin, w, bias = rn(B, V, 4), rn(B, V, dt=torch.bfloat16), rn(V, 4), rn(V)
    ms = _time(lambda: bm.ops.conv_step(win, xin, w, bias), args.iters, flush)
    nbytes = 2 * win.numel() * 4 + 2 * xin.numel() * 2
    out.append(dict(kernel="conv_step (b256 v5376 k4)", ms=ms, bytes=nbytes))

    # angle scan (b16 L2048 H32 a64)
    rot_s, dt_s = rn(16, 2048, 64), torch.rand(16, 2048, 32, device=dev) * 0.1
    ms = _time(lambda: bm.ops.angle_cumsum(rot_s, dt_s), args.iters, flush)
    nbytes = 16 * 2048 * 32 * 64 * 4 + rot_s.numel() * 4 + dt_s.numel() * 4
    out.append(dict(kernel="angle_cumsum (b16 L2048 H32 a64)", ms=ms, bytes=nbytes))

    for o in out:
        o["gbs"] = o["bytes"] / (o["ms"] * 1e-3) / 1e9
        o["frac_of_hbm_peak"] = o["gbs"] / peak
        o["peak_gbs"] = peak
        o["peak_source"] = src
        print(json.dumps(o), flush=True)


if __name__ == "__main__":
    main()
