#!/usr/bin/env python
"""Benchmark of the SSM hot path: Mamba-2 SSD prefill at the 2.7B layer shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--regions R] [--impl reference]

One "step" = one pass of the Mamba-2 SSD forward (bm_ssd2_fwd) over the synthetic batch of the
2.7B-shape prefill configuration: batch 8, L 4096, H 80, P 64, N 128, G 1, chunk 256, bf16
activations, float32 decay/state.  `value` is tokens/s with inputs resident in HBM; `e2e` is the same
call made with HOST buffers (pinned -> device copies of x, dt, B, C and device -> host copies of y and
the final state inside the timed region).

With N > 1 (torchrun, one rank per GPU) the ONE batch-8 problem is split by (batch x head) units:
every rank generates and runs only its own units (whole batch rows for N = 2, 4, 8), there is no
data-path collective, and `value` = 32 768 tokens / max-over-ranks time ("scaling": "strong").  The
same line also carries `replicated` (every rank runs the whole problem: the weak-scaling figure) and
`head_split` (N/2 batch rows, each row's heads on two ranks, y all-gathered along heads over NCCL and
compared bit for bit with the one-GPU result) and `sequence_parallel` (one long sequence cut along time over the
ranks: zero-state pass, all-gather of the slice maps, second pass from the folded entering state; compared with the
one-GPU run of the whole sequence).

The timed region is repeated `--regions` times (each region: barrier, K back-to-back launches between
two CUDA events, barrier; per region the maximum over ranks); ms_per_step is the median region, min and
max are reported beside it.  Before timing, a few (batch, head) units of the very launch that is timed
are compared with the float32 exact path (`selfcheck_rel_l2`).

On one GPU the line also carries the other kernels of the path at their configured shapes (`kernels`),
the 64-layer decode step (`decode_step`: the SSM-step kernels alone and the whole step()), and the CPU
restatement of the reference timed on the host cores (`cpu_baseline`, all cores and one thread).

`--impl reference` times the CPU restatement of the reference's algorithm (oracle/csrc, C with
pthreads over batch x head) on a bounded sample of the same configuration: the reference itself
(Rust + un-vendored Burn) cannot be built without a Rust toolchain.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(batch=8, seqlen=4096, nheads=80, headdim=64, state_rank=128, ngroups=1, chunk_len=256)
WORKLOAD = "mamba2_ssd_prefill_2.7B_b8_L4096_H80_P64_N128_G1_Q256"
METRIC = "mamba2_ssd_prefill_tokens_per_s"
UNIT = "tokens/s"
SEED = 2
L2_BYTES = 126 << 20


def algorithmic_bytes(c, units=None):
    """x + y (bf16), B + C (bf16), dt (f32) per token, plus initial and final state (f32), for `units`
    (batch x head) units of configuration c (default: all of them)."""
    b, s, h, p, r, g = c["batch"], c["seqlen"], c["nheads"], c["headdim"], c["state_rank"], c["ngroups"]
    units = b * h if units is None else units
    per_unit_token = 2 * p * 2 + 4                       # x, y, dt of one head
    bc = 2 * 2 * g * r * b * s * (units / (b * h))       # B, C of the rows involved, shared by their heads
    return int(units * s * per_unit_token + bc + units * 2 * p * r * 4)


def algorithmic_flops(c, units=None):
    """Dense GEMM count of the chunked form, C.B^T counted once per group:
    2 [H P (Q + 2N) + G Q N] per token."""
    b, s, h, p, r, g, q = (c[k] for k in ("batch", "seqlen", "nheads", "headdim", "state_rank", "ngroups", "chunk_len"))
    units = b * h if units is None else units
    return int(2 * (h * p * (q + 2 * r) + g * q * r) * b * s * (units / (b * h)))


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            j = json.load(f)
        return float(j["hbm_gbs"]), float(j["bf16_tflops"]), "measured (MEASURED_PEAKS.json)"
    except Exception:
        return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and clock-event reasons of one GPU while the timed region runs (read-only).
    The samples come from NVML inside this process: a separate nvidia-smi polling loop was seen to hold
    driver locks for tens of milliseconds at a time, which stalled the kernel launches it was meant to
    observe.  nvidia-smi is only the fallback when the NVML binding is missing."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index, uuid=None, period_s=0.02):
        self.index, self.uuid, self.period = index, uuid, period_s
        self.rows, self.proc, self.thread, self.stop_flag, self.source = [], None, None, False, None

    # -- NVML in-process ---------------------------------------------------------------------
    def _nvml_loop(self, nv, handle):
        bits = [nv.nvmlClocksEventReasonHwSlowdown, nv.nvmlClocksEventReasonHwThermalSlowdown,
                nv.nvmlClocksEventReasonSwThermalSlowdown, nv.nvmlClocksEventReasonSwPowerCap]
        mx = nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM)
        while not self.stop_flag:
            try:
                sm = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(handle)
                self.rows.append([sm, mx] + ["Active" if mask & b else "Not Active" for b in bits])
            except Exception:
                pass
            time.sleep(self.period)

    def _start_nvml(self):
        import pynvml as nv
        nv.nvmlInit()
        handle = None
        if self.uuid:
            try:
                handle = nv.nvmlDeviceGetHandleByUUID(("GPU-" + self.uuid).encode())
            except Exception:
                handle = None
        if handle is None:
            handle = nv.nvmlDeviceGetHandleByIndex(self.index)
        nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)   # fail here, not in the thread
        self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
        self.thread.start()
        self.source = "nvml"

    # -- nvidia-smi fallback -----------------------------------------------------------------
    def _start_smi(self):
        self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index), "-lms", "200"], stdout=subprocess.PIPE,
                                     stderr=subprocess.DEVNULL, text=True)
        threading.Thread(target=self._read, daemon=True).start()
        self.source = "nvidia-smi"

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([p.strip() for p in line.split(",")])

    def start(self):
        try:
            try:
                self._start_nvml()
            except Exception:
                self._start_smi()
            # the first sample marks the end of the sampler's own start-up work
            t0 = time.time()
            while not self.rows and time.time() - t0 < 10.0:
                time.sleep(0.02)
            self.warm = len(self.rows)
        except Exception:
            self.proc = None

    def stop(self):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=2)
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm, mx, reasons = [], [], set()
        for r in self.rows[getattr(self, "warm", 0):] or self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                for n, v in zip(self.NAMES, r[2:6]):
                    if str(v).lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": self.source}


def head_params(torch, seed, c):
    """Per-head parameters of the configuration (the same on every rank): dt_bias, A, D."""
    g = torch.Generator().manual_seed(seed)
    h = c["nheads"]
    lo, hi = torch.log(torch.tensor(1e-3)), torch.log(torch.tensor(1e-1))
    dt0 = torch.exp(torch.rand(h, generator=g) * (hi - lo) + lo)
    dt_bias = dt0 + torch.log(-torch.expm1(-dt0))
    a = -(torch.rand(h, generator=g) * 15.0 + 1.0)
    d = torch.rand(h, generator=g)
    return dt_bias.float(), a.float(), d.float()


def make_rows(torch, seed, c, b_lo, b_hi, h_lo, h_hi, dt_bias):
    """Seeded synthetic inputs of batch rows [b_lo, b_hi), heads [h_lo, h_hi) of the configuration (host,
    pinned).  Every batch row has its own generator, so a rank can draw exactly its rows and any other
    rank (or a one-GPU run) draws the same values for them."""
    s, h, p, r, ng = c["seqlen"], c["nheads"], c["headdim"], c["state_rank"], c["ngroups"]
    xs, dts, bs, cs = [], [], [], []
    for row in range(b_lo, b_hi):
        g = torch.Generator().manual_seed(seed * 1009 + row)
        xs.append(torch.randn((s, h, p), generator=g).to(torch.bfloat16)[:, h_lo:h_hi])
        dts.append(torch.nn.functional.softplus(torch.randn((s, h), generator=g) + dt_bias).float()[:, h_lo:h_hi])
        bs.append((torch.randn((s, ng, r), generator=g) / r ** 0.5).to(torch.bfloat16))
        cs.append((torch.randn((s, ng, r), generator=g) / r ** 0.5).to(torch.bfloat16))
    out = dict(x=torch.stack(xs), dt=torch.stack(dts), b=torch.stack(bs), c=torch.stack(cs))
    return {k: v.contiguous().pin_memory() for k, v in out.items()}


class Slice:
    """One rectangle (rows x heads) of the problem on this rank: host tensors, device copies, pinned
    result buffers."""

    def __init__(self, torch, dev, c, rect, params):
        self.rect = b_lo, b_hi, h_lo, h_hi = rect
        dt_bias, a, d = params
        self.host = make_rows(torch, SEED, c, b_lo, b_hi, h_lo, h_hi, dt_bias)
        self.a = a[h_lo:h_hi].clone().to(dev)
        self.d = d[h_lo:h_hi].clone().to(dev)
        self.dev = {k: v.to(dev, non_blocking=True) for k, v in self.host.items()}
        nb, nh = b_hi - b_lo, h_hi - h_lo
        self.units = nb * nh
        self.y_host = torch.empty((nb, c["seqlen"], nh, c["headdim"]), dtype=torch.bfloat16).pin_memory()
        self.h_host = torch.empty((nb, nh, c["headdim"], c["state_rank"]), dtype=torch.float32).pin_memory()

    def in_bytes(self):
        return sum(v.numel() * v.element_size() for v in self.host.values())


def run_ours(args):
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    bm = ge.load_package()
    c = dict(CFG, batch=args.batch)
    params = head_params(torch, SEED, c)
    parts = bm.shard.partition_units(c["batch"], c["nheads"], c["ngroups"], world)
    mine = parts[rank]
    slices = [Slice(torch, dev, c, rect, params) for rect in mine.calls()]
    torch.cuda.synchronize()
    Q = c["chunk_len"]

    # Input sets: when this rank's inputs are smaller than a few L2 sizes, the timed launches rotate through
    # copies of them so that no launch finds its inputs in L2
    in_bytes = sum(s.in_bytes() for s in slices)
    nsets = 1 if in_bytes > 2 * L2_BYTES else int(-(-3 * L2_BYTES // max(in_bytes, 1)))
    sets = [[s.dev for s in slices]] + [[{k: v.clone() for k, v in s.dev.items()} for s in slices]
                                        for _ in range(nsets - 1)]
    rot = [0]

    def step_resident():
        cur = sets[rot[0] % nsets]
        rot[0] += 1
        out = None
        for s, t in zip(slices, cur):
            out = bm.ops.ssd2_fwd(t["x"], t["dt"], s.a, t["b"], t["c"], s.d, None, chunk_len=Q, path="auto")
        return out

    # End-to-end leg: every step copies this rank's inputs from pinned host memory, runs the SSD and reads y
    # and the final state back.  The three stages run on three streams with two sets of device input buffers,
    # so the upload of step i+1 and the download of step i-1 overlap the kernel of step i (PCIe is full
    # duplex); a step still cannot start before its own inputs have landed, nor finish before its outputs are home.
    s_in, s_comp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    in_bufs = [[{k: torch.empty_like(v) for k, v in s.dev.items()} for s in slices] for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    e2e_count = [0]

    def step_e2e():
        i = e2e_count[0] & 1
        e2e_count[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[i])            # the kernel two steps back has finished with this set
            for s, t in zip(slices, in_bufs[i]):
                for k in t:
                    t[k].copy_(s.host[k], non_blocking=True)
            in_ready[i].record(s_in)
        outs = []
        with torch.cuda.stream(s_comp):
            s_comp.wait_event(in_ready[i])
            for s, t in zip(slices, in_bufs[i]):
                outs.append(bm.ops.ssd2_fwd(t["x"], t["dt"], s.a, t["b"], t["c"], s.d, None, chunk_len=Q, path="auto"))
            in_free[i].record(s_comp)
            done = torch.cuda.Event()
            done.record(s_comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            for s, (y, hf) in zip(slices, outs):
                s.y_host.copy_(y, non_blocking=True)
                s.h_host.copy_(hf, non_blocking=True)
                y.record_stream(s_out)
                hf.record_stream(s_out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, streams=(), regions=1):
        """CUDA-event times of `regions` regions of `steps` calls of fn, each region the maximum over ranks.
        `streams`: side streams fn issues work on; they start after the first event and the second event
        waits for all of them."""
        out = []
        for _ in range(regions):
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            ev0.record()
            for st in streams:
                st.wait_event(ev0)
            for _ in range(steps):
                fn()
            for st in streams:
                e = torch.cuda.Event()
                e.record(st)
                torch.cuda.current_stream().wait_event(e)
            ev1.record()
            barrier()
            out.append(ev0.elapsed_time(ev1))
        ms = torch.tensor(out, device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return [float(v) for v in ms.tolist()]

    for _ in range(max(args.warmup, 3)):
        step_resident()
    # device status of the tensor-core kernel (bounded waits) -- checked once, outside the timed region
    for s in slices:
        t = s.dev
        bm.ops.ssd2_fwd(t["x"], t["dt"], s.a, t["b"], t["c"], s.d, None, chunk_len=Q, path="auto", check_status=True)

    # Self-check of the launch that is timed: a few (batch, head) units of its output against the float32
    # exact path on the same device inputs (rel-L2 per unit; the parity tolerance for bf16 is 2e-2)
    def selfcheck():
        g = torch.Generator().manual_seed(1234 + rank)
        worst = 0.0
        for s in slices:
            t = s.dev
            y, hf = bm.ops.ssd2_fwd(t["x"], t["dt"], s.a, t["b"], t["c"], s.d, None, chunk_len=Q, path="auto")
            nb, nh = y.shape[0], y.shape[2]
            picks = {(0, 0), (nb - 1, nh - 1)}
            while len(picks) < min(4, nb * nh):
                picks.add((int(torch.randint(nb, (1,), generator=g)), int(torch.randint(nh, (1,), generator=g))))
            for bi, hi in sorted(picks):
                ye, he = bm.ops.ssd2_fwd(t["x"][bi:bi + 1, :, hi:hi + 1].contiguous(), t["dt"][bi:bi + 1, :, hi:hi + 1].contiguous(),
                                         s.a[hi:hi + 1].clone(), t["b"][bi:bi + 1].contiguous(), t["c"][bi:bi + 1].contiguous(),
                                         s.d[hi:hi + 1].clone(), None, chunk_len=Q, path="exact")
                rel = lambda got, want: float((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-30))
                worst = max(worst, rel(y[bi:bi + 1, :, hi:hi + 1], ye), rel(hf[bi:bi + 1, hi:hi + 1], he))
        w = torch.tensor([worst], device=dev)
        if world > 1:
            dist.all_reduce(w, op=dist.ReduceOp.MAX)
        return float(w.item())

    selfcheck_rel = selfcheck()
    if not selfcheck_rel <= 2e-2:
        raise RuntimeError(f"self-check failed: rel-L2 {selfcheck_rel} against the exact path exceeds 2e-2")

    try:
        gpu_uuid = str(torch.cuda.get_device_properties(local).uuid)
    except Exception:
        gpu_uuid = None
    sampler = ClockSampler(local, gpu_uuid)
    # reference point without any sampler running: a timed region several times slower than this is a
    # disturbed measurement (launches stalled behind a driver lock), which is taken once more and reported
    quick_ms = timed(step_resident, 10)[0] / 10
    if rank == 0:
        sampler.start()
    region_ms = timed(step_resident, args.steps, regions=args.regions)
    clocks = sampler.stop() if rank == 0 else None
    remeasured = None
    if statistics.median(region_ms) / args.steps > 2.5 * quick_ms:
        remeasured = {"first_ms_per_step": statistics.median(region_ms) / args.steps, "undisturbed_ms_per_step": quick_ms,
                      "reason": "timed regions >2.5x slower than the same launches without the clock sampler"}
        sampler = ClockSampler(local, gpu_uuid, period_s=0.05)
        if rank == 0:
            sampler.start()
        region_ms = timed(step_resident, args.steps, regions=args.regions)
        clocks = sampler.stop() if rank == 0 else None
    # a bounded wait that ran out during the timed launches would have left its code in the workspace
    st = bm.ops.last_workspace_status()
    if st != 0:
        raise RuntimeError(f"tensor-core kernel reported status {st} during the timed region")
    e2e_steps = max(1, min(args.steps, 20))
    if args.profile:  # kernel-only run for ncu captures: no end-to-end leg, no other legs
        ms_e2e = float("nan")
    else:
        for _ in range(2):
            step_e2e()
        ms_e2e = timed(step_e2e, e2e_steps, streams=(s_in, s_comp, s_out))[0]

    tokens = c["batch"] * c["seqlen"]
    per_step = sorted(m / args.steps for m in region_ms)
    ms_step = statistics.median(per_step)
    value = tokens / (ms_step * 1e-3)
    e2e_value = tokens / (ms_e2e / e2e_steps * 1e-3)
    peak, peak_tf, peak_src = measured_peaks()
    # roofline of this rank's kernel launch: the largest share any rank holds
    units_max = max(p.count for p in parts)
    abytes = algorithmic_bytes(c, units_max)
    achieved = abytes / (ms_step * 1e-3) / 1e9
    h2d = torch.tensor([float(in_bytes)], device=dev)
    d2h = torch.tensor([float(sum(s.y_host.numel() * 2 + s.h_host.numel() * 4 for s in slices))], device=dev)
    if world > 1:
        dist.all_reduce(h2d)
        dist.all_reduce(d2h)
    launches_per_step = len(slices)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "problem": dict(c),
                   "parallelism": f"(batch x head) units split over {world} rank(s): {[p.count for p in parts]} units, "
                                  f"no data-path collective",
                   "l2": (f"inputs larger than L2 ({in_bytes >> 20} MB read per step per rank)" if nsets == 1 else
                          f"{nsets} rotating input sets of {in_bytes >> 20} MB per rank (> 3 x L2 between reuses)"),
                   "path": "tcgen05 tensor-core kernel"},
        "regions": {"count": len(per_step), "steps_per_region": args.steps, "ms_per_step_median": ms_step,
                    "ms_per_step_min": per_step[0], "ms_per_step_max": per_step[-1]},
        "selfcheck_rel_l2": selfcheck_rel,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(h2d.item()), "d2h_bytes_per_step": int(d2h.item()),
                "steps": e2e_steps},
        "gpu_launches": args.steps * len(per_step) * launches_per_step,
        "clocks": clocks,
        "remeasured": remeasured,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_src, "algorithmic_bytes": abytes, "units_in_launch": units_max,
                     "traffic": traffic_bytes_per_launch(units_max),
                     "tensor_view": {"algorithmic_flops": algorithmic_flops(c, units_max),
                                     "achieved_tflops": algorithmic_flops(c, units_max) / (ms_step * 1e-3) / 1e12,
                                     "peak_tflops": peak_tf,
                                     "frac": algorithmic_flops(c, units_max) / (ms_step * 1e-3) / 1e12 / peak_tf}},
    }
    if world > 1 and not args.profile:
        line["replicated"] = replicated_leg(torch, dist, bm, dev, c, params, timed, world)
        line["head_split"] = head_split_leg(torch, dist, bm, dev, c, params, timed, rank, world)
        line["sequence_parallel"] = sequence_parallel_leg(torch, dist, bm, dev, c, rank, world)
    if rank == 0:
        extra = not args.profile and world == 1
        line["cpu_baseline"] = None if args.profile else cpu_baseline(budget_s=20.0, one_thread=True)
        line["kernels"] = kernel_legs(torch, bm, dev) if extra else None
        # second headline of the benchmark definition: decode-step time of the 64-layer stack (N = 1 only)
        line["decode_step"] = decode_step_leg(torch, bm, dev) if extra else None
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_leg(args):
    """One leg alone, for profiler captures (rank 0, one GPU): prints that leg's JSON."""
    import torch
    import __graft_entry__ as ge
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    bm = ge.load_package()
    if args.leg == "kernels":
        out = kernel_legs(torch, bm, dev, iters=3 if args.small else 10, small=args.small)
    else:
        out = decode_step_leg(torch, bm, dev, layers=2 if args.small else 64, steps=2 if args.small else 8)
    print(json.dumps({"leg": args.leg, "small": bool(args.small), "result": out}), flush=True)


def replicated_leg(torch, dist, bm, dev, c, params, timed, world):
    """Every rank runs the whole batch-8 problem (independent replicas): the weak-scaling figure."""
    s = Slice(torch, dev, c, (0, c["batch"], 0, c["nheads"]), params)
    t = s.dev
    fn = lambda: bm.ops.ssd2_fwd(t["x"], t["dt"], s.a, t["b"], t["c"], s.d, None, chunk_len=c["chunk_len"], path="auto")
    for _ in range(3):
        fn()
    ms = statistics.median(timed(fn, 20, regions=5)) / 20
    return {"value": c["batch"] * c["seqlen"] * world / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "scaling": "weak",
            "note": "every rank runs the whole problem; aggregate over ranks"}


def sequence_parallel_leg(torch, dist, bm, dev, c, rank, world, seqlen=131072, batch=2, iters=5):
    """One sequence of `batch` x `seqlen` tokens (the configuration's heads) cut along time into `world` slices
    (shard.ssd2_fwd_sequence_parallel): every rank runs its slice from zero, the slice end states and decays are
    all-gathered over NCCL, every rank but the first runs its slice again from its folded entering state.  Timed as
    the maximum over ranks; the result is compared with this rank's own one-GPU run of the whole sequence."""
    H, P, R, G, Q = c["nheads"], c["headdim"], c["state_rank"], c["ngroups"], c["chunk_len"]
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(batch, seqlen, H, P, generator=g, device=dev).bfloat16()
    dt = torch.exp(torch.rand(batch, seqlen, H, generator=g, device=dev) * 4.6 - 6.9)
    a = -torch.exp(torch.rand(H, generator=g, device=dev) * 2.0)
    b = torch.randn(batch, seqlen, G, R, generator=g, device=dev).bfloat16()
    cc = torch.randn(batch, seqlen, G, R, generator=g, device=dev).bfloat16()
    d = torch.ones(H, device=dev)
    fwd = lambda x_, dt_, a_, b_, c_, d_, h0_, q: bm.ops.ssd2_fwd(x_, dt_, a_, b_, c_, d_, h0_, chunk_len=q, path="auto")
    cuts = bm.shard.sequence_cuts(seqlen, world, Q)   # rank 0 runs once and takes a double slice
    cut = slice(*cuts[rank])
    xs, dts, bs, cs = (t[:, cut].contiguous() for t in (x, dt, b, cc))
    run = lambda: bm.shard.ssd2_fwd_sequence_parallel(fwd, xs, dts, a, bs, cs, d, None, Q, rank, world)
    for _ in range(3):
        y, hf = run()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        y, hf = run()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    for _ in range(2):
        y1, h1 = fwd(x, dt, a, b, cc, d, None, Q)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        y1, h1 = fwd(x, dt, a, b, cc, d, None, Q)
    e1.record()
    torch.cuda.synchronize()
    one = e0.elapsed_time(e1) / iters
    equal = torch.tensor([int(torch.equal(y, y1[:, cut])) and int(torch.allclose(hf, h1, rtol=1e-5, atol=1e-6))], device=dev)
    dist.all_reduce(equal, op=dist.ReduceOp.MIN)
    return {"batch": batch, "seqlen": seqlen, "slices": [hi - lo for lo, hi in cuts], "ms": ms.item(), "one_gpu_ms": one,
            "value": batch * seqlen / (ms.item() * 1e-3), "unit": "tokens/s",
            "y_equal_to_one_gpu_bitwise": bool(equal.item()),
            "exchange_bytes_per_rank": batch * H * P * R * 4 + batch * H * 4,
            "note": "two passes on every rank but the first; the exchange does not grow with the sequence"}


def head_split_leg(torch, dist, bm, dev, c, params, timed, rank, world):
    """world / 2 batch rows, each row's 80 heads on two ranks: SSD on the local heads, then the all-gather of
    y (and the final state) along heads over NCCL that the gated norm after the SSD needs
    (src/mamba2/mamba2.rs:776).  Each rank compares the gathered row bit for bit with its own one-GPU run of
    that row."""
    cc = dict(c, batch=max(world // 2, 1))
    shard = bm.shard
    parts = shard.partition_heads(cc["batch"], cc["nheads"], world)
    mine = parts[rank]
    sl = [Slice(torch, dev, cc, rect, params) for rect in mine.calls()]
    fwd = lambda x, dt, a, b, c_, d, h0, q: bm.ops.ssd2_fwd(x, dt, a, b, c_, d, h0, chunk_len=q, path="auto")

    def local():
        return [(s.rect[0], s.rect[1], s.rect[2], s.rect[3]) +
                tuple(fwd(s.dev["x"], s.dev["dt"], s.a, s.dev["b"], s.dev["c"], s.d, None, cc["chunk_len"])) for s in sl]

    def step():
        return shard.gather_heads(local(), parts, rank, world, cc["nheads"])

    rows = step()
    equal = True
    for row, (y, hf) in rows.items():
        full = Slice(torch, dev, cc, (row, row + 1, 0, cc["nheads"]), params)
        y1, h1 = fwd(full.dev["x"], full.dev["dt"], full.a, full.dev["b"], full.dev["c"], full.d, None, cc["chunk_len"])
        equal = equal and bool(torch.equal(y, y1)) and bool(torch.equal(hf, h1))
    eq = torch.tensor([1.0 if equal else 0.0], device=dev)
    dist.all_reduce(eq, op=dist.ReduceOp.MIN)
    for _ in range(2):
        step()
    ms_total = statistics.median(timed(step, 10, regions=5)) / 10
    ms_local = statistics.median(timed(local, 10, regions=5)) / 10
    gathered = sum(s.y_host.numel() * 2 + s.h_host.numel() * 4 for s in sl)
    return {"batch": cc["batch"], "units_per_rank": [p.count for p in parts], "ms_per_step": ms_total,
            "ms_ssd_only": ms_local, "ms_allgather": ms_total - ms_local, "bytes_contributed_per_rank": gathered,
            "value": cc["batch"] * cc["seqlen"] / (ms_total * 1e-3), "unit": UNIT,
            "bitwise_equal_to_one_gpu": bool(eq.item() == 1.0), "collective": "all_gather_into_tensor (NCCL) per split row"}


def _time_flushed(torch, fn, iters, flush):
    """Mean CUDA-event time of fn over `iters` launches, L2 flushed (a buffer larger than L2 rewritten)
    before each one."""
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def kernel_legs(torch, bm, dev, iters=10, small=False):
    """The other kernels of the path at their configured shapes: device time (CUDA events, L2 flushed between
    launches), algorithmic bytes or flops, and the fraction of the measured peak that bounds each.  `small` cuts
    the batch-like axes (profiler captures only; the figures are then not the configured shapes')."""
    sb = (lambda n, m=1: max(m, n // 8)) if small else (lambda n, m=1: n)
    peak, peak_tf, src = measured_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(3)
    rn = lambda *s, dt=torch.float32: torch.randn(*s, generator=g, device=dev).to(dt)
    bf = torch.bfloat16
    out = []

    def hbm(name, ms, nbytes):
        gbs = nbytes / (ms * 1e-3) / 1e9
        out.append({"kernel": name, "ms": ms, "bound": "hbm", "algorithmic_bytes": int(nbytes), "achieved_gbs": gbs,
                    "frac": gbs / peak, "peak": peak})

    def tensor(name, ms, flops, note):
        tf = flops / (ms * 1e-3) / 1e12
        out.append({"kernel": name, "ms": ms, "bound": "tensor", "algorithmic_flops": int(flops), "achieved_tflops": tf,
                    "frac": tf / peak_tf, "peak": peak_tf, "note": note})

    # Mamba-1 selective scan at its configuration (b4 L2048 i1536 N16, bf16, gate through SiLU)
    b1, L, I, N = sb(4), 2048, 1536, 16
    u, z = rn(b1, L, I, dt=bf), rn(b1, L, I, dt=bf)
    delta = torch.exp(torch.rand(b1, L, I, device=dev) * 4.6 - 6.9).to(bf)
    a1 = -torch.arange(1, N + 1, device=dev, dtype=torch.float32).repeat(I, 1).contiguous()
    b_, c_, d1 = rn(b1, L, N, dt=bf), rn(b1, L, N, dt=bf), torch.ones(I, device=dev)
    ms = _time_flushed(torch, lambda: bm.ops.selscan1_fwd(u, delta, a1, b_, c_, d1, z=z), iters, flush)
    hbm(f"selscan1_fwd (Mamba-1 scan, b{b1} L2048 i1536 N16, bf16)", ms,
        4 * u.numel() * 2 + 2 * b_.numel() * 2 + a1.numel() * 4 + 2 * b1 * I * N * 4)

    # Mamba-3 decode step (b256 H32 P64 N128 m4)
    B3, H3, M3, P, R = sb(256), 32, 4, 64, 128
    st3, ks, vs_, ang = 0.1 * rn(B3, H3, P, R), rn(B3, M3, H3, R), rn(B3, H3, P), rn(B3, H3, R // 2)
    x3, b3, c3, rot = rn(B3, H3, P), rn(B3, M3, H3, R), rn(B3, M3, H3, R), rn(B3, R // 2)
    sc = lambda: torch.rand(B3, H3, device=dev) * 0.1
    dt3, al, be, ga = sc(), 1 - sc(), sc(), sc()
    mx = torch.full((H3, M3, P), 0.25, device=dev)
    ms = _time_flushed(torch, lambda: bm.ops.step3(st3, ks, vs_, ang, x3, b3, c3, rot, dt3, al, be, ga, mx), iters, flush)
    hbm(f"step3 (Mamba-3 decode, b{B3} H32 P64 N128 m4)", ms,
        2 * st3.numel() * 4 + 4 * ks.numel() * 4 + 3 * vs_.numel() * 4 + M3 * vs_.numel() * 4)
    del st3

    # conv window step (b256, 5376 channels, k4)
    B, V = 256, 5376
    win, xin, w, bias = rn(B, V, 4), rn(B, V, dt=bf), rn(V, 4), rn(V)
    ms = _time_flushed(torch, lambda: bm.ops.conv_step(win, xin, w, bias), iters, flush)
    hbm("conv_step (b256 v5376 k4)", ms, 2 * win.numel() * 4 + 2 * xin.numel() * 2)

    # angle scan (b16 L2048 H32 a64)
    rot_s, dt_s = rn(16, 2048, 64), torch.rand(16, 2048, 32, device=dev) * 0.1
    ms = _time_flushed(torch, lambda: bm.ops.angle_cumsum(rot_s, dt_s), iters, flush)
    hbm("angle_cumsum (b16 L2048 H32 a64)", ms, 16 * 2048 * 32 * 64 * 4 + rot_s.numel() * 4 + dt_s.numel() * 4)
    del rot_s

    for extra in (_prefill_glue_legs, _ssd3_legs, _ssd2_bwd_leg):
        try:
            extra(torch, bm, dev, rn, flush, hbm, tensor, sb)
        except torch.cuda.OutOfMemoryError:
            out.append({"kernel": extra.__name__, "skipped": "out of device memory"})
        torch.cuda.empty_cache()
    return out


def _prefill_glue_legs(torch, bm, dev, rn, flush, hbm, tensor, sb):
    """Pre-/post-SSD kernels of the Mamba-2 block at the prefill configuration (when the library has them)."""
    bf = torch.bfloat16
    if hasattr(bm.ops, "conv1d_silu_fwd"):
        b, s, v, k = sb(8), 4096, 5376, 4
        xbc, w, bias, prev = rn(b, s, v, dt=bf), rn(v, k), rn(v), rn(b, v, k)
        ms = _time_flushed(torch, lambda: bm.ops.conv1d_silu_fwd(xbc, w, bias, prev, splits=(5120, 128, 128)), 5, flush)
        hbm(f"conv1d_silu_fwd (prefill conv k4 + bias + SiLU, b{b} L4096 v5376, bf16)", ms, 2 * xbc.numel() * 2)
    if hasattr(bm.ops, "rmsnorm_gated"):
        b, s, i = sb(8), 4096, 5120
        y, z, gamma = rn(b * s, i, dt=bf), rn(b * s, i, dt=bf), rn(i, dt=bf)
        ms = _time_flushed(torch, lambda: bm.ops.rmsnorm_gated(y, z, gamma), 5, flush)
        hbm(f"rmsnorm_gated (b{b} L4096 d_inner 5120, bf16)", ms, 3 * y.numel() * 2)


def _ssd3_legs(torch, bm, dev, rn, flush, hbm, tensor, sb):
    """Mamba-3 single SSD forward and recompute backward at the configured shape
    (b16 L2048 H32 P64 N128 m4 Q64, bf16 / float32 state)."""
    bf = torch.bfloat16
    b, s, m, h, p, r, q = sb(16, 2), 2048, 4, 32, 64, 128, 64
    v = rn(b, s, 1, h, p, dt=bf).expand(b, s, m, h, p).contiguous() / m
    bb, cc = rn(b, s, m, h, r, dt=bf) / r ** 0.5, rn(b, s, m, h, r, dt=bf) / r ** 0.5
    dt = torch.rand(b, s, h, device=dev) * 0.05 + 1e-3
    a = -(torch.rand(h, device=dev) * 15 + 1)
    lam = torch.sigmoid(rn(b, s, h))
    da, gamma = dt * a, lam * dt
    scale = gamma.clone()
    scale[:, :-1] += (dt * (1 - lam))[:, 1:]
    angles = torch.cumsum(dt[..., None] * rn(b, s, h, r // 2), dim=1)
    # forward flops: C.B^T 2 LM^2 N + intra 2 LM^2 P + state 2 LM N P + readout 2 LM N P per (b, chunk, h)
    lm = q * m
    flops = (2 * lm * lm * r + 2 * lm * lm * p + 4 * lm * r * p) * b * (s // q) * h
    path = "tensor" if getattr(bm.ops, "SSD3_TENSOR_PATH", False) else "exact"
    fwd = lambda: bm.ops.ssd3_single_fwd(v, da, bb, cc, gamma, scale, None, chunk_len=q, angles=angles, rope_dim=r, path=path)
    ms = _time_flushed(torch, fwd, 5, flush)
    tensor(f"ssd3_single_fwd (b{b} L2048 H32 P64 N128 m4 Q64, bf16, rotation from angles, {path} path)", ms, flops,
           "dense GEMM count of the fused (time x rank) axis")
    if hasattr(bm.ops, "mamba3_bc_prep"):
        # B / C from the projection's raw group columns to the rotated per-head tensors the slot takes, one kernel
        braw, craw = rn(b, s, m * r, dt=bf), rn(b, s, m * r, dt=bf)
        gam, bias = torch.ones(r, device=dev), 0.1 * rn(h, m, r)
        ms = _time_flushed(torch, lambda: bm.ops.mamba3_bc_prep(braw, craw, gam, gam, bias, bias, angles=angles, rope_dim=r,
                                                              pairwise=False, ngroups=1), 5, flush)
        hbm(f"mamba3_bc_prep (norm + expand + bias + rotation, b{b} L2048 m4 g1 H32 N128, bf16)", ms,
            2 * braw.numel() * 2 + angles.numel() * 4 + 2 * bb.numel() * 2)
    del angles
    dy = rn(b, s, m, h, p, dt=bf)
    bwd = lambda: bm.ops.ssd3_bwd(v, da, bb, cc, gamma, scale, None, dy, None, chunk_len=q, single=True)
    ms = _time_flushed(torch, bwd, 5, flush)
    tensor("ssd3_single_bwd (same shape, recompute backward on the tensor cores, pre-rotated B/C)", ms, 2.5 * flops, "2.5 x the forward count")


def _ssd2_bwd_leg(torch, bm, dev, rn, flush, hbm, tensor, sb):
    """Mamba-2 recompute backward at the prefill configuration (b8 L4096 H80 P64 N128 G1 Q256, bf16)."""
    bf = torch.bfloat16
    c = dict(CFG, batch=sb(8))
    b, s, h, p, r, q = c["batch"], c["seqlen"], c["nheads"], c["headdim"], c["state_rank"], c["chunk_len"]
    x, dy = rn(b, s, h, p, dt=bf), rn(b, s, h, p, dt=bf)
    dt = torch.rand(b, s, h, device=dev) * 0.05 + 1e-3
    a, d = -(torch.rand(h, device=dev) * 15 + 1), torch.rand(h, device=dev)
    bb, cc = rn(b, s, 1, r, dt=bf) / r ** 0.5, rn(b, s, 1, r, dt=bf) / r ** 0.5
    ms = _time_flushed(torch, lambda: bm.ops.ssd2_bwd(x, dt, a, bb, cc, d, None, dy, None, chunk_len=q), 5, flush)
    tensor(f"ssd2_bwd (b{b} L4096 H80 P64 N128 G1 Q256, bf16, recompute backward on the tensor cores)", ms, 2.5 * algorithmic_flops(c),
           "2.5 x the forward count")


def decode_step_leg(torch, bm, dev, layers=64, batch=256, steps=8):
    """Mamba-2 recurrent step() of a 64-layer stack at the 2.7B shape, batch 256, on per-layer float32 states
    resident in HBM (64 x 671 MB).  Two figures: the SSM-step kernels of every layer alone (conv window step +
    state update/readout: the hot path), and the whole step() of the stack (layer norm, in_proj, conv step,
    state step, gated norm, out_proj, residual per layer, src/modules/layers.rs:427-497) eagerly launched and
    replayed from a CUDA graph."""
    H, P, R, V, K, DM = 80, 64, 128, 5376, 4, 2560
    bf = torch.bfloat16
    try:
        states = [0.1 * torch.randn((batch, H, P, R), device=dev) for _ in range(layers)]
    except torch.cuda.OutOfMemoryError:
        return None
    wins = [0.1 * torch.randn((batch, V, K), device=dev) for _ in range(layers)]
    w, bias = torch.randn((V, K), device=dev), torch.randn((V,), device=dev)
    xin = torch.randn((batch, V), device=dev).to(bf)
    dt = torch.rand((batch, H), device=dev) * 0.1
    a, d = -(torch.rand(H, device=dev) * 15 + 1), torch.rand(H, device=dev)

    def ssm_only():
        for l in range(layers):
            x, bb, cc = bm.ops.conv_step(wins[l], xin, w, bias, splits=(H * P, R, R))
            bm.ops.step2(states[l], x.view(batch, H, P), dt, a, bb.view(batch, 1, R), cc.view(batch, 1, R), d)

    def time_steps(fn, n):
        for _ in range(2):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / n

    us = time_steps(ssm_only, steps)
    per_layer = 2 * batch * H * P * R * 4 + 2 * batch * V * K * 4 + 2 * batch * V * 2 + 2 * batch * H * P * 2 + batch * H * 4
    peak, _, _ = measured_peaks()
    gbs = per_layer * layers / (us * 1e-6) / 1e9
    res = {"us_per_step": us, "layers": layers, "batch": batch, "kernels_per_step": 2 * layers,
           "algorithmic_bytes_per_step": per_layer * layers, "achieved_gbs": gbs, "frac_of_hbm_peak": gbs / peak,
           "scope": "SSM-step kernels (conv_step + step2) of all layers; states larger than L2"}

    # whole step(): random-init weights of the 2.7B layer, bf16 activations / weights, float32 caches
    try:
        g = torch.Generator(device=dev).manual_seed(3)
        u = lambda *s, k=1.0: ((torch.rand(*s, generator=g, device=dev) * 2 - 1) * k)
        blocks, norms = [], []
        for l in range(layers):
            blk = bm.Mamba2(u(DM, 2 * H * P + 2 * R + H, k=DM ** -0.5).to(bf), u(V, K, k=0.5), u(V, k=0.5),
                            torch.log(torch.expm1(torch.full((H,), 0.01, device=dev))), torch.log(1 + 15 * torch.rand(H, generator=g, device=dev)),
                            torch.ones(H, device=dev), torch.ones(H * P, device=dev).to(bf), u(H * P, DM, k=(H * P) ** -0.5).to(bf),
                            nheads=H, state_rank=R, ngroups=1)
            blocks.append(blk)
            norms.append(torch.ones(DM, device=dev).to(bf))
        caches = [bm.Mamba2Cache(wins[l], states[l]) for l in range(layers)]
        h_in = torch.randn((batch, DM), device=dev).to(bf)
        stack_step = getattr(bm.mamba2, "stack_step")

        def whole():
            return stack_step(blocks, norms, caches, h_in)

        us_eager = time_steps(whole, 4)
        res["whole_step_us_eager"] = us_eager
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            whole()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            out = whole()
        us_graph = time_steps(graph.replay, 8)
        weights = layers * (DM * (2 * H * P + 2 * R + H) + H * P * DM) * 2
        res.update({"whole_step_us": us_graph, "whole_step_launch": "one CUDA graph replay per step",
                    "whole_step_bytes": per_layer * layers + weights,
                    "whole_step_frac_of_hbm_peak": (per_layer * layers + weights) / (us_graph * 1e-6) / 1e9 / peak,
                    "whole_step_finite": bool(torch.isfinite(out.float()).all())})
    except Exception as e:   # the SSM-step figure stands on its own
        res["whole_step_error"] = f"{type(e).__name__}: {e}"[:300]
    return res


# dram__bytes_read.sum + dram__bytes_write.sum of one tensor-core launch of the whole benchmark problem (640 units),
# from an ncu capture of that launch itself: 373.9 MB read + 313.3 MB written (part of y is still dirty in L2 when
# the kernel ends), per unit
TRAFFIC_BYTES_PER_UNIT = (373.9e6 + 313.3e6) / 640


def traffic_bytes_per_launch(units):
    return None if TRAFFIC_BYTES_PER_UNIT is None else TRAFFIC_BYTES_PER_UNIT * units


def cpu_sample(batch, nheads):
    """A bounded sample of the benchmark configuration for the CPU arm: full sequence length, full
    head shape, fewer (batch x head) units -- units are independent, so tokens/s scales by units."""
    import numpy as np
    rng = np.random.Generator(np.random.PCG64(2))
    c = dict(CFG, batch=batch, nheads=nheads)
    f = np.float32
    b, s, h, p, r, g = c["batch"], c["seqlen"], c["nheads"], c["headdim"], c["state_rank"], c["ngroups"]
    x = rng.standard_normal((b, s, h, p), dtype=f)
    dt = np.log1p(np.exp(rng.standard_normal((b, s, h), dtype=f) - 4.0)).astype(f)
    a = (-rng.uniform(1.0, 16.0, h)).astype(f)
    bb = (rng.standard_normal((b, s, g, r), dtype=f) / np.sqrt(r)).astype(f)
    cc = (rng.standard_normal((b, s, g, r), dtype=f) / np.sqrt(r)).astype(f)
    d = rng.uniform(0.0, 1.0, h).astype(f)
    return c, (x, dt, a, bb, cc, d)


def cpu_baseline(budget_s=20.0, steps=1, warmup=0, one_thread=False):
    """Times the C restatement of the reference's serial SSD on the host cores (all of them) on a
    sample of `units` (batch x head) problems; reported as whole-configuration tokens/s equivalents:
    tokens/s = (sample token-heads / s) / nheads of the full configuration.  With one_thread, one unit is also
    timed on a single thread (the reference's default CPU build does not enable its thread pool)."""
    from oracle import cport
    cores = cport.max_threads()
    # probe with one unit per core, then size the timed sample (whole waves of units) to the budget
    c, arrs = cpu_sample(1, min(cores, CFG["nheads"]))
    t0 = time.perf_counter()
    cport.ssd2_serial(*arrs, None, c["chunk_len"], nthreads=cores)
    wave_s = time.perf_counter() - t0
    waves = int(max(1, min(budget_s / (wave_s * (steps + warmup)), CFG["batch"] * CFG["nheads"] / cores)))
    units = waves * min(cores, CFG["nheads"])
    heads = min(units, CFG["nheads"])
    batch = max(1, units // heads)
    c, arrs = cpu_sample(batch, heads)
    for _ in range(warmup):
        cport.ssd2_serial(*arrs, None, c["chunk_len"], nthreads=cores)
    t0 = time.perf_counter()
    for _ in range(steps):
        cport.ssd2_serial(*arrs, None, c["chunk_len"], nthreads=cores)
    dt = (time.perf_counter() - t0) / steps
    token_heads_per_s = c["batch"] * c["seqlen"] * c["nheads"] / dt
    out = {"value": token_heads_per_s / CFG["nheads"], "unit": UNIT, "cores": cores, "kind": "port",
           "seconds_per_step": dt,
           "sample": f"{c['batch']} x {c['nheads']} (batch x head) units of the {CFG['batch']} x {CFG['nheads']} "
                     f"configuration at full L={c['seqlen']}, float32, C restatement of ssd_serial "
                     f"(reference backend-flex unavailable: no Rust toolchain)"}
    if one_thread:
        c1, arrs1 = cpu_sample(1, 1)
        t0 = time.perf_counter()
        cport.ssd2_serial(*arrs1, None, c1["chunk_len"], nthreads=1)
        dt1 = time.perf_counter() - t0
        out["one_thread"] = {"value": c1["seqlen"] / dt1 / CFG["nheads"], "unit": UNIT, "cores": 1,
                             "sample": "1 (batch x head) unit at full L, one thread"}
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    steps, warmup = max(args.steps, 1), max(args.warmup, 0)
    base = cpu_baseline(budget_s=90.0, steps=min(steps, 3), warmup=min(warmup, 1))
    tokens = CFG["batch"] * CFG["seqlen"]
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": world, "steps": min(steps, 3),
        "warmup": min(warmup, 1), "ms_per_step": tokens / base["value"] * 1e3, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "problem": dict(CFG), "note": "CPU arm runs on rank 0's host cores only"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--regions", type=int, default=30, help="timed regions of --steps launches each (median reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=CFG["batch"],
                    help="batch rows of the problem (default: the benchmark configuration; smaller only for profiler captures)")
    ap.add_argument("--profile", action="store_true", help="kernel-only run for ncu: skips every other leg")
    ap.add_argument("--leg", default="all", choices=["all", "kernels", "decode"],
                    help="profiler captures: run only the other-kernels leg or only the decode leg (no prefill timing)")
    ap.add_argument("--small", action="store_true", help="with --leg: cut batch-like axes so that a full-metric ncu capture stays small")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.leg != "all":
        run_leg(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
