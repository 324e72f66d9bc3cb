"""Block-level GPU parity through the reference-shaped host interface (Mamba2.forward / step,
Mamba2SsdInput.run, Mamba3.forward_single_ssd / forward_double_ssd / step_double_ssd): the CPU-runnable
benchmark configuration and the forward == step property."""
import numpy as np
import pytest
import torch

from oracle import mamba2 as o2
from oracle import mamba3 as o3
from oracle.numerics import rel_l2, bf16_round

pytestmark = pytest.mark.gpu


def _block(bm, w, dtype=torch.float32):
    t = lambda a, dt=None: torch.from_numpy(np.ascontiguousarray(a)).cuda().to(dt or torch.float32)
    return bm.Mamba2(t(w.w_in, dtype), t(w.conv_w), t(w.conv_b), t(w.dt_bias), t(w.a_log), t(w.d), t(w.norm_gamma, dtype),
                     t(w.w_out, dtype), nheads=w.nheads, state_rank=w.state_rank, ngroups=w.ngroups)


def test_cpu_runnable_configuration_block_forward_fp32(bm):
    """'Mamba-2 single SSM block forward, fp32, seed 0': d_model 256, d_inner 512, P 64 (H 8), N 64, G 1, Q 64,
    batch 2, L 512; compare output (2,512,256) and final SSM state (2,8,64,64) at rel-L2 <= 1e-4."""
    rng = np.random.Generator(np.random.PCG64(0))
    w = o2.Mamba2Weights(rng, d_model=256, d_inner=512, nheads=8, state_rank=64, ngroups=1, dtype=np.float32)
    u = rng.standard_normal((2, 512, 256), dtype=np.float32)
    conv0 = np.zeros((2, w.conv_dim, 4), np.float32)
    ssm0 = np.zeros((2, 8, 64, 64), np.float32)
    want_out, want_conv, want_state, pre = o2.block_forward(w, u.astype(np.float64), conv0.astype(np.float64),
                                                            ssm0.astype(np.float64), chunk_len=64, dtype_name="f32")
    blk = _block(bm, w)
    out, cache = blk.forward(torch.from_numpy(u).cuda(), None, bm.Mamba2SsdPath.serial_recalculated(64), kernel_path="exact")
    assert rel_l2(out.cpu().numpy(), want_out) <= 1e-4
    assert rel_l2(cache.ssm_bhpr.cpu().numpy(), want_state) <= 1e-4
    assert rel_l2(cache.conv_bvk.cpu().numpy(), want_conv) <= 1e-5
    # the slot alone, fed the oracle's pre-SSD tensors through the reference-shaped input bundle
    f = lambda a: torch.from_numpy(np.ascontiguousarray(a.astype(np.float32))).cuda()
    inp = bm.Mamba2SsdInput(f(pre["x"]).reshape(2, 8, 64, 8, 64), f(pre["dt"]).reshape(2, 8, 64, 8), f(pre["a"]),
                            f(pre["b"]).reshape(2, 8, 64, 1, 64), f(pre["c"]).reshape(2, 8, 64, 1, 64), f(w.d),
                            f(ssm0))
    y, hf = inp.run(bm.Mamba2SsdPath.serial_recalculated(64), kernel_path="exact")
    assert rel_l2(y.reshape(2, 512, 8, 64).cpu().numpy(), pre["y"]) <= 1e-4
    assert rel_l2(hf.cpu().numpy(), want_state) <= 1e-4
    with pytest.raises(AssertionError):   # serial variants reject a learnable init state (serial.rs:48-51)
        inp.init_state_hpr = f(np.zeros((8, 64, 64)))
        inp.run(bm.Mamba2SsdPath.serial(64))


@pytest.mark.parametrize("g", [1, 2])
def test_block_forward_equals_unrolled_step_and_split(bm, g):
    """forward == unrolled step on output, conv window and SSM state (src/mamba2/mamba2/tests.rs:202-252, tolerance
    1e-4 max-abs), split == full (:343-392), with a random initial cache (:290-328), CUDA vs CUDA."""
    rng = np.random.Generator(np.random.PCG64(5))
    w = o2.Mamba2Weights(rng, d_model=32, d_inner=64, nheads=4, state_rank=16, ngroups=g, dtype=np.float32)
    blk = _block(bm, w)
    bsz, s = 2, 21
    u = torch.from_numpy(rng.standard_normal((bsz, s, 32), dtype=np.float32)).cuda()
    c0 = bm.Mamba2Cache(0.1 * torch.randn(bsz, w.conv_dim, 4, device="cuda"), 0.1 * torch.randn(bsz, 4, 16, 16, device="cuda"))
    clone = lambda c: bm.Mamba2Cache(c.conv_bvk.clone(), c.ssm_bhpr.clone())
    out, cache = blk.forward(u, clone(c0), bm.Mamba2SsdPath.serial_recalculated(8), kernel_path="exact")
    c = clone(c0)
    for t in range(s):
        o, c = blk.step(u[:, t].contiguous(), c)
        assert torch.max(torch.abs(o - out[:, t])).item() <= 1e-4
    assert torch.max(torch.abs(c.ssm_bhpr - cache.ssm_bhpr)).item() <= 1e-4
    assert torch.max(torch.abs(c.conv_bvk - cache.conv_bvk)).item() <= 1e-5
    o1, c1 = blk.forward(u[:, :9].contiguous(), clone(c0), bm.Mamba2SsdPath.serial_recalculated(8), kernel_path="exact")
    o2_, c2 = blk.forward(u[:, 9:].contiguous(), c1, bm.Mamba2SsdPath.serial_recalculated(8), kernel_path="exact")
    assert torch.max(torch.abs(torch.cat([o1, o2_], 1) - out)).item() <= 1e-4
    assert torch.max(torch.abs(c2.ssm_bhpr - cache.ssm_bhpr)).item() <= 1e-4


def test_decode_prefix_equals_forward_at_the_2_7b_head_shape(bm):
    """'Mamba-2 recurrent step() decode ... check the outputs equal the matching positions of forward() on the same
    128-token prefix' -- one layer at the 2.7B head shape (P 64, N 128) with a reduced width (H 8, batch 4) so the
    test stays small; bf16 activations, tensor-core prefill vs step kernels, initial cache ~ N(0, 0.1)."""
    rng = np.random.Generator(np.random.PCG64(3))
    w = o2.Mamba2Weights(rng, d_model=256, d_inner=512, nheads=8, state_rank=128, ngroups=1, dtype=np.float32)
    blk = _block(bm, w, torch.bfloat16)
    bsz, s = 4, 128
    u = torch.from_numpy(rng.standard_normal((bsz, s, 256), dtype=np.float32)).cuda().to(torch.bfloat16)
    c0 = bm.Mamba2Cache(0.1 * torch.randn(bsz, w.conv_dim, 4, device="cuda"), 0.1 * torch.randn(bsz, 8, 64, 128, device="cuda"))
    clone = lambda c: bm.Mamba2Cache(c.conv_bvk.clone(), c.ssm_bhpr.clone())
    out, cache = blk.forward(u, clone(c0), bm.Mamba2SsdPath.serial_recalculated(256), kernel_path="tensor")
    c = clone(c0)
    steps = []
    for t in range(s):
        o, c = blk.step(u[:, t].contiguous(), c)
        steps.append(o)
    got = torch.stack(steps, 1)
    assert rel_l2(got.float().cpu().numpy(), out.float().cpu().numpy()) <= 2e-2
    assert rel_l2(c.ssm_bhpr.cpu().numpy(), cache.ssm_bhpr.cpu().numpy()) <= 2e-2


# ------------------------------------------------------------------ Mamba-3 block
def _m3_cache(rng, w, bsz, scale=0.1):
    c = o3.zero_cache(w, bsz)
    return {k: (scale * rng.standard_normal(v.shape)).astype(np.float32) for k, v in c.items()}


def _to_dev(cache):
    return {k: torch.from_numpy(np.ascontiguousarray(v)).cuda() for k, v in cache.items()}


@pytest.mark.parametrize("m,g,frac", [(1, 1, 1.0), (2, 1, 1.0), (4, 2, 0.5)])
def test_mamba3_block_forward_matches_oracle(bm, m, g, frac):
    """Both prefill pathways of the block against the oracle's float64 block (which itself holds
    single == double == recurrence, tests/test_oracle_invariants.py) from a random cache: output and all
    four cache tensors."""
    rng = np.random.Generator(np.random.PCG64(11 + m))
    w = o3.Mamba3Weights(rng, d_model=48, d_inner=64, nheads=4, state_rank=16, ngroups=g, mimo_rank=m,
                         rope_fraction=frac)
    bsz, s = 2, 37
    u = rng.standard_normal((bsz, s, 48)).astype(np.float32)
    c0 = _m3_cache(rng, w, bsz)
    c64 = {k: v.astype(np.float64) for k, v in c0.items()}
    want_out, want_cache, _ = o3.block_forward_single(w, u.astype(np.float64), c64, chunk_len=8)
    blk = bm.Mamba3.from_oracle_weights(w, "cuda")
    for fwd in (blk.forward_single_ssd, blk.forward_double_ssd):
        out, cache = fwd(torch.from_numpy(u).cuda(), _to_dev(c0), chunk_len=8)
        assert rel_l2(out.cpu().numpy(), want_out) <= 1e-4, fwd.__name__
        for k in ("ssm", "k", "v"):
            assert rel_l2(cache[k].cpu().numpy(), want_cache[k]) <= 1e-4, (fwd.__name__, k)
        assert np.abs(cache["angle"].cpu().numpy() - want_cache["angle"]).max() <= 1e-4


@pytest.mark.parametrize("m", [1, 4])
def test_mamba3_block_forward_equals_unrolled_step(bm, m):
    """forward == unrolled step_double_ssd on the output and the cache, CUDA vs CUDA
    (the property the reference asserts for its block, src/mamba3/mamba3/tests.rs)."""
    rng = np.random.Generator(np.random.PCG64(21 + m))
    w = o3.Mamba3Weights(rng, d_model=32, d_inner=64, nheads=4, state_rank=16, ngroups=1, mimo_rank=m)
    blk = bm.Mamba3.from_oracle_weights(w, "cuda")
    bsz, s = 2, 19
    u = torch.from_numpy(rng.standard_normal((bsz, s, 32)).astype(np.float32)).cuda()
    c0 = _m3_cache(rng, w, bsz)
    out, cache = blk.forward_double_ssd(u, _to_dev(c0), chunk_len=8)
    c = _to_dev(c0)
    outs = []
    for t in range(s):
        o, c = blk.step_double_ssd(u[:, t].contiguous(), c)
        outs.append(o)
    stepped = torch.stack(outs, dim=1)
    assert (out - stepped).abs().max().item() <= 1e-4
    for k in ("ssm", "k", "v"):
        assert rel_l2(cache[k].cpu().numpy(), c[k].cpu().numpy()) <= 1e-4, k
    assert (cache["angle"] - c["angle"]).abs().max().item() <= 1e-4


# ------------------------------------------------------------------ pre- / post-SSD kernels of the block
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("b,s,k", [(2, 70, 4), (1, 3, 4), (2, 33, 2), (1, 1, 4)])
def test_conv1d_silu_prefill_matches_window_slide_and_conv(bm, dtype, b, s, k):
    """Causal depthwise conv + bias + SiLU over a sequence with the cache window as left context
    (src/mamba2/mamba2.rs:618-654), input read in place from a column slice, outputs split into x / B / C."""
    from oracle.numerics import silu
    rng = np.random.default_rng(5)
    v, sx, sbc = 48, 32, 8
    wide = rng.standard_normal((b, s, 16 + v + 8)).astype(np.float32)     # xbc sits in the middle of a wider row
    win = rng.standard_normal((b, v, k)).astype(np.float32)
    w = rng.standard_normal((v, k)).astype(np.float32)
    bias = rng.standard_normal(v).astype(np.float32)
    wide_t = torch.from_numpy(wide).cuda().to(dtype)
    xin = wide_t.float().cpu().numpy()[:, :, 16:16 + v]
    padded = np.concatenate([win[:, :, 1:], xin.transpose(0, 2, 1)], axis=2)           # b v (k-1+s)
    want = np.stack([(padded[:, :, t:t + k] * w[None]).sum(-1) + bias[None] for t in range(s)], axis=1)
    want = silu(want)
    (x, bb, cc), new_win = bm.ops.conv1d_silu_fwd(wide_t[:, :, 16:16 + v], torch.from_numpy(w).cuda(),
                                                  torch.from_numpy(bias).cuda(), torch.from_numpy(win).cuda(),
                                                  splits=(sx, sbc, sbc))
    got = torch.cat([x, bb, cc], dim=2).float().cpu().numpy()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert rel_l2(got, want) <= tol
    assert np.array_equal(new_win.cpu().numpy(), padded[:, :, s - 1:].astype(np.float32))
    whole, _ = bm.ops.conv1d_silu_fwd(wide_t[:, :, 16:16 + v], torch.from_numpy(w).cuda(), torch.from_numpy(bias).cuda(),
                                      None, want_window=False)
    padded0 = np.concatenate([np.zeros((b, v, k - 1), np.float32), xin.transpose(0, 2, 1)], axis=2)
    want0 = silu(np.stack([(padded0[:, :, t:t + k] * w[None]).sum(-1) + bias[None] for t in range(s)], axis=1))
    assert rel_l2(whole.float().cpu().numpy(), want0) <= tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("norm_before_gate", [False, True])
def test_rmsnorm_gated_matches_oracle(bm, dtype, norm_before_gate):
    """RmsNormGated (src/modules/norm/rms_norm_gated.rs:70-135) and the plain RmsNorm (z = None), with z read
    in place from a column slice of a wider row."""
    from oracle.numerics import rms_norm, rms_norm_gated
    rng = np.random.default_rng(6)
    rows, d = 37, 5120
    x = rng.standard_normal((rows, d)).astype(np.float32)
    wide = rng.standard_normal((rows, d + 264)).astype(np.float32)
    gamma = rng.standard_normal(d).astype(np.float32)
    xt, wt, gt = (torch.from_numpy(t).cuda().to(dtype) for t in (x, wide, gamma))
    xq, zq, gq = xt.float().cpu().numpy(), wt.float().cpu().numpy()[:, 8:8 + d], gt.float().cpu().numpy()
    name = "f32" if dtype == torch.float32 else "bf16"
    want = rms_norm_gated(xq.astype(np.float64), zq.astype(np.float64), gq.astype(np.float64), norm_before_gate, name)
    got = bm.ops.rmsnorm_gated(xt, wt[:, 8:8 + d], gt, norm_before_gate=norm_before_gate)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert rel_l2(got.float().cpu().numpy(), want) <= tol
    plain = bm.ops.rmsnorm_gated(xt.reshape(1, rows, d), None, gt)
    assert rel_l2(plain.float().cpu().numpy()[0], rms_norm(xq.astype(np.float64), gq.astype(np.float64), name)) <= tol


# ------------------------------------------------------------------ Mamba-3 B / C preparation (norm, expand, bias, rotation)
@pytest.mark.parametrize("dtype,m,g,h,r,rope", [
    ("f32", 1, 1, 4, 32, 32),      # pairwise rotation (MIMO rank 1)
    ("f32", 4, 2, 6, 64, 32),      # halves, partial rotation, two groups
    ("bf16", 4, 1, 32, 128, 128),  # the configured head shape
    ("bf16", 2, 1, 8, 128, 0),     # no rotation
])
def test_mamba3_bc_prep_matches_norm_expand_bias_and_rotation(bm, dtype, m, g, h, r, rope):
    """One kernel against the oracle's chain qk_norm_expand_bias -> apply_rope_partial (src/mamba3/helpers.rs:82-95,
    src/modules/misc/rope.rs:50-170), with the raw rows taken as column slices of a wider projection output."""
    rng = np.random.default_rng(91)
    b, s = 2, 37
    tdt = torch.float32 if dtype == "f32" else torch.bfloat16
    width = 2 * m * g * r + 24
    proj = rng.standard_normal((b, s, width)).astype(np.float32)
    if dtype == "bf16":
        proj = bf16_round(proj)
    braw, craw = proj[..., 8:8 + m * g * r], proj[..., 8 + m * g * r:8 + 2 * m * g * r]
    gam = [1.0 + 0.1 * rng.standard_normal(r).astype(np.float32) for _ in range(2)]
    bias = [0.3 * rng.standard_normal((h, m, r)).astype(np.float32) for _ in range(2)]
    ang = (3.0 * rng.standard_normal((b, s, h, max(rope // 2, 1)))).astype(np.float32) if rope else None
    want = []
    for raw, gm, bi in ((braw, gam[0], bias[0]), (craw, gam[1], bias[1])):
        t = o3.qk_norm_expand_bias(raw.reshape(b, s, m, g, r), gm, bi, h, dtype)
        want.append(o3.apply_rope_partial(t, ang[:, :, None], rope, m == 1) if rope else t)
    pd = torch.as_tensor(proj).cuda().to(tdt)
    dev = lambda a: None if a is None else torch.as_tensor(a).cuda()
    got = bm.ops.mamba3_bc_prep(pd[..., 8:8 + m * g * r], pd[..., 8 + m * g * r:8 + 2 * m * g * r], dev(gam[0]), dev(gam[1]),
                                dev(bias[0]), dev(bias[1]), angles=dev(ang), rope_dim=rope, pairwise=m == 1, ngroups=g)
    tol = 1e-5 if dtype == "f32" else 6e-3
    for gt, wt in zip(got, want):
        assert gt.shape == (b, s, m, h, r)
        assert rel_l2(gt.float().cpu().numpy(), wt) <= tol, rel_l2(gt.float().cpu().numpy(), wt)
