"""Host-side mirror of the reference's Mamba-2 interface around the SSD slot.

Names, argument meaning and error behaviour follow the reference so that tests read like its own:
`Mamba2SsdPath` (src/mamba2/ssd/ssd_path.rs:20-53), `Mamba2SsdInput.run` (:58-87, :149-155),
`Mamba2Cache` (src/mamba2/cache.rs:98-122), `Mamba2.forward` / `Mamba2.step`
(src/mamba2/mamba2.rs:546-786, :820-1004).  The SSM core (SSD, conv-window step, state step) runs in
libbm_b200; the prefill convolution (+ SiLU, split into x / B / C) and the gated norm around it run in libbm_b200 as well
(bm_conv1d_silu_fwd, bm_rmsnorm_gated); the two projections are library GEMMs (torch).
"""
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from . import ops


@dataclass(frozen=True)
class Mamba2SsdPath:
    """Which exact SSD algorithm the reference would run and with which chunk length.  All three
    variants are the same function (the reference tests assert it, src/mamba2/ssd/ssd_path/tests.rs:184-336);
    here they all dispatch to bm_ssd2_fwd and only the chunk length matters."""
    kind: str = "SerialRecalculated"
    chunk_len: Optional[int] = None

    @staticmethod
    def minimal(chunk_len=None):
        return Mamba2SsdPath("Minimal", chunk_len)

    @staticmethod
    def serial(chunk_len=None):
        return Mamba2SsdPath("Serial", chunk_len)

    @staticmethod
    def serial_recalculated(chunk_len=None):
        return Mamba2SsdPath("SerialRecalculated", chunk_len)

    @staticmethod
    def optimal_chunk_len(state_rank, per_head_dim):
        """ceil32(isqrt(N * P)) capped at 512 (src/mamba2/ssd/ssd_path.rs:109-114)."""
        import math
        return min(((math.isqrt(state_rank * per_head_dim) + 31) // 32) * 32, 512)

    def chunk_len_or_optimal(self, state_rank, per_head_dim):
        return self.chunk_len if self.chunk_len is not None else self.optimal_chunk_len(state_rank, per_head_dim)


@dataclass
class Mamba2SsdInput:
    """The slot's input bundle (src/mamba2/ssd/ssd_path.rs:58-87) in the chunked layout of the reference:
    x [b,n,l,h,p], dt [b,n,l,h], a_decay [h], b / c [b,n,l,g,r] (groups, or g = h when already expanded),
    d [h], initial_state [b,h,p,r]."""
    x_bnlhp: torch.Tensor
    dt_bnlh: torch.Tensor
    a_decay_h: torch.Tensor
    b_bnlgr: torch.Tensor
    c_bnlgr: torch.Tensor
    d_h: torch.Tensor
    initial_state_bhpr: torch.Tensor
    init_state_hpr: Optional[torch.Tensor] = None

    def run(self, path: Mamba2SsdPath, kernel_path="auto"):
        """-> (y_bnlhp, final_state_bhpr).  Like the reference's Serial / SerialRecalculated variants
        (src/mamba2/ssd/serial.rs:48-51, serial_recalculated.rs:41-44) a learnable init_state_hpr is only
        accepted by the Minimal variant, where it is added to the initial state (minimal.rs:317-328)."""
        b, n, l, h, p = self.x_bnlhp.shape
        if n < 1:
            raise AssertionError("sequence length must be at least 1")
        h0 = self.initial_state_bhpr
        if self.init_state_hpr is not None:
            if path.kind != "Minimal":
                raise AssertionError("init_state_hpr is not supported by the serial SSD variants; use Minimal")
            h0 = h0 + self.init_state_hpr.unsqueeze(0)
        g, r = self.b_bnlgr.shape[3], self.b_bnlgr.shape[4]
        y, hf = ops.ssd2_fwd(self.x_bnlhp.reshape(b, n * l, h, p), self.dt_bnlh.reshape(b, n * l, h).float(),
                             self.a_decay_h.float(), self.b_bnlgr.reshape(b, n * l, g, r),
                             self.c_bnlgr.reshape(b, n * l, g, r), self.d_h.float(), h0.float(), chunk_len=l,
                             path=kernel_path)
        return y.reshape(b, n, l, h, p), hf


@dataclass
class Mamba2Cache:
    """conv window [b, v, k] (raw pre-conv columns, newest last) and SSM state [b, h, p, r]
    (src/mamba2/cache.rs:98-122); both float32."""
    conv_bvk: torch.Tensor
    ssm_bhpr: torch.Tensor


DIV_EPS = {torch.float32: 8.1584695e-8, torch.bfloat16: 2.0885676e-5}   # src/utils/mod.rs:50-95


class Mamba2:
    """One Mamba-2 block with the reference's parameter set (src/mamba2/mamba2.rs:408-490).  Weights are
    plain tensors: w_in [d_model, d_inner + conv_dim + h], conv_w [conv_dim, k], conv_b [conv_dim],
    dt_bias [h], a_log [h], d [h], norm_gamma [d_inner], w_out [d_inner, d_model]."""

    def __init__(self, w_in, conv_w, conv_b, dt_bias, a_log, d, norm_gamma, w_out, nheads, state_rank, ngroups=1,
                 dt_limit=(0.0, 65504.0), norm_before_gate=False):
        self.w_in, self.conv_w, self.conv_b, self.w_out = w_in, conv_w, conv_b, w_out
        self.dt_bias, self.a_log, self.d, self.norm_gamma = dt_bias.float(), a_log.float(), d.float(), norm_gamma
        self.nheads, self.state_rank, self.ngroups = nheads, state_rank, ngroups
        self.d_inner = norm_gamma.shape[0]
        self.per_head_dim = self.d_inner // nheads
        self.conv_dim, self.conv_kernel = conv_w.shape
        self.dt_limit, self.norm_before_gate = dt_limit, norm_before_gate
        self._conv_w32, self._conv_b32 = conv_w.float().contiguous(), conv_b.float().contiguous()
        self._a = -torch.exp(self.a_log)
        assert self.conv_dim == self.d_inner + 2 * ngroups * state_rank
        assert nheads % ngroups == 0

    def zero_cache(self, batch):
        dev = self.w_in.device
        return Mamba2Cache(torch.zeros((batch, self.conv_dim, self.conv_kernel), device=dev),
                           torch.zeros((batch, self.nheads, self.per_head_dim, self.state_rank), device=dev))

    def _gated_norm(self, y, z):
        """RmsNormGated (src/modules/norm/rms_norm_gated.rs:70-135): one kernel, z read in place from the
        projection's columns."""
        return ops.rmsnorm_gated(y, z, self.norm_gamma.to(y.dtype), norm_before_gate=self.norm_before_gate)

    def forward(self, input_bsm, cache: Optional[Mamba2Cache] = None, ssd_path: Mamba2SsdPath = Mamba2SsdPath(),
                kernel_path="auto"):
        """Mamba2::forward (src/mamba2/mamba2.rs:546-786) -> (out_bsm, cache)."""
        bsz, s, _ = input_bsm.shape
        if s < 1:
            raise AssertionError("sequence length must be at least 1")
        cache = cache or self.zero_cache(bsz)
        act = input_bsm.dtype
        proj = input_bsm @ self.w_in
        z, xbc, dt_raw = torch.split(proj, [self.d_inner, self.conv_dim, self.nheads], dim=2)
        # window slide + causal depthwise conv + bias + SiLU in one kernel, reading xbc in place from the
        # projection's columns and writing x, B, C as the three dense tensors the SSD takes
        gr = self.ngroups * self.state_rank
        (x, bm, cm), new_conv = ops.conv1d_silu_fwd(xbc, self._conv_w32, self._conv_b32, cache.conv_bvk,
                                                    splits=(self.d_inner, gr, gr))
        x = x.view(bsz, s, self.nheads, self.per_head_dim)
        bm = bm.view(bsz, s, self.ngroups, self.state_rank)
        cm = cm.view(bsz, s, self.ngroups, self.state_rank)
        a = self._a
        chunk_len = ssd_path.chunk_len_or_optimal(self.state_rank, self.per_head_dim)
        # softplus(dt_raw + dt_bias) and the clamp are fused into the SSD's decay scan; the tail chunk is
        # handled inside the kernel (dt = 0 padding semantics), so no explicit pad / unpad here
        y, hf = ops.ssd2_fwd(x, dt_raw.float().contiguous(), a, bm, cm, self.d, cache.ssm_bhpr, chunk_len=chunk_len,
                             path=kernel_path, dt_bias=self.dt_bias, dt_limit=self.dt_limit)
        out = self._gated_norm(y.reshape(bsz, s, self.d_inner), z) @ self.w_out
        return out, Mamba2Cache(new_conv, hf)

    def step(self, input_bm, cache: Optional[Mamba2Cache] = None, residual=None):
        """Mamba2::step (src/mamba2/mamba2.rs:820-1004) -> (out_bm, cache).  The cache tensors are updated
        in place by the kernels and returned.  `residual` (the layer's skip connection) is added to the output
        inside the out-projection GEMM when given."""
        bsz = input_bm.shape[0]
        cache = cache or self.zero_cache(bsz)
        proj = input_bm @ self.w_in
        z, xbc, dt_raw = torch.split(proj, [self.d_inner, self.conv_dim, self.nheads], dim=1)
        # window slide + conv + SiLU, reading xbc in place and writing x / B / C as the step's three dense inputs
        gr = self.ngroups * self.state_rank
        x, bm, cm = ops.conv_step(cache.conv_bvk, xbc, self._conv_w32, self._conv_b32, splits=(self.d_inner, gr, gr))
        y = ops.step2(cache.ssm_bhpr, x.view(bsz, self.nheads, self.per_head_dim), dt_raw.float().contiguous(), self._a,
                      bm.view(bsz, self.ngroups, self.state_rank), cm.view(bsz, self.ngroups, self.state_rank), self.d,
                      dt_bias=self.dt_bias, dt_limit=self.dt_limit)
        g = self._gated_norm(y.reshape(bsz, self.d_inner), z)
        out = g @ self.w_out if residual is None else torch.addmm(residual, g, self.w_out)
        return out, cache


def rms_norm(x, gamma):
    """RmsNorm (src/modules/norm/rms_norm.rs:53-98): x / sqrt(mean(x^2) + eps) * gamma, one kernel."""
    return ops.rmsnorm_gated(x, None, gamma.to(x.dtype))


def stack_step(blocks, norm_gammas, caches, x_bm):
    """One decode step through a stack of pre-norm residual layers, the default (no class latents, plain
    residual) path of Layers::step / Layer::step_one (src/modules/layers.rs:427-497,
    src/modules/layer.rs:224-229): x <- x + block.step(norm(x)).  `caches` is one Mamba2Cache per layer,
    updated in place.  Returns the output of the last layer [b, d_model].  Per layer this is seven launches
    (norm, in-projection, conv step, state step, gated norm, out-projection with the residual folded in as the
    GEMM's addend, plus the dt cast); none of them depends on the host, so the whole step can be replayed from a
    CUDA graph."""
    for blk, gamma, cache in zip(blocks, norm_gammas, caches):
        x_bm = blk.step(rms_norm(x_bm, gamma), cache, residual=x_bm)[0]
    return x_bm
