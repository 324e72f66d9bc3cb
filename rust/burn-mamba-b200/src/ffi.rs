//! `extern "C"` mirror of include/bm_b200.h, field by field.  All pointers are device pointers.
#![allow(non_camel_case_types)]
use std::ffi::{c_char, c_void};

pub const BM_OK: i32 = 0;
pub const BM_DTYPE_F32: i32 = 0;
pub const BM_DTYPE_BF16: i32 = 1;
pub const BM_PATH_AUTO: i32 = 0;
pub const BM_PATH_EXACT: i32 = 1;
pub const BM_PATH_TENSOR: i32 = 2;
pub const BM_PATH_TENSOR_SINGLE: i32 = 3;
pub const BM_PATH_TENSOR_PAIR: i32 = 4;

#[repr(C)]
pub struct BmSsd2FwdArgs {
    pub batch: i32, pub seqlen: i32, pub nheads: i32, pub headdim: i32, pub state_rank: i32,
    pub ngroups: i32, pub chunk_len: i32, pub dtype: i32, pub path: i32, pub reserved: i32,
    pub x: *const c_void, pub dt: *const f32, pub a: *const f32, pub b: *const c_void, pub c: *const c_void,
    pub d: *const f32, pub h0: *const f32, pub dt_bias: *const f32, pub dt_min: f32, pub dt_max: f32,
    pub z: *const c_void, pub y: *mut c_void, pub h_final: *mut f32, pub chunk_states: *mut f32,
}

#[repr(C)]
pub struct BmSsd2BwdArgs {
    pub batch: i32, pub seqlen: i32, pub nheads: i32, pub headdim: i32, pub state_rank: i32,
    pub ngroups: i32, pub chunk_len: i32, pub dtype: i32,
    pub x: *const c_void, pub dt: *const f32, pub a: *const f32, pub b: *const c_void, pub c: *const c_void,
    pub d: *const f32, pub h0: *const f32, pub dy: *const c_void, pub dh_final: *const f32,
    pub dx: *mut f32, pub ddt: *mut f32, pub da: *mut f32, pub db: *mut f32, pub dc: *mut f32, pub dd: *mut f32,
    pub dh0: *mut f32,
    pub path: i32, pub reserved: i32,
}

#[repr(C)]
pub struct BmSsd3FwdArgs {
    pub batch: i32, pub seqlen: i32, pub nheads: i32, pub headdim: i32, pub state_rank: i32,
    pub mimo_rank: i32, pub chunk_len: i32, pub dtype: i32, pub path: i32, pub rope_dim: i32,
    pub v: *const c_void, pub da: *const f32, pub b: *const c_void, pub c: *const c_void,
    pub gamma: *const f32, pub scale: *const f32, pub h0: *const f32, pub angles: *const f32,
    pub y: *mut c_void, pub h_final: *mut f32,
}

#[repr(C)]
pub struct BmSsd3BwdArgs {
    pub batch: i32, pub seqlen: i32, pub nheads: i32, pub headdim: i32, pub state_rank: i32,
    pub mimo_rank: i32, pub chunk_len: i32, pub dtype: i32,
    pub v: *const c_void, pub da: *const f32, pub b: *const c_void, pub c: *const c_void,
    pub gamma: *const f32, pub scale: *const f32, pub h0: *const f32, pub dy: *const c_void,
    pub dh_final: *const f32, pub dv: *mut f32, pub dda: *mut f32, pub db: *mut f32, pub dc: *mut f32,
    pub dgamma: *mut f32, pub dscale: *mut f32, pub dh0: *mut f32,
    pub path: i32, pub reserved: i32,
}

#[repr(C)]
pub struct BmStep2Args {
    pub batch: i32, pub nheads: i32, pub headdim: i32, pub state_rank: i32, pub ngroups: i32, pub dtype: i32,
    pub state: *mut f32, pub x: *const c_void, pub dt: *const f32, pub a: *const f32, pub b: *const c_void,
    pub c: *const c_void, pub d: *const f32, pub dt_bias: *const f32, pub dt_min: f32, pub dt_max: f32,
    pub z: *const c_void, pub y: *mut c_void,
}

#[repr(C)]
pub struct BmConvStepArgs {
    pub batch: i32, pub channels: i32, pub kernel: i32, pub dtype: i32,
    pub window: *mut f32, pub xin: *const c_void, pub weight: *const f32, pub bias: *const f32, pub out: *mut c_void,
    pub out_b: *mut c_void, pub out_c: *mut c_void,
    pub xin_stride: i32, pub split_x: i32, pub split_bc: i32, pub reserved: i32,
}

#[repr(C)]
pub struct BmConv1dSiluArgs {
    pub batch: i32, pub seqlen: i32, pub channels: i32, pub kernel: i32, pub dtype: i32, pub xin_stride: i32,
    pub split_x: i32, pub split_bc: i32,
    pub xin: *const c_void, pub weight: *const f32, pub bias: *const f32, pub window: *const f32,
    pub new_window: *mut f32, pub out_x: *mut c_void, pub out_b: *mut c_void, pub out_c: *mut c_void,
}

#[repr(C)]
pub struct BmRmsnormGatedArgs {
    pub rows: i32, pub width: i32, pub dtype: i32, pub norm_before_gate: i32, pub x_stride: i32, pub z_stride: i32,
    pub eps: f32,
    pub x: *const c_void, pub z: *const c_void, pub gamma: *const c_void, pub out: *mut c_void,
}

#[repr(C)]
pub struct BmMamba3BcPrepArgs {
    pub batch: i32, pub seqlen: i32, pub mimo_rank: i32, pub ngroups: i32, pub nheads: i32, pub state_rank: i32,
    pub dtype: i32, pub raw_stride: i32, pub rope_dim: i32, pub pairwise: i32, pub eps: f32, pub reserved: i32,
    pub b_raw: *const c_void, pub c_raw: *const c_void, pub b_gamma: *const f32, pub c_gamma: *const f32,
    pub b_bias: *const f32, pub c_bias: *const f32, pub angles: *const f32, pub b_out: *mut c_void, pub c_out: *mut c_void,
}

#[repr(C)]
pub struct BmSelscan1Args {
    pub batch: i32, pub seqlen: i32, pub d_inner: i32, pub state_rank: i32, pub dtype: i32, pub delta_softplus: i32,
    pub u: *const c_void, pub delta: *const c_void, pub a: *const f32, pub b: *const c_void, pub c: *const c_void,
    pub d: *const f32, pub delta_bias: *const f32, pub z: *const c_void, pub h0: *const f32,
    pub y: *mut c_void, pub h_final: *mut f32,
}

#[repr(C)]
pub struct BmStep1Args {
    pub batch: i32, pub d_inner: i32, pub state_rank: i32, pub dtype: i32, pub delta_softplus: i32,
    pub state: *mut f32, pub u: *const c_void, pub delta: *const c_void, pub a: *const f32, pub b: *const c_void,
    pub c: *const c_void, pub d: *const f32, pub delta_bias: *const f32, pub z: *const c_void, pub y: *mut c_void,
}

#[repr(C)]
pub struct BmAngleCumsumArgs {
    pub batch: i32, pub seqlen: i32, pub nheads: i32, pub nangles: i32, pub range: f32,
    pub rot: *const f32, pub dt: *const f32, pub prev: *const f32, pub theta: *mut f32, pub last: *mut f32,
}

#[repr(C)]
pub struct BmStep3Args {
    pub batch: i32, pub nheads: i32, pub headdim: i32, pub state_rank: i32, pub mimo_rank: i32, pub rope_dim: i32,
    pub range: f32,
    pub state: *mut f32, pub k_state: *mut f32, pub v_state: *mut f32, pub angle: *mut f32, pub x: *const f32,
    pub b: *const f32, pub c: *const f32, pub rot: *const f32, pub dt: *const f32, pub alpha: *const f32,
    pub beta: *const f32, pub gamma: *const f32, pub mimo_x: *const f32, pub y: *mut f32,
}

extern "C" {
    pub fn bm_version() -> i32;
    pub fn bm_last_error_string() -> *const c_char;
    pub fn bm_ssd2_fwd_workspace_bytes(args: *const BmSsd2FwdArgs) -> usize;
    pub fn bm_ssd2_fwd(args: *const BmSsd2FwdArgs, ws: *mut c_void, ws_bytes: usize, stream: *mut c_void) -> i32;
    pub fn bm_ssd2_fwd_noalloc(args: *const BmSsd2FwdArgs, stream: *mut c_void) -> i32;
    pub fn bm_workspace_status(ws: *const c_void, stream: *mut c_void) -> i32;
    pub fn bm_ssd2_bwd_workspace_bytes(args: *const BmSsd2BwdArgs) -> usize;
    pub fn bm_ssd2_bwd(args: *const BmSsd2BwdArgs, ws: *mut c_void, ws_bytes: usize, stream: *mut c_void) -> i32;
    pub fn bm_ssd3_fwd_workspace_bytes(args: *const BmSsd3FwdArgs) -> usize;
    pub fn bm_ssd3_single_fwd(args: *const BmSsd3FwdArgs, ws: *mut c_void, ws_bytes: usize, stream: *mut c_void) -> i32;
    pub fn bm_ssd3_double_fwd(args: *const BmSsd3FwdArgs, ws: *mut c_void, ws_bytes: usize, stream: *mut c_void) -> i32;
    pub fn bm_ssd3_bwd_workspace_bytes(args: *const BmSsd3BwdArgs) -> usize;
    pub fn bm_ssd3_single_bwd(args: *const BmSsd3BwdArgs, ws: *mut c_void, ws_bytes: usize, stream: *mut c_void) -> i32;
    pub fn bm_ssd3_double_bwd(args: *const BmSsd3BwdArgs, ws: *mut c_void, ws_bytes: usize, stream: *mut c_void) -> i32;
    pub fn bm_step2(args: *const BmStep2Args, stream: *mut c_void) -> i32;
    pub fn bm_conv_step(args: *const BmConvStepArgs, stream: *mut c_void) -> i32;
    pub fn bm_conv1d_silu_fwd(args: *const BmConv1dSiluArgs, stream: *mut c_void) -> i32;
    pub fn bm_rmsnorm_gated(args: *const BmRmsnormGatedArgs, stream: *mut c_void) -> i32;
    pub fn bm_mamba3_bc_prep(args: *const BmMamba3BcPrepArgs, stream: *mut c_void) -> i32;
    pub fn bm_selscan1_fwd(args: *const BmSelscan1Args, stream: *mut c_void) -> i32;
    pub fn bm_selscan1_fwd_workspace_bytes(args: *const BmSelscan1Args) -> usize;
    pub fn bm_selscan1_fwd_ws(args: *const BmSelscan1Args, ws: *mut c_void, ws_bytes: usize, stream: *mut c_void) -> i32;
    pub fn bm_step1(args: *const BmStep1Args, stream: *mut c_void) -> i32;
    pub fn bm_angle_cumsum(args: *const BmAngleCumsumArgs, stream: *mut c_void) -> i32;
    pub fn bm_step3(args: *const BmStep3Args, stream: *mut c_void) -> i32;
}
