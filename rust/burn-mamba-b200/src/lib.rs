//! B200 backend type for burn-mamba: the three SSD extension traits implemented by calls into libbm_b200.
//!
//! burn-mamba opts every Burn backend into the default (Burn-op) body of its extension traits with empty
//! `impl` blocks, including a blanket `impl<R: CubeRuntime> … for CubeBackend<R>`
//! (src/utils/backend_macros.rs:14-35).  A newtype backend `B200` over `CubeBackend<CudaRuntime>` is therefore
//! what carries the overriding impls; every other `Backend` item is forwarded to the inner backend
//! (the forwarding impl is mechanical and omitted from this file: `burn::backend_newtype!`-style delegation).
//!
//! What a raw-pointer accessor needs from Burn (`device_ptr`, `stream`, `alloc_like` below) lives in
//! burn-cubecl / cubecl-cuda, which are not vendored next to this crate; their three call sites are
//! marked `cubecl:`.
pub mod ffi;

use std::ffi::{c_void, CStr};

use burn::tensor::backend::Backend;
use burn::tensor::ops::FloatTensor;
use burn_mamba::mamba2::ssd::serial_recalculated::Mamba2BackendExt;
use burn_mamba::mamba3::double_ssd::ssd::serial_recalculated::Mamba3DoubleSsdBackendExt;
use burn_mamba::mamba3::single_ssd::ssd::serial_recalculated::Mamba3SingleSsdBackendExt;

use ffi::*;

/// `CubeBackend<CudaRuntime, f32, i32, u8>` under a new name, so that the extension traits can be
/// implemented for it without colliding with burn-mamba's blanket impl.
#[derive(Clone, Copy, Debug, Default)]
pub struct B200;

type Inner = burn_cubecl::CubeBackend<burn::backend::cuda::CudaRuntime, f32, i32, u8>;

/// Dense row-major dims of a primitive.
fn dims<const D: usize>(t: &FloatTensor<B200>) -> [usize; D] {
    let s = t.shape();                     // cubecl: CubeTensor::shape
    core::array::from_fn(|i| s.dims[i])
}
/// Base device address of the buffer a primitive views.  For the permuted `dt` view this is the address of
/// the [b, n, l, h] memory it was permuted from, which is the dense [b, s, h] tensor the library takes.
fn device_ptr(t: &FloatTensor<B200>) -> *const c_void {
    t.client.get_resource(t.handle.clone().binding()).resource().ptr as *const c_void   // cubecl: raw CUdeviceptr
}
fn stream(t: &FloatTensor<B200>) -> *mut c_void {
    t.client.stream_handle() as *mut c_void                                              // cubecl: CUstream of the client
}
fn alloc_like(t: &FloatTensor<B200>, shape: &[usize], f32_out: bool) -> FloatTensor<B200> {
    burn_cubecl::ops::numeric::empty_device_dtype(t.client.clone(), t.device.clone(), shape.into(),
        if f32_out { burn::tensor::DType::F32 } else { t.dtype })                        // cubecl: uninitialised output
}
fn dtype_of(t: &FloatTensor<B200>) -> i32 {
    match t.dtype { burn::tensor::DType::BF16 => BM_DTYPE_BF16, burn::tensor::DType::F32 => BM_DTYPE_F32,
                    other => panic!("libbm_b200 takes f32 or bf16 activations, got {other:?}") }
}
fn check(rc: i32, what: &str) {
    // the reference panics at the same seam (assert!/unwrap in serial_recalculated.rs:39-44)
    if rc != BM_OK {
        let msg = unsafe { CStr::from_ptr(bm_last_error_string()) }.to_string_lossy().into_owned();
        panic!("{what} failed with status {rc}: {msg}");
    }
}
/// B / C reach the slot already expanded from groups to heads (src/modules/misc/gqa.rs:53-55).  When the
/// expand is still a stride-0 view the un-expanded [b, s, g, r] buffer can be passed with ngroups = g;
/// when Burn has materialised it, the per-head copy is passed with ngroups = h.
fn groups_of(t: &FloatTensor<B200>, nheads: usize) -> i32 {
    let st = &t.strides;                   // cubecl: CubeTensor::strides, element units
    if st[3] == 0 { 1 } else { nheads as i32 }
}

impl Mamba2BackendExt for B200 {
    fn ssd_serial_recalculated(
        x_bnlhp: FloatTensor<Self>, dt_discretized_bhnl: FloatTensor<Self>, b_bnlhr: FloatTensor<Self>,
        c_bnlhr: FloatTensor<Self>, d_h: FloatTensor<Self>, initial_state_bhpr: FloatTensor<Self>,
        a_decay_h: FloatTensor<Self>,
    ) -> (FloatTensor<Self>, FloatTensor<Self>) {
        let [b, n, l, h, p] = dims::<5>(&x_bnlhp);
        assert!(n > 0, "sequence length must be at least 1");
        let r = dims::<5>(&b_bnlhr)[4];
        let y = alloc_like(&x_bnlhp, &[b, n, l, h, p], false);
        let final_state = alloc_like(&x_bnlhp, &[b, h, p, r], true);
        // dt_discretized_bhnl is permute(0, 3, 1, 2) of [b, n, l, h] memory (serial_recalculated.rs:48): its base
        // pointer addresses exactly the dense [b, s, h] layout of the C ABI, no copy needed.
        let dt_bsh = device_ptr(&dt_discretized_bhnl) as *const f32;
        let mut args: BmSsd2FwdArgs = unsafe { core::mem::zeroed() };
        args.batch = b as i32; args.seqlen = (n * l) as i32; args.nheads = h as i32; args.headdim = p as i32;
        args.state_rank = r as i32; args.ngroups = groups_of(&b_bnlhr, h); args.chunk_len = l as i32;
        args.dtype = dtype_of(&x_bnlhp); args.path = BM_PATH_AUTO;
        args.x = device_ptr(&x_bnlhp); args.dt = dt_bsh; args.a = device_ptr(&a_decay_h) as *const f32;
        args.b = device_ptr(&b_bnlhr); args.c = device_ptr(&c_bnlhr); args.d = device_ptr(&d_h) as *const f32;
        args.h0 = device_ptr(&initial_state_bhpr) as *const f32;
        args.y = device_ptr(&y) as *mut c_void; args.h_final = device_ptr(&final_state) as *mut f32;
        let ws_bytes = unsafe { bm_ssd2_fwd_workspace_bytes(&args) };
        let ws = alloc_like(&x_bnlhp, &[ws_bytes.div_ceil(4)], true);
        check(unsafe { bm_ssd2_fwd(&args, device_ptr(&ws) as *mut c_void, ws_bytes, stream(&x_bnlhp)) }, "bm_ssd2_fwd");
        (y, final_state)
    }
}

impl Mamba3SingleSsdBackendExt for B200 {
    fn single_ssd_serial_recalculated(
        v_bnlmhp: FloatTensor<Self>, da_bnlh: FloatTensor<Self>, b_bnlmhr: FloatTensor<Self>,
        c_bnlmhr: FloatTensor<Self>, gamma_bnlh: FloatTensor<Self>, scale_bnlh: FloatTensor<Self>,
        initial_state_bhpr: FloatTensor<Self>, _siso_specialization: bool,
    ) -> (FloatTensor<Self>, FloatTensor<Self>) {
        ssd3(v_bnlmhp, da_bnlh, b_bnlmhr, c_bnlmhr, Some((gamma_bnlh, scale_bnlh)), initial_state_bhpr)
    }
}

impl Mamba3DoubleSsdBackendExt for B200 {
    fn double_ssd_serial_recalculated(
        v_bnlmhp: FloatTensor<Self>, da_bnlh: FloatTensor<Self>, b_bnlmhr: FloatTensor<Self>,
        c_bnlmhr: FloatTensor<Self>, initial_state_bhpr: FloatTensor<Self>,
    ) -> (FloatTensor<Self>, FloatTensor<Self>) {
        ssd3(v_bnlmhp, da_bnlh, b_bnlmhr, c_bnlmhr, None, initial_state_bhpr)
    }
}

fn ssd3(
    v: FloatTensor<B200>, da: FloatTensor<B200>, bm: FloatTensor<B200>, cm: FloatTensor<B200>,
    gamma_scale: Option<(FloatTensor<B200>, FloatTensor<B200>)>, h0: FloatTensor<B200>,
) -> (FloatTensor<B200>, FloatTensor<B200>) {
    let [b, n, l, m, h, p] = dims::<6>(&v);
    let r = dims::<6>(&bm)[5];
    let y = alloc_like(&v, &[b, n, l, m, h, p], false);
    let final_state = alloc_like(&v, &[b, h, p, r], true);
    let mut args: BmSsd3FwdArgs = unsafe { core::mem::zeroed() };
    args.batch = b as i32; args.seqlen = (n * l) as i32; args.nheads = h as i32; args.headdim = p as i32;
    args.state_rank = r as i32; args.mimo_rank = m as i32; args.chunk_len = l as i32;
    args.dtype = dtype_of(&v); args.path = BM_PATH_AUTO;
    args.v = device_ptr(&v); args.da = device_ptr(&da) as *const f32; args.b = device_ptr(&bm); args.c = device_ptr(&cm);
    if let Some((g, s)) = &gamma_scale {
        args.gamma = device_ptr(g) as *const f32; args.scale = device_ptr(s) as *const f32;
    }
    args.h0 = device_ptr(&h0) as *const f32;   // B / C are already rotated at this seam: angles stays NULL
    args.y = device_ptr(&y) as *mut c_void; args.h_final = device_ptr(&final_state) as *mut f32;
    let ws_bytes = unsafe { bm_ssd3_fwd_workspace_bytes(&args) };
    let ws = alloc_like(&v, &[ws_bytes.div_ceil(4)], true);
    let (wp, st) = (device_ptr(&ws) as *mut c_void, stream(&v));
    let rc = unsafe { if gamma_scale.is_some() { bm_ssd3_single_fwd(&args, wp, ws_bytes, st) } else { bm_ssd3_double_fwd(&args, wp, ws_bytes, st) } };
    check(rc, "bm_ssd3_fwd");
    (y, final_state)
}

// The seams without a trait slot -- Mamba1::selective_scan / selective_scan_step (src/mamba1/mamba1.rs:422, :666),
// the state update of Mamba2::step (src/mamba2/mamba2.rs:907-991) and Mamba3::step_double_ssd
// (src/mamba3/double_ssd/double_ssd/mod.rs:672-757) -- are plain functions of burn-mamba; the patch that swaps
// their bodies for bm_selscan1_fwd, bm_step1, bm_conv_step + bm_step2 and bm_step3 when the tensors live on `B200`
// follows the same pattern as above (fill the args struct from `dims` / `device_ptr`, call, `check`).
// The custom backward (src/mamba2/ssd/serial_recalculated/backward.rs:29-321) keeps its structure: its
// `Backward::backward` hands the saved forward inputs plus (dy, d_final_state) to bm_ssd2_bwd / bm_ssd3_*_bwd.
