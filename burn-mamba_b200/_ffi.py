"""ctypes binding of libbm_b200.so (the C ABI declared in include/bm_b200.h).

The library is the product; this module only loads it and describes its structs.  There is no
fallback: if the shared library is missing, importing this module raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# BM_B200_LIB selects another build of the same library (e.g. an instrumented development build)
LIB_PATH = os.environ.get("BM_B200_LIB") or os.path.join(_HERE, "libbm_b200.so")

BM_OK = 0
BM_ERR_NULL_POINTER, BM_ERR_BAD_SHAPE, BM_ERR_BAD_ALIGNMENT, BM_ERR_UNSUPPORTED = -1, -2, -3, -4
BM_ERR_WORKSPACE_TOO_SMALL, BM_ERR_CUDA, BM_ERR_TIMEOUT = -5, -6, -7
BM_DTYPE_F32, BM_DTYPE_BF16 = 0, 1
BM_PATH_AUTO, BM_PATH_EXACT, BM_PATH_TENSOR, BM_PATH_TENSOR_SINGLE, BM_PATH_TENSOR_PAIR = 0, 1, 2, 3, 4
BM_SSD2_NOALLOC_SCRATCH_BYTES = 32 << 20
BM_DEBUG_STALL_LOADS = 0x57A11   # bm_ssd2_fwd_args.reserved: test hook that makes a bounded wait run out

_i32, _f32, _vp = C.c_int32, C.c_float, C.c_void_p


class Ssd2FwdArgs(C.Structure):
    _fields_ = [(n, _i32) for n in ("batch", "seqlen", "nheads", "headdim", "state_rank", "ngroups", "chunk_len",
                                    "dtype", "path", "reserved")] + [
        ("x", _vp), ("dt", _vp), ("a", _vp), ("b", _vp), ("c", _vp), ("d", _vp), ("h0", _vp), ("dt_bias", _vp),
        ("dt_min", _f32), ("dt_max", _f32), ("z", _vp), ("y", _vp), ("h_final", _vp), ("chunk_states", _vp)]


class Step2Args(C.Structure):
    _fields_ = [(n, _i32) for n in ("batch", "nheads", "headdim", "state_rank", "ngroups", "dtype")] + [
        ("state", _vp), ("x", _vp), ("dt", _vp), ("a", _vp), ("b", _vp), ("c", _vp), ("d", _vp), ("dt_bias", _vp),
        ("dt_min", _f32), ("dt_max", _f32), ("z", _vp), ("y", _vp)]


class ConvStepArgs(C.Structure):
    _fields_ = [(n, _i32) for n in ("batch", "channels", "kernel", "dtype")] + [
        ("window", _vp), ("xin", _vp), ("weight", _vp), ("bias", _vp), ("out", _vp), ("out_b", _vp), ("out_c", _vp),
        ("xin_stride", _i32), ("split_x", _i32), ("split_bc", _i32), ("reserved", _i32)]


class Conv1dSiluArgs(C.Structure):
    _fields_ = [(n, _i32) for n in ("batch", "seqlen", "channels", "kernel", "dtype", "xin_stride", "split_x", "split_bc")] + [
        ("xin", _vp), ("weight", _vp), ("bias", _vp), ("window", _vp), ("new_window", _vp), ("out_x", _vp),
        ("out_b", _vp), ("out_c", _vp)]


class RmsnormGatedArgs(C.Structure):
    _fields_ = [(n, _i32) for n in ("rows", "width", "dtype", "norm_before_gate", "x_stride", "z_stride")] + [
        ("eps", _f32), ("x", _vp), ("z", _vp), ("gamma", _vp), ("out", _vp)]


class Selscan1Args(C.Structure):
    _fields_ = [(n, _i32) for n in ("batch", "seqlen", "d_inner", "state_rank", "dtype", "delta_softplus")] + [
        ("u", _vp), ("delta", _vp), ("a", _vp), ("b", _vp), ("c", _vp), ("d", _vp), ("delta_bias", _vp), ("z", _vp),
        ("h0", _vp), ("y", _vp), ("h_final", _vp)]


class Step1Args(C.Structure):
    _fields_ = [(n, _i32) for n in ("batch", "d_inner", "state_rank", "dtype", "delta_softplus")] + [
        ("state", _vp), ("u", _vp), ("delta", _vp), ("a", _vp), ("b", _vp), ("c", _vp), ("d", _vp),
        ("delta_bias", _vp), ("z", _vp), ("y", _vp)]


class Ssd3FwdArgs(C.Structure):
    _fields_ = [(n, _i32) for n in ("batch", "seqlen", "nheads", "headdim", "state_rank", "mimo_rank", "chunk_len",
                                    "dtype", "path", "rope_dim")] + [
        ("v", _vp), ("da", _vp), ("b", _vp), ("c", _vp), ("gamma", _vp), ("scale", _vp), ("h0", _vp), ("angles", _vp),
        ("y", _vp), ("h_final", _vp)]


class Ssd2BwdArgs(C.Structure):
    _fields_ = [(n, _i32) for n in ("batch", "seqlen", "nheads", "headdim", "state_rank", "ngroups", "chunk_len",
                                    "dtype")] + [
        (n, _vp) for n in ("x", "dt", "a", "b", "c", "d", "h0", "dy", "dh_final", "dx", "ddt", "da", "db", "dc", "dd",
                           "dh0")] + [("path", _i32), ("reserved", _i32)]


class Ssd3BwdArgs(C.Structure):
    _fields_ = [(n, _i32) for n in ("batch", "seqlen", "nheads", "headdim", "state_rank", "mimo_rank", "chunk_len",
                                    "dtype")] + [
        (n, _vp) for n in ("v", "da", "b", "c", "gamma", "scale", "h0", "dy", "dh_final", "dv", "dda", "db", "dc",
                           "dgamma", "dscale", "dh0")] + [("path", _i32), ("reserved", _i32)]


class Mamba3BcPrepArgs(C.Structure):
    _fields_ = [(n, _i32) for n in ("batch", "seqlen", "mimo_rank", "ngroups", "nheads", "state_rank", "dtype", "raw_stride",
                                    "rope_dim", "pairwise")] + [("eps", _f32), ("reserved", _i32)] + [
        (n, _vp) for n in ("b_raw", "c_raw", "b_gamma", "c_gamma", "b_bias", "c_bias", "angles", "b_out", "c_out")]


class AngleCumsumArgs(C.Structure):
    _fields_ = [(n, _i32) for n in ("batch", "seqlen", "nheads", "nangles")] + [
        ("range", _f32), ("rot", _vp), ("dt", _vp), ("prev", _vp), ("theta", _vp), ("last", _vp)]


class Step3Args(C.Structure):
    _fields_ = [(n, _i32) for n in ("batch", "nheads", "headdim", "state_rank", "mimo_rank", "rope_dim")] + [
        ("range", _f32), ("state", _vp), ("k_state", _vp), ("v_state", _vp), ("angle", _vp), ("x", _vp), ("b", _vp),
        ("c", _vp), ("rot", _vp), ("dt", _vp), ("alpha", _vp), ("beta", _vp), ("gamma", _vp), ("mimo_x", _vp),
        ("y", _vp)]


# symbol -> (restype, argtypes); every function include/bm_b200.h declares
SYMBOLS = {
    "bm_version": (_i32, []),
    "bm_build_info": (C.c_char_p, []),
    "bm_last_error_string": (C.c_char_p, []),
    "bm_ssd2_fwd_workspace_bytes": (C.c_size_t, [C.POINTER(Ssd2FwdArgs)]),
    "bm_ssd2_fwd": (_i32, [C.POINTER(Ssd2FwdArgs), _vp, C.c_size_t, _vp]),
    "bm_workspace_status": (_i32, [_vp, _vp]),
    "bm_ssd2_fwd_noalloc": (_i32, [C.POINTER(Ssd2FwdArgs), _vp]),
    "bm_ssd2_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(Ssd2BwdArgs)]),
    "bm_ssd2_bwd": (_i32, [C.POINTER(Ssd2BwdArgs), _vp, C.c_size_t, _vp]),
    "bm_ssd3_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(Ssd3BwdArgs)]),
    "bm_ssd3_single_bwd": (_i32, [C.POINTER(Ssd3BwdArgs), _vp, C.c_size_t, _vp]),
    "bm_ssd3_double_bwd": (_i32, [C.POINTER(Ssd3BwdArgs), _vp, C.c_size_t, _vp]),
    "bm_step2": (_i32, [C.POINTER(Step2Args), _vp]),
    "bm_conv_step": (_i32, [C.POINTER(ConvStepArgs), _vp]),
    "bm_conv1d_silu_fwd": (_i32, [C.POINTER(Conv1dSiluArgs), _vp]),
    "bm_rmsnorm_gated": (_i32, [C.POINTER(RmsnormGatedArgs), _vp]),
    "bm_mamba3_bc_prep": (_i32, [C.POINTER(Mamba3BcPrepArgs), _vp]),
    "bm_selscan1_fwd": (_i32, [C.POINTER(Selscan1Args), _vp]),
    "bm_selscan1_fwd_workspace_bytes": (C.c_size_t, [C.POINTER(Selscan1Args)]),
    "bm_selscan1_fwd_ws": (_i32, [C.POINTER(Selscan1Args), _vp, C.c_size_t, _vp]),
    "bm_step1": (_i32, [C.POINTER(Step1Args), _vp]),
    "bm_ssd3_fwd_workspace_bytes": (C.c_size_t, [C.POINTER(Ssd3FwdArgs)]),
    "bm_ssd3_single_fwd": (_i32, [C.POINTER(Ssd3FwdArgs), _vp, C.c_size_t, _vp]),
    "bm_ssd3_double_fwd": (_i32, [C.POINTER(Ssd3FwdArgs), _vp, C.c_size_t, _vp]),
    "bm_angle_cumsum": (_i32, [C.POINTER(AngleCumsumArgs), _vp]),
    "bm_step3": (_i32, [C.POINTER(Step3Args), _vp]),
}


def load(path=LIB_PATH):
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: build it with `python burn-mamba_b200/build.py` "
                          "(there is no fallback implementation)")
    lib = C.CDLL(path)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = load()


class BmError(RuntimeError):
    """A non-zero bm_status; mirrors the reference's panics (assert!/unwrap) at the same call sites."""

    def __init__(self, code, where):
        self.code = code
        msg = lib.bm_last_error_string().decode()
        super().__init__(f"{where} failed with status {code}: {msg}")


def check(code, where):
    if code != BM_OK:
        raise BmError(code, where)
