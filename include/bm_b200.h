/*
 * bm_b200.h -- C ABI of libbm_b200.so: the burn-mamba SSM hot path for NVIDIA B200 (sm_100a).
 *
 * Every entry point
 *   - takes DEVICE pointers owned by the caller (plain pointers and sizes, no framework types),
 *   - is asynchronous on the CUDA stream passed as `stream` (a cudaStream_t cast to void*; NULL =
 *     the legacy default stream) and runs on the caller's current device,
 *   - allocates nothing: scratch memory is a caller-provided workspace whose size the matching
 *     *_workspace_bytes() function reports (a pure host function); the one exception is
 *     bm_ssd2_fwd_noalloc, which takes no workspace and uses a scratch array built into the library,
 *   - returns a bm_status (0 = OK, negative = error) and never aborts or throws; the message of the
 *     last error on the calling thread is available from bm_last_error_string().
 *
 * Layouts are dense row-major with the last-listed axis contiguous.  Shape letters follow the
 * reference crate: b batch, s sequence, h heads, p per-head dim, r state rank, g groups,
 * m MIMO rank, a rope angles, i d_inner (Mamba-1), v conv channels, k conv kernel.
 * "act dtype" tensors are float32 or bfloat16 as selected by the `dtype` field; decay inputs
 * (dt, da, A, D, gamma, scale, angles) and every recurrent state are always float32.
 * Pointers must be 16-byte aligned.  Head h reads B/C group h / (nheads / ngroups).
 *
 * Tensors are dense: there are no stride arguments.  The reference's slot receives two kinds of views,
 * and a binding re-bases both without copying:
 *   - dt arrives as [b, h, n, l], a permute(0, 3, 1, 2) of memory laid out [b, n, l, h]
 *     (src/mamba2/ssd/serial_recalculated/serial_recalculated.rs:48).  That memory *is* the dense
 *     [b, s, h] tensor this ABI takes (s = n * l): pass the view's base pointer.
 *   - B / C arrive group->head expanded (src/modules/misc/gqa.rs:53-55).  Pass the un-expanded
 *     [b, s, g, r] tensor with `ngroups` = g (head h reads group h / (nheads / ngroups)), or, if only the
 *     materialised per-head copy exists, pass it with `ngroups` = nheads.
 *
 * Citations are file:line inside swfsql/burn-mamba.
 */
#ifndef BM_B200_H
#define BM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    BM_OK = 0,
    BM_ERR_NULL_POINTER = -1,
    BM_ERR_BAD_SHAPE = -2,
    BM_ERR_BAD_ALIGNMENT = -3,
    BM_ERR_UNSUPPORTED = -4,
    BM_ERR_WORKSPACE_TOO_SMALL = -5,
    BM_ERR_CUDA = -6,
    BM_ERR_TIMEOUT = -7
} bm_status;

typedef enum { BM_DTYPE_F32 = 0, BM_DTYPE_BF16 = 1 } bm_dtype;

/* Kernel-family selection for the SSD forward entry points. */
typedef enum {
    BM_PATH_AUTO = 0,    /* tensor-core path when dtype/shape allow it, else the exact path */
    BM_PATH_EXACT = 1,   /* CUDA-core float32 arithmetic for any shape and dtype */
    BM_PATH_TENSOR = 2,  /* tcgen05/TMEM/TMA path; BM_ERR_UNSUPPORTED if the shape is not covered */
    /* the two kernels of the tensor-core path, which BM_PATH_AUTO / BM_PATH_TENSOR choose between by problem size */
    BM_PATH_TENSOR_SINGLE = 3,  /* one head per CTA */
    BM_PATH_TENSOR_PAIR = 4     /* two heads of a B/C group per CTA (even heads per group), sequence segments */
} bm_path;

/* ABI version (major << 16 | minor) and a human-readable build string. */
int32_t bm_version(void);
const char* bm_build_info(void);
/* Message of the last error raised on the calling thread ("" if none). */
const char* bm_last_error_string(void);

/* ------------------------------------------------------------------------------------------------
 * Mamba-2 chunked SSD forward.
 * Replaces Mamba2BackendExt::ssd_serial_recalculated
 *   (src/mamba2/ssd/serial_recalculated/serial_recalculated.rs:86-156) and the K1..K5 chain of
 *   ssd_serial (src/mamba2/ssd/serial.rs:34-506); call site src/mamba2/mamba2.rs:737-748.
 * seqlen need not be a multiple of chunk_len: the tail chunk behaves as if padded with dt = 0
 *   (src/mamba2/mamba2.rs:703-722).
 * y = exp(cum) (C . h^T) + ((C B^T) * exp(cum_t - cum_s)[s<=t] * dt_s) X + D X; h_final = state after
 * the last token.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
    int32_t batch, seqlen, nheads, headdim, state_rank, ngroups, chunk_len;
    int32_t dtype;            /* bm_dtype of x, b, c, y, z */
    int32_t path;             /* bm_path */
    int32_t reserved;         /* 0, or BM_DEBUG_STALL_LOADS (tests only, see below) */
    const void* x;            /* [b, s, h, p] act dtype */
    const float* dt;          /* [b, s, h]   discretised step (post softplus/clamp), or raw when dt_bias set */
    const float* a;           /* [h]         A_h = -exp(a_log_h) */
    const void* b;            /* [b, s, g, r] act dtype */
    const void* c;            /* [b, s, g, r] act dtype */
    const float* d;           /* [h] skip weight; NULL = no skip */
    const float* h0;          /* [b, h, p, r] initial state; NULL = zeros */
    const float* dt_bias;     /* [h] optional: dt := clamp(softplus(dt + dt_bias), dt_min, dt_max)
                                 (src/mamba2/mamba2.rs:692-697); NULL = dt used as given */
    float dt_min, dt_max;     /* clamp limits used with dt_bias (reference default 0, 65504) */
    const void* z;            /* [b, s, h, p] optional gate: y := y * silu(z)
                                 (the gate half of src/modules/norm/rms_norm_gated.rs:70-135); NULL = none */
    void* y;                  /* [b, s, h, p] act dtype */
    float* h_final;           /* [b, h, p, r] */
    float* chunk_states;      /* optional [b, ceil(s/chunk_len), h, p, r]: state entering every chunk
                                 (what K4 emits, src/mamba2/ssd/serial.rs:275-343); NULL = not wanted */
} bm_ssd2_fwd_args;

size_t bm_ssd2_fwd_workspace_bytes(const bm_ssd2_fwd_args* args);
int32_t bm_ssd2_fwd(const bm_ssd2_fwd_args* args, void* workspace, size_t workspace_bytes, void* stream);

/* Test-only value of bm_ssd2_fwd_args.reserved (no counterpart in the reference): the tensor-core kernel's
 * loader issues no loads, so the first bounded wait runs out (after about a second), every role leaves its
 * loop and the launch ends with BM_ERR_TIMEOUT in the workspace status word and unspecified outputs.  Nothing faults or hangs; the next call on the same context runs normally. */
#define BM_DEBUG_STALL_LOADS 0x57A11

/* Device-side status of the last SSD call that used `workspace` (no counterpart in the reference, whose
 * ops cannot time out).  The tensor-core kernels bound every wait on a barrier; a wait that gives up
 * records BM_ERR_TIMEOUT in the first word of the workspace and the kernel returns early with
 * unspecified outputs.  This call synchronises `stream`, reads that word and returns it (BM_OK when
 * the kernel ran to completion, or for paths that cannot time out). */
int32_t bm_workspace_status(const void* workspace, void* stream);

/* Allocation-free variant of bm_ssd2_fwd (exact path).  It has no counterpart in the reference.
 * It exists for callers that must not, or cannot, allocate device memory while running -- a server
 * with a memory budget fixed at start-up, or a plugin that receives raw tensor pointers from its
 * framework without access to the framework's allocator and so has nowhere to get a workspace from.
 * The scratch is a device array of BM_SSD2_NOALLOC_SCRATCH_BYTES built into the library (each GPU
 * that loads the library holds it until the process exits); the call allocates and frees nothing.
 *   - Same arguments, layouts and results as bm_ssd2_fwd with path BM_PATH_AUTO / BM_PATH_EXACT (float32
 *     arithmetic on CUDA cores; BM_PATH_TENSOR is refused with BM_ERR_UNSUPPORTED).
 *   - Problems whose scratch need (what bm_ssd2_fwd_workspace_bytes reports for BM_PATH_EXACT) exceeds the
 *     array are refused with BM_ERR_WORKSPACE_TOO_SMALL; nothing is launched.
 *   - The first call on each device looks the array's device address up (with that device current);
 *     make that first call outside any stream capture.  The address is cached for the life of the
 *     device's primary context: after cudaDeviceReset(), or any other teardown of that context, the
 *     library must be reloaded before this entry point is used again on that device.
 *   - All calls on a device share the one array and it keeps the previous call's contents; nothing in
 *     it needs clearing between calls, but two calls that overlap on the GPU (different streams) race
 *     on it: serialise them. */
#define BM_SSD2_NOALLOC_SCRATCH_BYTES (32u << 20)
int32_t bm_ssd2_fwd_noalloc(const bm_ssd2_fwd_args* args, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Mamba-2 chunked SSD backward (recompute: only the forward inputs are needed, no saved activations).
 * Replaces combined_backward (src/mamba2/ssd/serial_recalculated/combined_backward.rs:126-590) behind the
 * Autodiff impl of the slot (src/mamba2/ssd/serial_recalculated/backward.rs:29-321).
 * Forward inputs as in bm_ssd2_fwd (dt already discretised: dt_bias fusion is not differentiated here);
 * dy / dh_final are the upstream gradients of y and of the final state.  All gradients are float32.
 * db / dc are per group: already summed over the heads of each group (the reference returns them per
 * head and leaves that sum to the autodiff of its group->head expand, src/modules/misc/gqa.rs:30-56;
 * pass ngroups = nheads with per-head B/C to get exactly the per-head tensors).
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
    int32_t batch, seqlen, nheads, headdim, state_rank, ngroups, chunk_len;
    int32_t dtype;            /* bm_dtype of x, b, c, dy */
    const void* x;            /* [b, s, h, p] */
    const float* dt;          /* [b, s, h] */
    const float* a;           /* [h] */
    const void* b;            /* [b, s, g, r] */
    const void* c;            /* [b, s, g, r] */
    const float* d;           /* [h] or NULL */
    const float* h0;          /* [b, h, p, r] or NULL */
    const void* dy;           /* [b, s, h, p] act dtype */
    const float* dh_final;    /* [b, h, p, r] or NULL (zero) */
    float* dx;                /* [b, s, h, p] */
    float* ddt;               /* [b, s, h] */
    float* da;                /* [h] */
    float* db;                /* [b, s, g, r] */
    float* dc;                /* [b, s, g, r] */
    float* dd;                /* [h] or NULL */
    float* dh0;               /* [b, h, p, r] */
    int32_t path;             /* bm_path: AUTO = tensor-core kernel when dtype / shape allow it (bf16, headdim 64,
                                 state_rank 128), else the exact path; EXACT and TENSOR force one */
    int32_t reserved;         /* 0 */
} bm_ssd2_bwd_args;

size_t bm_ssd2_bwd_workspace_bytes(const bm_ssd2_bwd_args* args);
int32_t bm_ssd2_bwd(const bm_ssd2_bwd_args* args, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Mamba-2 recurrent step: state update + readout for one token, state updated in place.
 * Replaces the body of Mamba2::step between the conv and the gated norm
 *   (src/mamba2/mamba2.rs:907-991): h = exp(dt A) h + dt B (x) x ; y = sum_r C h + D x.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
    int32_t batch, nheads, headdim, state_rank, ngroups;
    int32_t dtype;            /* bm_dtype of x, b, c, y, z */
    float* state;             /* [b, h, p, r] in/out (Mamba2Cache.ssm_bhpr, src/mamba2/cache.rs:98-122) */
    const void* x;            /* [b, h, p] */
    const float* dt;          /* [b, h] discretised step, or raw when dt_bias set */
    const float* a;           /* [h] */
    const void* b;            /* [b, g, r] */
    const void* c;            /* [b, g, r] */
    const float* d;           /* [h] or NULL */
    const float* dt_bias;     /* [h] optional fused softplus(dt + bias) + clamp */
    float dt_min, dt_max;
    const void* z;            /* [b, h, p] optional gate y *= silu(z) */
    void* y;                  /* [b, h, p] */
} bm_step2_args;

int32_t bm_step2(const bm_step2_args* args, void* stream);

/* Causal depthwise conv window slide + dot + bias + SiLU for one token
 * (src/mamba2/mamba2.rs:865-902; Mamba-1 twin src/mamba1/mamba1.rs:556-590).
 * window: [b, v, k] float32, newest column last (src/mamba2/cache.rs:98-110); updated in place. */
typedef struct {
    int32_t batch, channels, kernel;
    int32_t dtype;            /* bm_dtype of xin / out */
    float* window;            /* [b, v, k] in/out */
    const void* xin;          /* [b, v] new pre-conv column */
    const float* weight;      /* [v, k] */
    const float* bias;        /* [v] or NULL */
    void* out;                /* [b, v] = silu(sum_k window * weight + bias); [b, split_x] when out_b is given */
    void* out_b;              /* optional [b, split_bc]: with out_c, the output leaves split along channels as the */
    void* out_c;              /*   x / B / C tensors bm_step2 reads (split_x + 2 split_bc = v); NULL = one tensor */
    int32_t xin_stride;       /* elements between batch rows of xin (a column slice of the projection); 0 = dense */
    int32_t split_x, split_bc;
    int32_t reserved;
} bm_conv_step_args;

int32_t bm_conv_step(const bm_conv_step_args* args, void* stream);

/* Prefill twin of bm_conv_step: causal depthwise conv over a whole sequence + bias + SiLU, with the left context
 * taken from the cache window and the new window written out (src/mamba2/mamba2.rs:618-654: window slide, Conv1d,
 * SiLU; Mamba-1 twin src/mamba1/mamba1.rs:316-340).  The input may be a column slice of the in-projection's
 * output (row stride `xin_stride`, elements).  The output is either one [b, s, v] tensor (out_b = out_c = NULL) or
 * the three tensors the SSD reads, split along channels exactly like the reference's split of xbc:
 * x [b, s, split_x], B [b, s, split_bc], C [b, s, split_bc] (split_x + 2 split_bc = v, multiples of 8).
 *   out[t, c] = silu(bias[c] + sum_k w[c, k] in[t - (K-1) + k, c]),  in[t < 0] = window[c, K + t]. */
typedef struct {
    int32_t batch, seqlen, channels, kernel;   /* kernel: 2, 3 or 4 taps */
    int32_t dtype;            /* bm_dtype of xin and the outputs */
    int32_t xin_stride;       /* elements between consecutive tokens of xin (>= channels, multiple of 8) */
    int32_t split_x, split_bc;
    const void* xin;          /* [b, s, v] rows of stride xin_stride */
    const float* weight;      /* [v, k] */
    const float* bias;        /* [v] or NULL */
    const float* window;      /* [b, v, k] cache window before the sequence (newest column last); NULL = zeros */
    float* new_window;        /* [b, v, k] window after the sequence, or NULL; must not alias `window` */
    void* out_x;              /* [b, s, split_x], or the whole [b, s, v] when out_b is NULL */
    void* out_b;              /* [b, s, split_bc] or NULL */
    void* out_c;              /* [b, s, split_bc] or NULL */
} bm_conv1d_silu_args;

int32_t bm_conv1d_silu_fwd(const bm_conv1d_silu_args* args, void* stream);

/* Gated RMS norm over the last axis, one row per token (RmsNormGated, src/modules/norm/rms_norm_gated.rs:70-135;
 * with z = NULL the plain RmsNorm, src/modules/norm/rms_norm.rs:53-98):
 *   norm_before_gate = 0 (the reference's default):  g = x silu(z);  out = g / sqrt(mean(g^2) + eps) * gamma
 *   norm_before_gate = 1:                            out = x / sqrt(mean(x^2) + eps) * gamma * silu(z)
 * x and z may be column slices of wider rows (row strides in elements); out is dense [rows, width]. */
typedef struct {
    int32_t rows, width;      /* width: multiple of 8, at most 8192 */
    int32_t dtype;            /* bm_dtype of x, z, gamma, out */
    int32_t norm_before_gate;
    int32_t x_stride, z_stride;
    float eps;                /* the reference's per-dtype epsilon (src/utils/mod.rs:50-95) */
    const void* x;
    const void* z;            /* or NULL */
    const void* gamma;        /* [width] */
    void* out;                /* [rows, width] */
} bm_rmsnorm_gated_args;

int32_t bm_rmsnorm_gated(const bm_rmsnorm_gated_args* args, void* stream);

/* Mamba-3: B and C from the in-projection's raw columns to what the SSD slot takes, in one pass:
 * RMS norm over r (weights b_gamma / c_gamma), group -> head expansion, + bias[h, m, r]
 * (qk_norm_expand_bias, src/mamba3/helpers.rs:82-95; call sites src/mamba3/single_ssd/single_ssd/mod.rs:156-169),
 * then the data-dependent rotation of the leading rope_dim entries by the cumulative angles
 * (rotate_bc_forward, src/mamba3/rotation/mod.rs:653-679; pairs (2j, 2j+1) when pairwise -- the reference's rule for
 * MIMO rank 1 -- else (j, j + r/2), src/modules/misc/rope.rs:50-170).  angles = NULL skips the rotation.
 * The raw rows may be column slices of the projection output (raw_stride elements between tokens). */
typedef struct {
    int32_t batch, seqlen, mimo_rank, ngroups, nheads, state_rank;   /* state_rank: multiple of 16 */
    int32_t dtype;            /* bm_dtype of the raw rows and the outputs */
    int32_t raw_stride;       /* elements between consecutive tokens of b_raw / c_raw (>= m g r) */
    int32_t rope_dim;         /* even, <= state_rank */
    int32_t pairwise;         /* 1: pairs (2j, 2j+1); 0: pairs (j, j + r/2) */
    float eps;                /* the reference's per-dtype epsilon (src/utils/mod.rs:50-95) */
    int32_t reserved;
    const void* b_raw;        /* [b, s, m, g, r] */
    const void* c_raw;
    const float* b_gamma;     /* [r] */
    const float* c_gamma;
    const float* b_bias;      /* [h, m, r] */
    const float* c_bias;
    const float* angles;      /* [b, s, h, rope_dim / 2] cumulative angles (bm_angle_cumsum), or NULL */
    void* b_out;              /* [b, s, m, h, r] */
    void* c_out;
} bm_mamba3_bc_prep_args;

int32_t bm_mamba3_bc_prep(const bm_mamba3_bc_prep_args* args, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Mamba-1 selective scan (sequence) and single-token step.
 * Replace Mamba1::selective_scan (src/mamba1/mamba1.rs:422-523) and
 *   Mamba1::selective_scan_step (src/mamba1/mamba1.rs:666-733):
 *   h = h exp(delta (x) A) + delta B u ; y = h . C + D u ; optional y *= silu(z) (the block's gate,
 *   src/mamba1/mamba1.rs:348).  All sequence tensors are batch-major [b, s, ...].
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
    int32_t batch, seqlen, d_inner, state_rank;
    int32_t dtype;            /* bm_dtype of u, delta, b, c, z, y */
    int32_t delta_softplus;   /* 1: delta := softplus(delta + delta_bias) (stock softplus, mamba1.rs:394) */
    const void* u;            /* [b, s, i] */
    const void* delta;        /* [b, s, i] */
    const float* a;           /* [i, r]  A = -exp(a_log) */
    const void* b;            /* [b, s, r] */
    const void* c;            /* [b, s, r] */
    const float* d;           /* [i] or NULL */
    const float* delta_bias;  /* [i] or NULL (only read when delta_softplus) */
    const void* z;            /* [b, s, i] or NULL */
    const float* h0;          /* [b, i, r] or NULL */
    void* y;                  /* [b, s, i] */
    float* h_final;           /* [b, i, r] */
} bm_selscan1_args;

int32_t bm_selscan1_fwd(const bm_selscan1_args* args, void* stream);

/* The same scan, parallel over the sequence as well (replaces the same reference function): the sequence is cut
 * into segments that are scanned on two levels (segment summaries, a short carry pass, outputs), which needs a
 * caller-provided workspace for the per-segment states.  Same arguments and results as bm_selscan1_fwd; covers
 * state_rank 16 (the reference's default) and falls back to bm_selscan1_fwd's kernels for other ranks. */
size_t bm_selscan1_fwd_workspace_bytes(const bm_selscan1_args* args);
int32_t bm_selscan1_fwd_ws(const bm_selscan1_args* args, void* workspace, size_t workspace_bytes, void* stream);

typedef struct {
    int32_t batch, d_inner, state_rank;
    int32_t dtype;
    int32_t delta_softplus;
    float* state;             /* [b, i, r] in/out (Mamba1Cache.ssm_bir, src/mamba1/cache.rs:30-47) */
    const void* u;            /* [b, i] */
    const void* delta;        /* [b, i] */
    const float* a;           /* [i, r] */
    const void* b;            /* [b, r] */
    const void* c;            /* [b, r] */
    const float* d;           /* [i] or NULL */
    const float* delta_bias;  /* [i] or NULL */
    const void* z;            /* [b, i] or NULL */
    void* y;                  /* [b, i] */
} bm_step1_args;

int32_t bm_step1(const bm_step1_args* args, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Mamba-3 SSD forward (single-pass and generic/double-pass cores).
 * bm_ssd3_single_fwd replaces Mamba3SingleSsdBackendExt::single_ssd_serial_recalculated
 *   (src/mamba3/single_ssd/ssd/serial_recalculated/serial_recalculated.rs:86-163; math in
 *   src/mamba3/single_ssd/ssd/serial.rs:56-268 and src/mamba3/single_ssd/ssd/diag.rs:50-100).
 * bm_ssd3_double_fwd replaces Mamba3DoubleSsdBackendExt::double_ssd_serial_recalculated
 *   (src/mamba3/double_ssd/ssd/serial_recalculated/serial_recalculated.rs:76-97; math in
 *   src/mamba3/double_ssd/ssd/serial.rs:56-409): gamma = scale = NULL, non-strict mask.
 * B and C are per head.  When `angles` is given, B and C are the *un-rotated* (normed + biased)
 * tensors and the data-dependent rotation of src/mamba3/rotation/mod.rs:653-679 /
 * src/modules/misc/rope.rs:50-170 is applied as they are loaded.
 * ---------------------------------------------------------------------------------------------- */
typedef struct {
    int32_t batch, seqlen, nheads, headdim, state_rank, mimo_rank, chunk_len;
    int32_t dtype;            /* bm_dtype of v, b, c, y */
    int32_t path;             /* bm_path */
    int32_t rope_dim;         /* number of leading B/C entries that rotate (even, <= r); used with angles */
    const void* v;            /* [b, s, m, h, p] */
    const float* da;          /* [b, s, h]  dt * A_t */
    const void* b;            /* [b, s, m, h, r] */
    const void* c;            /* [b, s, m, h, r] */
    const float* gamma;       /* [b, s, h] (single) or NULL (double) */
    const float* scale;       /* [b, s, h] (single) or NULL (double) */
    const float* h0;          /* [b, h, p, r] or NULL */
    const float* angles;      /* [b, s, h, a] cumulative angles, a = rope_dim / 2; NULL = B/C already rotated */
    void* y;                  /* [b, s, m, h, p] */
    float* h_final;           /* [b, h, p, r] */
} bm_ssd3_fwd_args;

size_t bm_ssd3_fwd_workspace_bytes(const bm_ssd3_fwd_args* args);
int32_t bm_ssd3_single_fwd(const bm_ssd3_fwd_args* args, void* workspace, size_t workspace_bytes, void* stream);
int32_t bm_ssd3_double_fwd(const bm_ssd3_fwd_args* args, void* workspace, size_t workspace_bytes, void* stream);

/* Mamba-3 SSD backward (recompute).  bm_ssd3_single_bwd replaces combined_backward of the single-pass core
 * (src/mamba3/single_ssd/ssd/serial_recalculated/combined_backward.rs:74-536: gradients for v, da, b, c,
 * gamma, scale, h0), bm_ssd3_double_bwd the generic core's
 * (src/mamba3/double_ssd/ssd/serial_recalculated/combined_backward.rs:98; dgamma / dscale unused).
 * B and C are the rotated per-head tensors (the rotation is differentiated outside the slot, as in the
 * reference).  All gradients float32. */
typedef struct {
    int32_t batch, seqlen, nheads, headdim, state_rank, mimo_rank, chunk_len;
    int32_t dtype;            /* bm_dtype of v, b, c, dy */
    const void* v;            /* [b, s, m, h, p] */
    const float* da;          /* [b, s, h] */
    const void* b;            /* [b, s, m, h, r] */
    const void* c;            /* [b, s, m, h, r] */
    const float* gamma;       /* [b, s, h] (single) */
    const float* scale;       /* [b, s, h] (single) */
    const float* h0;          /* [b, h, p, r] or NULL */
    const void* dy;           /* [b, s, m, h, p] */
    const float* dh_final;    /* [b, h, p, r] or NULL */
    float* dv;                /* [b, s, m, h, p] */
    float* dda;               /* [b, s, h] */
    float* db;                /* [b, s, m, h, r] */
    float* dc;                /* [b, s, m, h, r] */
    float* dgamma;            /* [b, s, h] (single) */
    float* dscale;            /* [b, s, h] (single) */
    float* dh0;               /* [b, h, p, r] */
    int32_t path;             /* bm_path: AUTO = tensor-core kernel when dtype / shape allow it (bf16, headdim 64,
                                 state_rank 128, mimo_rank 1, 2 or 4), else the exact path; EXACT and TENSOR force one */
    int32_t reserved;         /* 0 */
} bm_ssd3_bwd_args;

size_t bm_ssd3_bwd_workspace_bytes(const bm_ssd3_bwd_args* args);
int32_t bm_ssd3_single_bwd(const bm_ssd3_bwd_args* args, void* workspace, size_t workspace_bytes, void* stream);
int32_t bm_ssd3_double_bwd(const bm_ssd3_bwd_args* args, void* workspace, size_t workspace_bytes, void* stream);

/* Cumulative rotation angles (Complex2D), replacing the angle part of rotate_bc_forward
 * (src/mamba3/rotation/mod.rs:653-679, increment :559-567):
 *   theta[b,s,h,a] = prev[b,h,a] + cumsum_s( dt[b,s,h] * range * pi * tanh(rot[b,s,a]) ),
 *   last[b,h,a] = wrap(theta[b,S-1,h,a]) (src/modules/misc/rope.rs:23-27). */
typedef struct {
    int32_t batch, seqlen, nheads, nangles;
    float range;
    const float* rot;         /* [b, s, a] */
    const float* dt;          /* [b, s, h] */
    const float* prev;        /* [b, h, a] or NULL */
    float* theta;             /* [b, s, h, a] */
    float* last;              /* [b, h, a] or NULL */
} bm_angle_cumsum_args;

int32_t bm_angle_cumsum(const bm_angle_cumsum_args* args, void* stream);

/* Mamba-3 recurrent step: rotation of B/C by the updated angle, state update, readout.
 * Replaces the core of Mamba3::step_double_ssd (src/mamba3/double_ssd/double_ssd/mod.rs:672-757;
 * rotation src/mamba3/rotation/mod.rs:729-764):
 *   h = alpha h + sum_m (gamma x*mx_m) (x) B_m + sum_m (beta x_prev*mx_m) (x) Bprev_m ; y_m = C_m . h
 * and rolls the cache: k_state := rotated B, v_state := x, angle := wrapped new angle. */
typedef struct {
    int32_t batch, nheads, headdim, state_rank, mimo_rank, rope_dim;
    float range;
    float* state;             /* [b, h, p, r] in/out */
    float* k_state;           /* [b, m, h, r] in/out: rotated B of the previous token */
    float* v_state;           /* [b, h, p]    in/out: x of the previous token */
    float* angle;             /* [b, h, a]    in/out, a = max(rope_dim / 2, 1) */
    const float* x;           /* [b, h, p] */
    const float* b;           /* [b, m, h, r] normed + biased, un-rotated */
    const float* c;           /* [b, m, h, r] normed + biased, un-rotated */
    const float* rot;         /* [b, a] raw rotation channels */
    const float* dt;          /* [b, h] */
    const float* alpha;       /* [b, h] */
    const float* beta;        /* [b, h] */
    const float* gamma;       /* [b, h] */
    const float* mimo_x;      /* [h, m, p] or NULL (treated as ones) */
    float* y;                 /* [b, m, h, p] = C_m . h (before the D skip) */
} bm_step3_args;

int32_t bm_step3(const bm_step3_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BM_B200_H */
