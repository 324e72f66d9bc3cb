// C-ABI entry points of the chunked SSD forward (Mamba-2, Mamba-3 single / double): argument
// validation and dispatch between the exact path and the tensor-core path.
#include <algorithm>
#include "common.cuh"
#include "ssd2_tc.cuh"
#include "ssd_exact.cuh"

using namespace bm;

static int32_t validate_ssd2(const bm_ssd2_fwd_args* a) {
    if (a == nullptr) return fail(BM_ERR_NULL_POINTER, "args is NULL");
    BM_REQUIRE(a->batch > 0 && a->seqlen > 0 && a->nheads > 0 && a->headdim > 0 && a->state_rank > 0, BM_ERR_BAD_SHAPE,
               "batch, seqlen, nheads, headdim, state_rank must be positive (sequence length must be at least 1)");
    BM_REQUIRE(a->chunk_len > 0, BM_ERR_BAD_SHAPE, "chunk_len must be positive");
    BM_REQUIRE(a->ngroups > 0 && a->nheads % a->ngroups == 0, BM_ERR_BAD_SHAPE, "nheads must be divisible by ngroups");
    BM_REQUIRE(a->dtype == BM_DTYPE_F32 || a->dtype == BM_DTYPE_BF16, BM_ERR_UNSUPPORTED, "dtype must be f32 or bf16");
    BM_REQUIRE(a->path >= BM_PATH_AUTO && a->path <= BM_PATH_TENSOR_PAIR, BM_ERR_UNSUPPORTED, "unknown path %d", a->path);
    BM_REQUIRE_PTR(a->x);
    BM_REQUIRE_PTR(a->dt);
    BM_REQUIRE_PTR(a->a);
    BM_REQUIRE_PTR(a->b);
    BM_REQUIRE_PTR(a->c);
    BM_REQUIRE_PTR(a->y);
    BM_REQUIRE_PTR(a->h_final);
    BM_OPTIONAL_PTR(a->d);
    BM_OPTIONAL_PTR(a->h0);
    BM_OPTIONAL_PTR(a->dt_bias);
    BM_OPTIONAL_PTR(a->z);
    BM_OPTIONAL_PTR(a->chunk_states);
    return BM_OK;
}

static bool ssd2_use_tensor(const bm_ssd2_fwd_args* a) {
    if (a->path == BM_PATH_EXACT) return false;
    return tc::ssd2_supported(a);
}

// Which tensor-core kernel serves the call: two heads per CTA when asked for, or when the problem has more
// (batch x head) units than SMs and its heads pair up; one head per CTA otherwise.
static bool ssd2_use_pair(const bm_ssd2_fwd_args* a) {
    if (a->path == BM_PATH_TENSOR_SINGLE) return false;
    if (a->path == BM_PATH_TENSOR_PAIR) return true;
    return tc::ssd2_pair_preferred(a);
}

static exact::Params ssd2_exact_params(const bm_ssd2_fwd_args* a) {
    exact::Params p{};
    p.B = a->batch, p.S = a->seqlen, p.H = a->nheads, p.P = a->headdim, p.R = a->state_rank;
    p.G = a->ngroups, p.M = 1, p.Q = a->chunk_len;
    p.dtype = a->dtype, p.strict = 0, p.cs_mode = 1, p.rope_dim = 0, p.pairwise = 1;
    p.v = a->x, p.bmat = a->b, p.cmat = a->c, p.dsrc = a->dt, p.a = a->a;
    p.dt_bias = a->dt_bias, p.dt_min = a->dt_min, p.dt_max = a->dt_max;
    p.d = a->d, p.h0 = a->h0, p.z = a->z, p.y = a->y, p.h_final = a->h_final;
    p.states = a->chunk_states;
    return p;
}

extern "C" size_t bm_ssd2_fwd_workspace_bytes(const bm_ssd2_fwd_args* a) {
    if (a == nullptr || a->batch <= 0 || a->seqlen <= 0 || a->nheads <= 0 || a->chunk_len <= 0) return 0;
    size_t ex = exact::workspace_bytes(a->batch, a->seqlen, a->nheads, a->headdim, a->state_rank, a->chunk_len,
                                       a->chunk_states == nullptr);
    if (a->path == BM_PATH_EXACT) return ex;
    size_t t = 0;
    if (tc::ssd2_supported(a)) {
        t = tc::ssd2_workspace_bytes(a);
        if (tc::ssd2_pair_supported(a) && a->path != BM_PATH_TENSOR_SINGLE) {
            const size_t tp = tc::ssd2_pair_workspace_bytes(a);
            t = tp > t ? tp : t;
        }
    }
    if (a->path != BM_PATH_AUTO) return t;
    return t > 0 ? t : ex;
}

extern "C" int32_t bm_ssd2_fwd(const bm_ssd2_fwd_args* a, void* workspace, size_t workspace_bytes, void* stream) {
    clear_error();
    if (int32_t e = validate_ssd2(a)) return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (a->path >= BM_PATH_TENSOR && !tc::ssd2_supported(a))
        return fail(BM_ERR_UNSUPPORTED, "tensor-core SSD path does not cover this shape/dtype: %s", tc::ssd2_why_not(a));
    if (a->path == BM_PATH_TENSOR_PAIR && !tc::ssd2_pair_supported(a))
        return fail(BM_ERR_UNSUPPORTED, "the paired tensor-core kernel needs an even number of heads per group");
    if (ssd2_use_tensor(a)) {
        if (ssd2_use_pair(a)) return tc::ssd2_pair_run(a, workspace, workspace_bytes, st);
        return tc::ssd2_run(a, workspace, workspace_bytes, st);
    }
    return exact::run(ssd2_exact_params(a), workspace, workspace_bytes, st);
}

extern "C" int32_t bm_ssd2_fwd_noalloc(const bm_ssd2_fwd_args* a, void* stream) {
    clear_error();
    if (int32_t e = validate_ssd2(a)) return e;
    if (a->path >= BM_PATH_TENSOR)
        return fail(BM_ERR_UNSUPPORTED, "bm_ssd2_fwd_noalloc runs the exact path only");
    return exact::run_noalloc(ssd2_exact_params(a), static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------
static int32_t validate_ssd3(const bm_ssd3_fwd_args* a, bool single) {
    if (a == nullptr) return fail(BM_ERR_NULL_POINTER, "args is NULL");
    BM_REQUIRE(a->batch > 0 && a->seqlen > 0 && a->nheads > 0 && a->headdim > 0 && a->state_rank > 0 && a->mimo_rank > 0,
               BM_ERR_BAD_SHAPE, "batch, seqlen, nheads, headdim, state_rank, mimo_rank must be positive");
    BM_REQUIRE(a->chunk_len > 0, BM_ERR_BAD_SHAPE, "chunk_len must be positive");
    BM_REQUIRE(a->dtype == BM_DTYPE_F32 || a->dtype == BM_DTYPE_BF16, BM_ERR_UNSUPPORTED, "dtype must be f32 or bf16");
    BM_REQUIRE_PTR(a->v);
    BM_REQUIRE_PTR(a->da);
    BM_REQUIRE_PTR(a->b);
    BM_REQUIRE_PTR(a->c);
    BM_REQUIRE_PTR(a->y);
    BM_REQUIRE_PTR(a->h_final);
    BM_OPTIONAL_PTR(a->h0);
    BM_OPTIONAL_PTR(a->angles);
    if (single) {
        BM_REQUIRE_PTR(a->gamma);
        BM_REQUIRE_PTR(a->scale);
    }
    if (a->angles) {
        BM_REQUIRE(a->rope_dim >= 0 && a->rope_dim % 2 == 0 && a->rope_dim <= a->state_rank, BM_ERR_BAD_SHAPE,
                   "rope_dim must be even and <= state_rank");
        BM_REQUIRE(a->state_rank % 2 == 0, BM_ERR_BAD_SHAPE, "state_rank must be even when rotating");
    }
    BM_REQUIRE(a->path >= BM_PATH_AUTO && a->path <= BM_PATH_TENSOR_SINGLE, BM_ERR_UNSUPPORTED,
               "path must be auto, exact or tensor (the Mamba-3 cores have no paired kernel: B and C are per head)");
    if (a->path >= BM_PATH_TENSOR && !tc::ssd3_supported(a))
        return fail(BM_ERR_UNSUPPORTED, "tensor-core SSD path does not cover this shape/dtype: %s", tc::ssd3_why_not(a));
    return BM_OK;
}

static exact::Params ssd3_exact_params(const bm_ssd3_fwd_args* a, bool single) {
    exact::Params p{};
    p.B = a->batch, p.S = a->seqlen, p.H = a->nheads, p.P = a->headdim, p.R = a->state_rank;
    p.G = a->nheads, p.M = a->mimo_rank, p.Q = a->chunk_len;
    p.dtype = a->dtype;
    p.strict = single ? 1 : 0;
    p.cs_mode = single ? 2 : 0;
    p.rope_dim = a->angles ? a->rope_dim : 0;
    p.pairwise = a->mimo_rank == 1;  // rotate_pairwise = mimo_rank == 1 (src/mamba3/rotation/mod.rs:665)
    p.v = a->v, p.bmat = a->b, p.cmat = a->c, p.dsrc = a->da, p.a = nullptr;
    p.colscale = single ? a->scale : nullptr;
    p.gamma = single ? a->gamma : nullptr;
    p.h0 = a->h0, p.angles = a->angles, p.y = a->y, p.h_final = a->h_final;
    return p;
}

static bool ssd3_use_tensor(const bm_ssd3_fwd_args* a) { return a->path != BM_PATH_EXACT && tc::ssd3_supported(a); }

extern "C" size_t bm_ssd3_fwd_workspace_bytes(const bm_ssd3_fwd_args* a) {
    if (a == nullptr || a->batch <= 0 || a->seqlen <= 0 || a->nheads <= 0 || a->chunk_len <= 0) return 0;
    if (ssd3_use_tensor(a)) return tc::ssd3_workspace_bytes(a);
    return exact::workspace_bytes(a->batch, a->seqlen, a->nheads, a->headdim, a->state_rank, a->chunk_len, true);
}

static int32_t ssd3_fwd(const bm_ssd3_fwd_args* a, bool single, void* ws, size_t ws_bytes, void* stream) {
    clear_error();
    if (int32_t e = validate_ssd3(a, single)) return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (ssd3_use_tensor(a)) return tc::ssd3_run(a, single, ws, ws_bytes, st);
    return exact::run(ssd3_exact_params(a, single), ws, ws_bytes, st);
}

extern "C" int32_t bm_ssd3_single_fwd(const bm_ssd3_fwd_args* a, void* ws, size_t ws_bytes, void* stream) {
    return ssd3_fwd(a, true, ws, ws_bytes, stream);
}

extern "C" int32_t bm_ssd3_double_fwd(const bm_ssd3_fwd_args* a, void* ws, size_t ws_bytes, void* stream) {
    return ssd3_fwd(a, false, ws, ws_bytes, stream);
}

extern "C" int32_t bm_workspace_status(const void* workspace, void* stream) {
    clear_error();
    if (workspace == nullptr) return fail(BM_ERR_NULL_POINTER, "workspace is NULL");
    int32_t word = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int32_t e = check_cuda(cudaMemcpyAsync(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync(status)"))
        return e;
    if (int32_t e = check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize")) return e;
    if (word == BM_ERR_TIMEOUT) return fail(BM_ERR_TIMEOUT, "a bounded barrier wait inside the SSD kernel ran out");
    return BM_OK;
}

// ---------------------------------------------------------------------------------------------
// Backward entry points
// ---------------------------------------------------------------------------------------------
extern "C" size_t bm_ssd2_bwd_workspace_bytes(const bm_ssd2_bwd_args* a) {
    if (a == nullptr || a->batch <= 0 || a->seqlen <= 0 || a->nheads <= 0 || a->chunk_len <= 0) return 0;
    size_t n = exact::bwd_workspace_bytes(a->batch, a->seqlen, a->nheads, a->headdim, a->state_rank, a->chunk_len, true);
    if (a->path != BM_PATH_EXACT && tc::ssd2_bwd_supported(a)) n = std::max(n, tc::ssd2_bwd_workspace_bytes(a));
    return n;
}

extern "C" int32_t bm_ssd2_bwd(const bm_ssd2_bwd_args* a, void* ws, size_t ws_bytes, void* stream) {
    clear_error();
    if (a == nullptr) return fail(BM_ERR_NULL_POINTER, "args is NULL");
    BM_REQUIRE(a->batch > 0 && a->seqlen > 0 && a->nheads > 0 && a->headdim > 0 && a->state_rank > 0, BM_ERR_BAD_SHAPE,
               "batch, seqlen, nheads, headdim, state_rank must be positive");
    BM_REQUIRE(a->chunk_len > 0, BM_ERR_BAD_SHAPE, "chunk_len must be positive");
    BM_REQUIRE(a->ngroups > 0 && a->nheads % a->ngroups == 0, BM_ERR_BAD_SHAPE, "nheads must be divisible by ngroups");
    BM_REQUIRE(a->dtype == BM_DTYPE_F32 || a->dtype == BM_DTYPE_BF16, BM_ERR_UNSUPPORTED, "dtype must be f32 or bf16");
    BM_REQUIRE_PTR(a->x); BM_REQUIRE_PTR(a->dt); BM_REQUIRE_PTR(a->a); BM_REQUIRE_PTR(a->b); BM_REQUIRE_PTR(a->c);
    BM_REQUIRE_PTR(a->dy); BM_REQUIRE_PTR(a->dx); BM_REQUIRE_PTR(a->ddt); BM_REQUIRE_PTR(a->da); BM_REQUIRE_PTR(a->db);
    BM_REQUIRE_PTR(a->dc); BM_REQUIRE_PTR(a->dh0);
    BM_OPTIONAL_PTR(a->d); BM_OPTIONAL_PTR(a->h0); BM_OPTIONAL_PTR(a->dh_final); BM_OPTIONAL_PTR(a->dd);
    BM_REQUIRE((a->d == nullptr) == (a->dd == nullptr), BM_ERR_NULL_POINTER, "d and dd must be given together");
    BM_REQUIRE(a->path == BM_PATH_AUTO || a->path == BM_PATH_EXACT || a->path == BM_PATH_TENSOR, BM_ERR_UNSUPPORTED,
               "path must be auto, exact or tensor");
    if (a->path != BM_PATH_EXACT) {
        if (tc::ssd2_bwd_supported(a)) return tc::ssd2_bwd_run(a, ws, ws_bytes, static_cast<cudaStream_t>(stream));
        if (a->path == BM_PATH_TENSOR) return fail(BM_ERR_UNSUPPORTED, "tensor-core backward: %s", tc::ssd2_bwd_why_not(a));
    }
    exact::BwdParams bp{};
    exact::Params& p = bp.fwd;
    p.B = a->batch, p.S = a->seqlen, p.H = a->nheads, p.P = a->headdim, p.R = a->state_rank;
    p.G = a->ngroups, p.M = 1, p.Q = a->chunk_len, p.dtype = a->dtype, p.strict = 0, p.cs_mode = 1, p.pairwise = 1;
    p.v = a->x, p.bmat = a->b, p.cmat = a->c, p.dsrc = a->dt, p.a = a->a, p.d = a->d, p.h0 = a->h0;
    bp.dy = a->dy, bp.dh_final = a->dh_final, bp.dv = a->dx, bp.db = a->db, bp.dc = a->dc;
    bp.d_dt = a->ddt, bp.d_a = a->da, bp.dd = a->dd, bp.dh0 = a->dh0;
    return exact::run_bwd(bp, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" size_t bm_ssd3_bwd_workspace_bytes(const bm_ssd3_bwd_args* a) {
    if (a == nullptr || a->batch <= 0 || a->seqlen <= 0 || a->nheads <= 0 || a->chunk_len <= 0) return 0;
    size_t n = exact::bwd_workspace_bytes(a->batch, a->seqlen, a->nheads, a->headdim, a->state_rank, a->chunk_len, false);
    if (a->path != BM_PATH_EXACT && tc::ssd3_bwd_supported(a)) n = std::max(n, tc::ssd3_bwd_workspace_bytes(a));
    return n;
}

static int32_t ssd3_bwd(const bm_ssd3_bwd_args* a, void* ws, size_t ws_bytes, void* stream, bool single) {
    clear_error();
    if (a == nullptr) return fail(BM_ERR_NULL_POINTER, "args is NULL");
    BM_REQUIRE(a->batch > 0 && a->seqlen > 0 && a->nheads > 0 && a->headdim > 0 && a->state_rank > 0 && a->mimo_rank > 0,
               BM_ERR_BAD_SHAPE, "batch, seqlen, nheads, headdim, state_rank, mimo_rank must be positive");
    BM_REQUIRE(a->chunk_len > 0, BM_ERR_BAD_SHAPE, "chunk_len must be positive");
    BM_REQUIRE(a->dtype == BM_DTYPE_F32 || a->dtype == BM_DTYPE_BF16, BM_ERR_UNSUPPORTED, "dtype must be f32 or bf16");
    BM_REQUIRE_PTR(a->v); BM_REQUIRE_PTR(a->da); BM_REQUIRE_PTR(a->b); BM_REQUIRE_PTR(a->c); BM_REQUIRE_PTR(a->dy);
    BM_REQUIRE_PTR(a->dv); BM_REQUIRE_PTR(a->dda); BM_REQUIRE_PTR(a->db); BM_REQUIRE_PTR(a->dc); BM_REQUIRE_PTR(a->dh0);
    BM_OPTIONAL_PTR(a->h0); BM_OPTIONAL_PTR(a->dh_final);
    if (single) {
        BM_REQUIRE_PTR(a->gamma); BM_REQUIRE_PTR(a->scale); BM_REQUIRE_PTR(a->dgamma); BM_REQUIRE_PTR(a->dscale);
    }
    BM_REQUIRE(a->path == BM_PATH_AUTO || a->path == BM_PATH_EXACT || a->path == BM_PATH_TENSOR, BM_ERR_UNSUPPORTED,
               "path must be auto, exact or tensor");
    if (a->path != BM_PATH_EXACT) {
        if (tc::ssd3_bwd_supported(a)) return tc::ssd3_bwd_run(a, single, ws, ws_bytes, static_cast<cudaStream_t>(stream));
        if (a->path == BM_PATH_TENSOR) return fail(BM_ERR_UNSUPPORTED, "tensor-core backward: %s", tc::ssd3_bwd_why_not(a));
    }
    exact::BwdParams bp{};
    exact::Params& p = bp.fwd;
    p.B = a->batch, p.S = a->seqlen, p.H = a->nheads, p.P = a->headdim, p.R = a->state_rank;
    p.G = a->nheads, p.M = a->mimo_rank, p.Q = a->chunk_len, p.dtype = a->dtype;
    p.strict = single ? 1 : 0, p.cs_mode = single ? 2 : 0, p.pairwise = a->mimo_rank == 1;
    p.v = a->v, p.bmat = a->b, p.cmat = a->c, p.dsrc = a->da, p.colscale = single ? a->scale : nullptr;
    p.gamma = single ? a->gamma : nullptr, p.h0 = a->h0;
    bp.dy = a->dy, bp.dh_final = a->dh_final, bp.dv = a->dv, bp.db = a->db, bp.dc = a->dc, bp.d_da = a->dda;
    bp.d_cs = single ? a->dscale : nullptr, bp.d_gs = single ? a->dgamma : nullptr, bp.dh0 = a->dh0;
    return exact::run_bwd(bp, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int32_t bm_ssd3_single_bwd(const bm_ssd3_bwd_args* a, void* ws, size_t ws_bytes, void* stream) {
    return ssd3_bwd(a, ws, ws_bytes, stream, true);
}
extern "C" int32_t bm_ssd3_double_bwd(const bm_ssd3_bwd_args* a, void* ws, size_t ws_bytes, void* stream) {
    return ssd3_bwd(a, ws, ws_bytes, stream, false);
}
