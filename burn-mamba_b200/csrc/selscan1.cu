// Mamba-1 selective scan over a sequence (replaces the per-token op loop of
// src/mamba1/mamba1.rs:422-523).  HBM-bound: u, delta, z are read once and y written once.
//
// Work split: one CTA per (batch row, tile of CH channels); a thread owns RPT consecutive states of
// one channel and keeps them in registers for the whole sequence.  Tokens are staged through shared
// memory in chunks of TCH with a two-stage cp.async pipeline, so global traffic is coalesced along
// the channel axis while the recurrence itself runs out of shared memory and registers.
#include "common.cuh"

using namespace bm;

namespace {

constexpr int TCH = 64;   // tokens per staged chunk
constexpr int RPT = 2;    // states per thread
constexpr int TU = 4;     // tokens processed together (independent loads / exps issued ahead of the recurrence)

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// Shared-memory layout of one pipeline stage for CH channels and state rank R (element counts of T):
// delta, u, z as [TCH][CH], then the B and C rows of the chunk as [TCH][R].
template <typename T>
struct StageView {
    T *delta, *u, *z, *bmat, *cmat;
    __device__ StageView(unsigned char* base, int ch, int r) {
        delta = reinterpret_cast<T*>(base);
        u = delta + TCH * ch;
        z = u + TCH * ch;
        bmat = z + TCH * ch;
        cmat = bmat + TCH * r;
    }
};
template <typename T>
__host__ __device__ constexpr size_t stage_bytes(int ch, int r) { return sizeof(T) * (size_t)TCH * (3 * ch + 2 * r); }

// Fast kernel: d_inner % CH == 0, state_rank % RPT == 0, state_rank <= 64, 16-byte-aligned rows.
// CH (channels per CTA) is chosen by the launcher so that the grid fills the machine in one wave.
template <typename T, int CH>
__global__ void selscan1_kernel(bm_selscan1_args a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int R = a.state_rank, I = a.d_inner, S = a.seqlen;
    const size_t sbytes = stage_bytes<T>(CH, R);
    float* ytile = reinterpret_cast<float*>(smem_raw + 2 * sbytes);  // [TCH][CH] pre-gate outputs
    const int tpc = R / RPT;  // threads per channel
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const int cl = tid / tpc, q = tid % tpc;  // channel in tile, state quarter
    const int ntile = I / CH;
    const int b = blockIdx.x / ntile, c0 = (blockIdx.x % ntile) * CH;
    const int ch = c0 + cl;
    constexpr int EPV = 16 / sizeof(T);  // elements per 16-byte vector

    float h[RPT], av[RPT];
#pragma unroll
    for (int k = 0; k < RPT; ++k) {
        av[k] = a.a[(int64_t)ch * R + q * RPT + k];
        h[k] = a.h0 ? a.h0[((int64_t)b * I + ch) * R + q * RPT + k] : 0.f;
    }
    const float dskip = a.d ? a.d[ch] : 0.f;
    const float dbias = (a.delta_softplus && a.delta_bias) ? a.delta_bias[ch] : 0.f;
    const T* ug = static_cast<const T*>(a.u) + (int64_t)b * S * I + c0;
    const T* dg = static_cast<const T*>(a.delta) + (int64_t)b * S * I + c0;
    const T* zg = a.z ? static_cast<const T*>(a.z) + (int64_t)b * S * I + c0 : nullptr;
    const T* bg = static_cast<const T*>(a.b) + (int64_t)b * S * R;
    const T* cg = static_cast<const T*>(a.c) + (int64_t)b * S * R;
    T* yg = static_cast<T*>(a.y) + (int64_t)b * S * I + c0;

    auto issue = [&](int chunk, int stg) {
        const int t0 = chunk * TCH;
        const int nt = min(TCH, S - t0);
        StageView<T> st(smem_raw + stg * sbytes, CH, R);
        constexpr int VPR = CH / EPV;  // vectors per token row
        for (int e = tid; e < nt * VPR; e += nthreads) {
            int t = e / VPR, vv = (e % VPR) * EPV;
            cp_async16(&st.delta[t * CH + vv], dg + (int64_t)(t0 + t) * I + vv);
            cp_async16(&st.u[t * CH + vv], ug + (int64_t)(t0 + t) * I + vv);
            if (zg) cp_async16(&st.z[t * CH + vv], zg + (int64_t)(t0 + t) * I + vv);
        }
        const int bcv = nt * R / EPV;  // B / C rows of a chunk are contiguous in memory
        for (int e = tid; e < bcv; e += nthreads) {
            cp_async16(&st.bmat[e * EPV], bg + (int64_t)t0 * R + e * EPV);
            cp_async16(&st.cmat[e * EPV], cg + (int64_t)t0 * R + e * EPV);
        }
    };

    const int nchunks = (S + TCH - 1) / TCH;
    issue(0, 0);
    cp_async_commit();
    for (int chunk = 0; chunk < nchunks; ++chunk) {
        const int stg = chunk & 1;
        if (chunk + 1 < nchunks) issue(chunk + 1, stg ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        StageView<T> st(smem_raw + stg * sbytes, CH, R);
        const int t0 = chunk * TCH, nt = min(TCH, S - t0);
        // The recurrence only chains through h; everything else of TU tokens (loads, softplus, exp,
        // input term) is issued first so the dependent FMAs of the TU steps run back to back.
        int t = 0;
        for (; t + TU <= nt; t += TU) {
            float dl[TU], uu[TU], ea[TU][RPT], bu[TU][RPT], ck[TU][RPT], part[TU];
#pragma unroll
            for (int j = 0; j < TU; ++j) {
                dl[j] = to_f32(st.delta[(t + j) * CH + cl]);
                if (a.delta_softplus) dl[j] = softplus_stock(dl[j] + dbias);
                uu[j] = to_f32(st.u[(t + j) * CH + cl]);
                const float du = dl[j] * uu[j];
#pragma unroll
                for (int k = 0; k < RPT; ++k) {
                    ea[j][k] = __expf(dl[j] * av[k]);
                    bu[j][k] = du * to_f32(st.bmat[(t + j) * R + q * RPT + k]);
                    ck[j][k] = to_f32(st.cmat[(t + j) * R + q * RPT + k]);
                }
            }
#pragma unroll
            for (int j = 0; j < TU; ++j) {
                part[j] = 0.f;
#pragma unroll
                for (int k = 0; k < RPT; ++k) {
                    h[k] = fmaf(h[k], ea[j][k], bu[j][k]);
                    part[j] = fmaf(h[k], ck[j][k], part[j]);
                }
            }
            for (int o = tpc >> 1; o > 0; o >>= 1) {
#pragma unroll
                for (int j = 0; j < TU; ++j) part[j] += __shfl_xor_sync(0xffffffffu, part[j], o);
            }
            if (q == 0) {
#pragma unroll
                for (int j = 0; j < TU; ++j) ytile[(t + j) * CH + cl] = fmaf(dskip, uu[j], part[j]);
            }
        }
        for (; t < nt; ++t) {
            float delta = to_f32(st.delta[t * CH + cl]);
            if (a.delta_softplus) delta = softplus_stock(delta + dbias);
            const float u = to_f32(st.u[t * CH + cl]);
            const float du = delta * u;
            float part = 0.f;
#pragma unroll
            for (int k = 0; k < RPT; ++k) {
                const float bk = to_f32(st.bmat[t * R + q * RPT + k]);
                const float ckk = to_f32(st.cmat[t * R + q * RPT + k]);
                h[k] = fmaf(h[k], __expf(delta * av[k]), du * bk);
                part = fmaf(h[k], ckk, part);
            }
            for (int o = tpc >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            if (q == 0) ytile[t * CH + cl] = fmaf(dskip, u, part);
        }
        __syncthreads();
        // gate and store: every thread handles one 16-byte vector of outputs (coalesced along channels)
        constexpr int VPR = CH / EPV;
        for (int e = tid; e < nt * VPR; e += nthreads) {
            const int tt = e / VPR, vv = (e % VPR) * EPV;
            alignas(16) T outv[EPV];
#pragma unroll
            for (int j = 0; j < EPV; ++j) {
                float y = ytile[tt * CH + vv + j];
                if (zg) y *= silu_f32(to_f32(st.z[tt * CH + vv + j]));
                outv[j] = from_f32<T>(y);
            }
            *reinterpret_cast<uint4*>(yg + (int64_t)(t0 + tt) * I + vv) = *reinterpret_cast<const uint4*>(outv);
        }
        // stage `stg` and ytile are refilled in the next iteration: every thread must be done reading them
        __syncthreads();
    }
#pragma unroll
    for (int k = 0; k < RPT; ++k) a.h_final[((int64_t)b * I + ch) * R + q * RPT + k] = h[k];
}

// Generic kernel: any d_inner / state_rank; one thread per (b, i) channel, states in local memory
// when state_rank is large.  Correct for every shape; used when the fast kernel's tiling does not fit.
template <typename T>
__global__ void selscan1_generic_kernel(bm_selscan1_args a) {
    constexpr int RMAX = 256;
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int I = a.d_inner, R = a.state_rank, S = a.seqlen;
    if (idx >= (int64_t)a.batch * I) return;
    const int i = idx % I, b = idx / I;
    float h[RMAX];
    for (int r = 0; r < R; ++r) h[r] = a.h0 ? a.h0[idx * R + r] : 0.f;
    const float* arow = a.a + (int64_t)i * R;
    const float dskip = a.d ? a.d[i] : 0.f;
    const float dbias = (a.delta_softplus && a.delta_bias) ? a.delta_bias[i] : 0.f;
    for (int t = 0; t < S; ++t) {
        int64_t gi = ((int64_t)b * S + t) * I + i;
        float delta = to_f32(static_cast<const T*>(a.delta)[gi]);
        if (a.delta_softplus) delta = softplus_stock(delta + dbias);
        const float u = to_f32(static_cast<const T*>(a.u)[gi]);
        const T* bv = static_cast<const T*>(a.b) + ((int64_t)b * S + t) * R;
        const T* cv = static_cast<const T*>(a.c) + ((int64_t)b * S + t) * R;
        float part = 0.f;
        for (int r = 0; r < R; ++r) {
            h[r] = fmaf(h[r], expf(delta * arow[r]), delta * u * to_f32(bv[r]));
            part = fmaf(h[r], to_f32(cv[r]), part);
        }
        float y = fmaf(dskip, u, part);
        if (a.z) y *= silu_f32(to_f32(static_cast<const T*>(a.z)[gi]));
        static_cast<T*>(a.y)[gi] = from_f32<T>(y);
    }
    for (int r = 0; r < R; ++r) a.h_final[idx * R + r] = h[r];
}

template <typename T>
int32_t launch(const bm_selscan1_args& a, cudaStream_t st) {
    const int R = a.state_rank, I = a.d_inner;
    const int tpc = R / RPT;
    const bool pow2 = tpc > 0 && (tpc & (tpc - 1)) == 0;
    constexpr int EPV = 16 / sizeof(T);
    const bool fast = I % 32 == 0 && R % RPT == 0 && R <= 64 && pow2 && tpc <= 32 && (R % EPV == 0);
    if (fast) {
        // 16 channels per CTA unless 32 already give every SM several CTAs: the sequence is walked serially,
        // so the only parallelism is across CTAs and a second, partly filled wave doubles the run time
        const bool wide = (int64_t)a.batch * (I / 32) >= 4 * 148;
        const int ch = wide ? 32 : 16;
        size_t smem = 2 * stage_bytes<T>(ch, R) + sizeof(float) * TCH * ch;
        auto kern = wide ? selscan1_kernel<T, 32> : selscan1_kernel<T, 16>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(selscan1)");
        unsigned grid = (unsigned)((int64_t)a.batch * (I / ch));
        kern<<<grid, ch * tpc, smem, st>>>(a);
        return check_launch("selscan1");
    }
    if (R > 256) return fail(BM_ERR_UNSUPPORTED, "state_rank %d above 256", R);
    int64_t total = (int64_t)a.batch * I;
    selscan1_generic_kernel<T><<<(unsigned)cdiv(total, 64), 64, 0, st>>>(a);
    return check_launch("selscan1_generic");
}

}  // namespace

namespace bm {
int32_t validate_selscan1(const bm_selscan1_args* a) {
    if (a == nullptr) return fail(BM_ERR_NULL_POINTER, "args is NULL");
    BM_REQUIRE(a->batch > 0 && a->seqlen > 0 && a->d_inner > 0 && a->state_rank > 0, BM_ERR_BAD_SHAPE,
               "batch, seqlen, d_inner, state_rank must be positive");
    BM_REQUIRE(a->dtype == BM_DTYPE_F32 || a->dtype == BM_DTYPE_BF16, BM_ERR_UNSUPPORTED, "dtype must be f32 or bf16");
    BM_REQUIRE_PTR(a->u);
    BM_REQUIRE_PTR(a->delta);
    BM_REQUIRE_PTR(a->a);
    BM_REQUIRE_PTR(a->b);
    BM_REQUIRE_PTR(a->c);
    BM_REQUIRE_PTR(a->y);
    BM_REQUIRE_PTR(a->h_final);
    BM_OPTIONAL_PTR(a->d);
    BM_OPTIONAL_PTR(a->delta_bias);
    BM_OPTIONAL_PTR(a->z);
    BM_OPTIONAL_PTR(a->h0);
    return BM_OK;
}
}  // namespace bm

extern "C" int32_t bm_selscan1_fwd(const bm_selscan1_args* a, void* stream) {
    clear_error();
    if (int32_t e = validate_selscan1(a)) return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return a->dtype == BM_DTYPE_F32 ? launch<float>(*a, st) : launch<__nv_bfloat16>(*a, st);
}
