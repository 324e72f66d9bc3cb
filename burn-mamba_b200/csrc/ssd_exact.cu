// Exact chunked SSD: K1 chunk cumsum, K3 chunk state, K4 state passing, K5 chunk scan, in float32
// on CUDA cores.  Serves float32 inputs (rel-L2 1e-4 parity), shapes the tensor-core path does not
// cover, and is the on-device cross-check for the tensor-core kernels.
//
// Reference decomposition: src/mamba2/ssd/serial.rs:138-506 (Mamba-2),
// src/mamba3/double_ssd/ssd/serial.rs:118-409 and src/mamba3/single_ssd/ssd/serial.rs:56-268 (Mamba-3).
#include "ssd_exact.cuh"

#include <mutex>

namespace bm {
namespace exact {

constexpr int kThreads = 256;

// One B/C element for (row pointer, r) with the optional data-dependent rotation applied
// (src/modules/misc/rope.rs:50-170): pairwise mode rotates (2j, 2j+1), half mode (j, j + R/2);
// only the first rope_dim entries (pairwise) / first rope_dim/2 of each half rotate.
template <typename T>
__device__ __forceinline__ float bc_elem(const T* row, const float* ang, int r, int R, int rope_dim, int pairwise) {
    float self = to_f32(row[r]);
    if (ang == nullptr || rope_dim == 0) return self;
    if (pairwise) {
        if (r >= rope_dim) return self;
        int j = r >> 1;
        float th = wrap_angle(ang[j]);
        float c = cosf(th), s = sinf(th);
        float other = to_f32(row[r ^ 1]);
        return (r & 1) ? (s * other + c * self) : (c * self - s * other);
    }
    int half = R >> 1, na = rope_dim >> 1;
    if (r < na) {
        float th = wrap_angle(ang[r]);
        return cosf(th) * self - sinf(th) * to_f32(row[r + half]);
    }
    if (r >= half && r < half + na) {
        float th = wrap_angle(ang[r - half]);
        return sinf(th) * to_f32(row[r - half]) + cosf(th) * self;
    }
    return self;
}

// K1: per (b, chunk, h) serial inclusive cumsum of da over the chunk; also records the effective
// source-column scale.  Positions past seqlen behave as dt = 0 padding (src/mamba2/mamba2.rs:703-722).
__global__ void chunk_cumsum_kernel(Params p) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = (int64_t)p.B * p.NC * p.H;
    if (idx >= total) return;
    int h = idx % p.H;
    int n = (idx / p.H) % p.NC;
    int b = idx / ((int64_t)p.H * p.NC);
    float* cum = p.cum + (((int64_t)b * p.H + h) * p.NC + n) * p.Q;
    float* cs = p.cs + (((int64_t)b * p.H + h) * p.NC + n) * p.Q;
    float ah = p.a ? p.a[h] : 1.f;
    float bias = p.dt_bias ? p.dt_bias[h] : 0.f;
    float run = 0.f;
    for (int l = 0; l < p.Q; ++l) {
        int s = n * p.Q + l;
        float da = 0.f, c = 0.f;
        if (s < p.S) {
            int64_t g = ((int64_t)b * p.S + s) * p.H + h;
            float raw = p.dsrc[g];
            if (p.dt_bias) raw = fminf(fmaxf(softplus_f32(raw + bias), p.dt_min), p.dt_max);
            da = raw * ah;
            c = p.cs_mode == 1 ? raw : (p.cs_mode == 2 ? p.colscale[g] : 1.f);
        }
        run += da;
        cum[l] = run;
        cs[l] = c;
    }
}

// K3: S_n[p, r] = sum_j v_j[p] * B_j[r] * cs_t(j) * exp(Aend - cum_t(j)) over the fused (t, m) rows.
template <typename T>
__global__ void chunk_state_kernel(Params p) {
    constexpr int TJ = 16, OPT = 8;
    extern __shared__ float smem[];
    float* vs = smem;             // [TJ][P]
    float* bs = smem + TJ * p.P;  // [TJ][R]
    const int n = blockIdx.x, h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
    const int g = h / (p.H / p.G);
    const float* cum = p.cum + (((int64_t)b * p.H + h) * p.NC + n) * p.Q;
    const float* cs = p.cs + (((int64_t)b * p.H + h) * p.NC + n) * p.Q;
    const float aend = cum[p.Q - 1];
    const int PR = p.P * p.R, QM = p.Q * p.M;
    const T* v = static_cast<const T*>(p.v);
    const T* bm_ = static_cast<const T*>(p.bmat);
    const int na = p.rope_dim >> 1;
    for (int ob = 0; ob < PR; ob += kThreads * OPT) {
        float acc[OPT];
#pragma unroll
        for (int k = 0; k < OPT; ++k) acc[k] = 0.f;
        for (int j0 = 0; j0 < QM; j0 += TJ) {
            __syncthreads();
            for (int e = tid; e < TJ * p.P; e += kThreads) {
                int jj = e / p.P, pp = e % p.P, j = j0 + jj, t = j / p.M, mu = j % p.M, s = n * p.Q + t;
                float val = 0.f;
                if (j < QM && s < p.S) val = to_f32(v[((((int64_t)b * p.S + s) * p.M + mu) * p.H + h) * p.P + pp]);
                vs[e] = val;
            }
            for (int e = tid; e < TJ * p.R; e += kThreads) {
                int jj = e / p.R, rr = e % p.R, j = j0 + jj, t = j / p.M, mu = j % p.M, s = n * p.Q + t;
                float val = 0.f;
                if (j < QM && s < p.S) {
                    const T* row = bm_ + ((((int64_t)b * p.S + s) * p.M + mu) * p.G + g) * p.R;
                    const float* ang = p.angles ? p.angles + (((int64_t)b * p.S + s) * p.H + h) * na : nullptr;
                    val = bc_elem(row, ang, rr, p.R, p.rope_dim, p.pairwise) * cs[t] * expf(aend - cum[t]);
                }
                bs[e] = val;
            }
            __syncthreads();
#pragma unroll
            for (int k = 0; k < OPT; ++k) {
                int o = ob + tid + k * kThreads;
                if (o < PR) {
                    int pp = o / p.R, rr = o % p.R;
                    float a = acc[k];
#pragma unroll
                    for (int jj = 0; jj < TJ; ++jj) a = fmaf(vs[jj * p.P + pp], bs[jj * p.R + rr], a);
                    acc[k] = a;
                }
            }
        }
#pragma unroll
        for (int k = 0; k < OPT; ++k) {
            int o = ob + tid + k * kThreads;
            if (o < PR) p.states[(((int64_t)b * p.NC + n) * p.H + h) * PR + o] = acc[k];
        }
    }
}

// K4: h_{n+1} = exp(Aend_n) h_n + S_n; the buffer of S_n is overwritten with the state entering
// chunk n (src/mamba2/ssd/serial.rs:275-343).
__global__ void state_passing_kernel(Params p) {
    const int PR = p.P * p.R;
    int o = blockIdx.x * blockDim.x + threadIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    if (o >= PR) return;
    float run = p.h0 ? p.h0[((int64_t)b * p.H + h) * PR + o] : 0.f;
    for (int n = 0; n < p.NC; ++n) {
        int64_t idx = (((int64_t)b * p.NC + n) * p.H + h) * PR + o;
        float s = p.states[idx];
        p.states[idx] = run;
        float aend = p.cum[(((int64_t)b * p.H + h) * p.NC + n) * p.Q + p.Q - 1];
        run = fmaf(expf(aend), run, s);
    }
    p.h_final[((int64_t)b * p.H + h) * PR + o] = run;
}

// K5: y_i = exp(cum_t(i)) C_i . h_n + sum_j (C_i . B_j) kern(i, j) v_j (+ D v_i) (* silu(z_i)), with
//   kern(i, j) = exp(cum_t(i) - cum_t(j)) cs_t(j)   for t(j) <  t(i)
//              = cs_t (non-strict) | gamma_t (strict) for t(j) == t(i)
//              = 0                                     for t(j) >  t(i)
// (src/mamba2/ssd/serial.rs:349-506; src/mamba3/single_ssd/ssd/serial.rs:156-268 with the same-step
// term of src/mamba3/single_ssd/ssd/diag.rs:50-100 folded into the same-time block).
template <typename T>
__global__ void chunk_scan_kernel(Params p) {
    constexpr int TI = 32, TJ = 32, RT = 32, PT = 64, OPT = TI * PT / kThreads, WPT = TI * TJ / kThreads;
    __shared__ float Cs[TI][RT + 1];
    __shared__ float Bs[TJ][RT + 1];
    __shared__ float Ws[TI][TJ + 1];
    __shared__ float Vs[TJ][PT + 1];
    const int tid = threadIdx.x;
    const int QM = p.Q * p.M;
    const int ntile = (QM + TI - 1) / TI;
    int64_t bx = blockIdx.x;
    const int it = bx % ntile;
    const int h = (bx / ntile) % p.H;
    const int n = bx / ((int64_t)ntile * p.H);
    const int b = blockIdx.y;
    const int g = h / (p.H / p.G);
    const int i0 = it * TI;
    const int na = p.rope_dim >> 1;
    const float* cum = p.cum + (((int64_t)b * p.H + h) * p.NC + n) * p.Q;
    const float* cs = p.cs + (((int64_t)b * p.H + h) * p.NC + n) * p.Q;
    const T* v = static_cast<const T*>(p.v);
    const T* bm_ = static_cast<const T*>(p.bmat);
    const T* cm = static_cast<const T*>(p.cmat);
    const float* hin = p.states + (((int64_t)b * p.NC + n) * p.H + h) * (int64_t)p.P * p.R;
    const int i_last = min(i0 + TI, QM) - 1;
    const int j_end = min(QM, (i_last / p.M + 1) * p.M);  // columns with t(j) <= t(i_last)

    auto stage_bc = [&](float (*dst)[RT + 1], const T* src, int row0, int r0) {
        for (int e = tid; e < TI * RT; e += kThreads) {
            int ii = e / RT, rr = e % RT, i = row0 + ii, r = r0 + rr;
            int t = i / p.M, mu = i % p.M, s = n * p.Q + t;
            float val = 0.f;
            if (i < QM && s < p.S && r < p.R) {
                const T* row = src + ((((int64_t)b * p.S + s) * p.M + mu) * p.G + g) * p.R;
                const float* ang = p.angles ? p.angles + (((int64_t)b * p.S + s) * p.H + h) * na : nullptr;
                val = bc_elem(row, ang, r, p.R, p.rope_dim, p.pairwise);
            }
            dst[ii][rr] = val;
        }
    };

    for (int p0 = 0; p0 < p.P; p0 += PT) {
        float acc[OPT];
#pragma unroll
        for (int k = 0; k < OPT; ++k) acc[k] = 0.f;
        // ---- state term: sum_r C[i][r] h[p][r]; h tile staged in Vs as [pp][rr] (RT <= PT) ----
        for (int r0 = 0; r0 < p.R; r0 += RT) {
            __syncthreads();
            stage_bc(Cs, cm, i0, r0);
            for (int e = tid; e < PT * RT; e += kThreads) {
                int pp = e / RT, rr = e % RT;
                float val = 0.f;
                if (p0 + pp < p.P && r0 + rr < p.R) val = hin[(int64_t)(p0 + pp) * p.R + r0 + rr];
                Vs[rr][pp] = val;
            }
            __syncthreads();
#pragma unroll
            for (int k = 0; k < OPT; ++k) {
                int o = tid + k * kThreads, ii = o / PT, pp = o % PT;
                float a = acc[k];
#pragma unroll
                for (int rr = 0; rr < RT; ++rr) a = fmaf(Cs[ii][rr], Vs[rr][pp], a);
                acc[k] = a;
            }
        }
#pragma unroll
        for (int k = 0; k < OPT; ++k) {
            int o = tid + k * kThreads, ii = o / PT, i = i0 + ii;
            if (i < QM) acc[k] *= expf(cum[i / p.M]);
        }
        // ---- intra-chunk term ----
        for (int j0 = 0; j0 < j_end; j0 += TJ) {
            float w[WPT];
#pragma unroll
            for (int k = 0; k < WPT; ++k) w[k] = 0.f;
            for (int r0 = 0; r0 < p.R; r0 += RT) {
                __syncthreads();
                stage_bc(Cs, cm, i0, r0);
                stage_bc(Bs, bm_, j0, r0);
                __syncthreads();
#pragma unroll
                for (int k = 0; k < WPT; ++k) {
                    int o = tid + k * kThreads, ii = o / TJ, jj = o % TJ;
                    float a = w[k];
#pragma unroll
                    for (int rr = 0; rr < RT; ++rr) a = fmaf(Cs[ii][rr], Bs[jj][rr], a);
                    w[k] = a;
                }
            }
#pragma unroll
            for (int k = 0; k < WPT; ++k) {
                int o = tid + k * kThreads, ii = o / TJ, jj = o % TJ, i = i0 + ii, j = j0 + jj;
                float kern = 0.f;
                if (i < QM && j < QM) {
                    int ti = i / p.M, tj = j / p.M;
                    if (tj < ti) {
                        kern = expf(cum[ti] - cum[tj]) * cs[tj];
                    } else if (tj == ti) {
                        int s = n * p.Q + ti;
                        if (!p.strict) kern = cs[ti];
                        else if (p.gamma && s < p.S) kern = p.gamma[((int64_t)b * p.S + s) * p.H + h];
                    }
                }
                Ws[ii][jj] = w[k] * kern;
            }
            for (int e = tid; e < TJ * PT; e += kThreads) {
                int jj = e / PT, pp = e % PT, j = j0 + jj, t = j / p.M, mu = j % p.M, s = n * p.Q + t;
                float val = 0.f;
                if (j < QM && s < p.S && p0 + pp < p.P)
                    val = to_f32(v[((((int64_t)b * p.S + s) * p.M + mu) * p.H + h) * p.P + p0 + pp]);
                Vs[jj][pp] = val;
            }
            __syncthreads();
#pragma unroll
            for (int k = 0; k < OPT; ++k) {
                int o = tid + k * kThreads, ii = o / PT, pp = o % PT;
                float a = acc[k];
#pragma unroll
                for (int jj = 0; jj < TJ; ++jj) a = fmaf(Ws[ii][jj], Vs[jj][pp], a);
                acc[k] = a;
            }
        }
        // ---- epilogue: D skip, optional gate, store ----
#pragma unroll
        for (int k = 0; k < OPT; ++k) {
            int o = tid + k * kThreads, ii = o / PT, pp = o % PT, i = i0 + ii;
            int t = i / p.M, mu = i % p.M, s = n * p.Q + t;
            if (i < QM && s < p.S && p0 + pp < p.P) {
                int64_t gi = ((((int64_t)b * p.S + s) * p.M + mu) * p.H + h) * p.P + p0 + pp;
                float out = acc[k];
                if (p.d) out = fmaf(p.d[h], to_f32(v[gi]), out);
                if (p.z) out *= silu_f32(to_f32(static_cast<const T*>(p.z)[gi]));
                static_cast<T*>(p.y)[gi] = from_f32<T>(out);
            }
        }
        __syncthreads();
    }
}

size_t workspace_bytes(int B, int S, int H, int P, int R, int Q, bool need_states) {
    int64_t nc = cdiv(S, Q);
    size_t cum = align_up((size_t)B * H * nc * Q * sizeof(float), 256);
    size_t st = need_states ? align_up((size_t)B * nc * H * P * R * sizeof(float), 256) : 0;
    return 2 * cum + st;
}

template <typename T>
static int32_t launch(Params p, cudaStream_t stream) {
    {
        int64_t total = (int64_t)p.B * p.NC * p.H;
        chunk_cumsum_kernel<<<(unsigned)cdiv(total, 128), 128, 0, stream>>>(p);
        if (int32_t e = check_launch("chunk_cumsum")) return e;
    }
    {
        dim3 grid(p.NC, p.H, p.B);
        size_t smem = (size_t)16 * (p.P + p.R) * sizeof(float);
        chunk_state_kernel<T><<<grid, kThreads, smem, stream>>>(p);
        if (int32_t e = check_launch("chunk_state")) return e;
    }
    {
        dim3 grid((unsigned)cdiv((int64_t)p.P * p.R, kThreads), p.H, p.B);
        state_passing_kernel<<<grid, kThreads, 0, stream>>>(p);
        if (int32_t e = check_launch("state_passing")) return e;
    }
    {
        int64_t ntile = cdiv((int64_t)p.Q * p.M, 32);
        dim3 grid((unsigned)(ntile * p.H * p.NC), p.B);
        chunk_scan_kernel<T><<<grid, kThreads, 0, stream>>>(p);
        if (int32_t e = check_launch("chunk_scan")) return e;
    }
    return BM_OK;
}

int32_t run(Params p, void* workspace, size_t ws_bytes, cudaStream_t stream) {
    p.NC = (int)cdiv(p.S, p.Q);
    const bool need_states = p.states == nullptr;
    size_t need = workspace_bytes(p.B, p.S, p.H, p.P, p.R, p.Q, need_states);
    if (workspace == nullptr || ws_bytes < need)
        return fail(BM_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", ws_bytes, need);
    if (!aligned16(workspace)) return fail(BM_ERR_BAD_ALIGNMENT, "workspace is not 16-byte aligned");
    if ((int64_t)p.P * p.R > 256 * 256 || p.P > 1024 || p.R > 1024)
        return fail(BM_ERR_UNSUPPORTED, "headdim %d x state_rank %d is beyond the exact path's tile limits", p.P, p.R);
    if (p.B > 65535 || p.H > 65535) return fail(BM_ERR_UNSUPPORTED, "batch / nheads above 65535");
    size_t cumb = align_up((size_t)p.B * p.H * p.NC * p.Q * sizeof(float), 256);
    char* w = static_cast<char*>(workspace);
    p.cum = reinterpret_cast<float*>(w);
    p.cs = reinterpret_cast<float*>(w + cumb);
    if (need_states) p.states = reinterpret_cast<float*>(w + 2 * cumb);
    if ((size_t)16 * (p.P + p.R) * sizeof(float) > 48 * 1024)
        return fail(BM_ERR_UNSUPPORTED, "headdim + state_rank too large for the exact path");
    return p.dtype == BM_DTYPE_F32 ? launch<float>(p, stream) : launch<__nv_bfloat16>(p, stream);
}

}  // namespace exact
}  // namespace bm

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the exact Mamba-2 SSD forward.
//
// Some hosts of this library may never allocate device memory once they are running: a serving
// process whose memory budget is fixed and handed out at start-up, a plugin that is given raw tensor
// pointers by its framework but has no handle on that framework's allocator (so it cannot size and
// obtain the workspace bm_ssd2_fwd asks for), or code that runs where cudaMalloc would serialise
// the whole device.  For them the scratch of the exact path lives inside the library image: a
// file-scope device array that every GPU loading the library holds until the process exits.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_noalloc_scratch[BM_SSD2_NOALLOC_SCRATCH_BYTES];

namespace bm {
namespace exact {

// In host code `g_noalloc_scratch` is only a stand-in for the symbol; the address the kernels can
// use comes from cudaGetSymbolAddress, asked once per device with that device current.
static int32_t noalloc_scratch_ptr(void** out) {
    constexpr int kMaxDevices = 64;
    static void* ptrs[kMaxDevices] = {nullptr};
    static std::mutex mu;
    int dev = -1;
    if (int32_t e = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return e;
    if (dev < 0 || dev >= kMaxDevices) return fail(BM_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (ptrs[dev] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return check_cuda(e, "cudaGetSymbolAddress(scratch)");
        if (p == nullptr) return fail(BM_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return BM_OK;
}

int32_t run_noalloc(Params p, cudaStream_t stream) {
    p.NC = (int)cdiv(p.S, p.Q);
    const size_t need = workspace_bytes(p.B, p.S, p.H, p.P, p.R, p.Q, p.states == nullptr);
    if (need > (size_t)BM_SSD2_NOALLOC_SCRATCH_BYTES)
        return fail(BM_ERR_WORKSPACE_TOO_SMALL,
                    "this problem needs %zu bytes of scratch, the built-in scratch holds %zu: use bm_ssd2_fwd with a "
                    "caller-provided workspace",
                    need, (size_t)BM_SSD2_NOALLOC_SCRATCH_BYTES);
    void* scratch = nullptr;
    if (int32_t e = noalloc_scratch_ptr(&scratch)) return e;
    // Nothing in the scratch has to start at zero: K1 writes every cumsum / column-scale entry and K3
    // writes every chunk state before anything reads them, so the previous call's contents are dead.
    return run(p, scratch, (size_t)BM_SSD2_NOALLOC_SCRATCH_BYTES, stream);
}

}  // namespace exact
}  // namespace bm
