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
        if (p.gs) {
            // same-time weight: column scale (non-strict cores) or gamma (strict core)
            float g = c;
            if (p.strict) g = (p.gamma && s < p.S) ? p.gamma[((int64_t)b * p.S + s) * p.H + h] : 0.f;
            p.gs[(((int64_t)b * p.H + h) * p.NC + n) * p.Q + l] = g;
        }
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
                    const float wgt = p.state_weight_mode == 0 ? cs[t] * expf(aend - cum[t]) : expf(cum[t]);
                    val = bc_elem(row, ang, rr, p.R, p.rope_dim, p.pairwise) * wgt;
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

// =============================================================================================
// Backward of the general chunked SSD (float32, CUDA cores).
//
// Follows the structure of the reference's recompute backward
// (src/mamba2/ssd/serial_recalculated/combined_backward.rs:126-590,
//  src/mamba3/single_ssd/ssd/serial_recalculated/combined_backward.rs:74-536): K1-K4 are recomputed
// from the saved inputs; the chunk-scan gradient splits into the state-readout term ("BLUE"), the
// intra-chunk term ("ORANGE" / lower + same-step), the state-passing recurrence run in reverse, and the
// chunk-state term; the cumulative-decay gradient is a suffix sum inside each chunk.
// With W = CB * kern, kern(i, j) = exp(cum_ti - cum_tj) cs_tj (t_j < t_i) | gs_t (t_j == t_i):
//   dW = dy v^T        dCB = dW * kern       dkern = dW * CB
//   dv_j = sum_i W_ij dy_i + w_j dS B_j (+ D dy_j)          w_j = cs_tj exp(Aend - cum_tj)
//   dB_j = sum_i dCB_ij C_i + w_j dS^T v_j
//   dC_i = sum_j dCB_ij B_j + e_i h_n^T dy_i                e_i = exp(cum_ti)
//   dh_n = exp(Aend_n) dh_{n+1} + sum_i e_i dy_i (x) C_i ,  dS_n = dh_{n+1}
//   dcum, dcs, dgs, dAend collect the scalar terms; d_da = suffix sum of dcum within the chunk.
// =============================================================================================
namespace bm {
namespace exact {

constexpr int BT = 32;  // fused rows / columns per backward tile

struct BwdWork {
    float* gs;        // [b, h, nc, Q] same-time weights
    float* dstates;   // [b, nc, h, p, r]: readout gradient G_n, overwritten with dS_n by the reverse pass
    float* dcum;      // [b, h, nc, Q] accumulators (zeroed)
    float* dcs;       // [b, h, nc, Q]
    float* dgs;       // [b, h, nc, Q]
    float* daend;     // [b, h, nc]
};

// Reverse state passing: dS_n = dh_{n+1}; dh_n = exp(Aend_n) dh_{n+1} + G_n; dAend_n += <dh_{n+1}, exp(Aend_n) h_n>.
__global__ void bwd_state_passing_kernel(Params p, BwdWork w, const float* dh_final, float* dh0) {
    const int PR = p.P * p.R;
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    __shared__ float red[32];
    float dh = (o < PR && dh_final) ? dh_final[((int64_t)b * p.H + h) * PR + o] : 0.f;
    for (int n = p.NC - 1; n >= 0; --n) {
        const int64_t idx = (((int64_t)b * p.NC + n) * p.H + h) * PR + o;
        const float e = expf(p.cum[(((int64_t)b * p.H + h) * p.NC + n) * p.Q + p.Q - 1]);
        float g = 0.f, part = 0.f;
        if (o < PR) {
            g = w.dstates[idx];
            w.dstates[idx] = dh;
            part = dh * e * p.states[idx];
        }
        // block reduction of the dAend contribution
        for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
        __syncthreads();
        if (threadIdx.x < 32) {
            float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (threadIdx.x == 0) atomicAdd(&w.daend[((int64_t)b * p.H + h) * p.NC + n], v);
        }
        __syncthreads();
        dh = fmaf(e, dh, g);
    }
    if (o < PR) dh0[((int64_t)b * p.H + h) * PR + o] = dh;
}

// Shared-memory view used by the two tile kernels.
struct BwdTiles {
    float *dyI, *vJ, *cI, *bJ;   // [BT][P+1], [BT][P+1], [BT][R+1], [BT][R+1]
    float *Ws, *dCBs, *dKs, *Ks; // [BT][BT+1] each
    float* big;                  // [P][R] (dS_n or h_n)
    float* sc;                   // 4 x BT scalars
};
__device__ __forceinline__ BwdTiles carve_tiles(float* sm, int P, int R) {
    BwdTiles t;
    t.dyI = sm; sm += BT * (P + 1);
    t.vJ = sm; sm += BT * (P + 1);
    t.cI = sm; sm += BT * (R + 1);
    t.bJ = sm; sm += BT * (R + 1);
    t.Ws = sm; sm += BT * (BT + 1);
    t.dCBs = sm; sm += BT * (BT + 1);
    t.dKs = sm; sm += BT * (BT + 1);
    t.Ks = sm; sm += BT * (BT + 1);
    t.sc = sm; sm += 4 * BT;
    t.big = sm;
    return t;
}
static size_t bwd_smem_bytes(int P, int R) {
    return sizeof(float) * (size_t)(2 * BT * (P + 1) + 2 * BT * (R + 1) + 4 * BT * (BT + 1) + 4 * BT + P * R);
}

template <typename T>
__device__ __forceinline__ void stage_rows(float* dst, int ld, const T* src, const Params& p, int b, int n, int h_or_g, int HG,
                                           int width, int row0, int tid) {
    // rows = fused indices row0 .. row0 + BT of chunk n; src layout [b, s, m, HG, width]
    const int QM = p.Q * p.M;
    for (int e = tid; e < BT * width; e += kThreads) {
        const int ii = e / width, x = e % width, i = row0 + ii, t = i / p.M, mu = i % p.M, s = n * p.Q + t;
        float val = 0.f;
        if (i < QM && s < p.S) val = to_f32(src[((((int64_t)b * p.S + s) * p.M + mu) * HG + h_or_g) * width + x]);
        dst[ii * ld + x] = val;
    }
}

// dW, CB, kern for the (I, J) block -> Ws = CB*kern, dCBs = dW*kern, dKs = dW*CB, Ks = kern (0 where masked).
__device__ __forceinline__ void block_products(const BwdTiles& t, const Params& p, const float* cum, const float* cs,
                                               const float* gs, int i0, int j0, int tid) {
    const int QM = p.Q * p.M;
#pragma unroll
    for (int k = 0; k < BT * BT / kThreads; ++k) {
        const int o = tid + k * kThreads, ii = o / BT, jj = o % BT, i = i0 + ii, j = j0 + jj;
        float dw = 0.f, cb = 0.f;
        for (int x = 0; x < p.P; ++x) dw = fmaf(t.dyI[ii * (p.P + 1) + x], t.vJ[jj * (p.P + 1) + x], dw);
        for (int x = 0; x < p.R; ++x) cb = fmaf(t.cI[ii * (p.R + 1) + x], t.bJ[jj * (p.R + 1) + x], cb);
        float kern = 0.f;
        if (i < QM && j < QM) {
            const int ti = i / p.M, tj = j / p.M;
            if (tj < ti) kern = expf(cum[ti] - cum[tj]) * cs[tj];
            else if (tj == ti) kern = gs[ti];
        }
        t.Ws[ii * (BT + 1) + jj] = cb * kern;
        t.dCBs[ii * (BT + 1) + jj] = dw * kern;
        t.dKs[ii * (BT + 1) + jj] = dw * cb;
        t.Ks[ii * (BT + 1) + jj] = kern;
    }
}

// Column-tile kernel: everything that is a sum over target rows i for a tile J of source columns:
// dv_J, dB_J, and the column-indexed scalar gradients (dcs, the negative half of dcum, dgs, dAend).
template <typename T>
__global__ void bwd_columns_kernel(Params p, BwdWork w, const T* dy, float* dv, float* db, float* dd) {
    extern __shared__ float sm[];
    BwdTiles t = carve_tiles(sm, p.P, p.R);
    const int tid = threadIdx.x;
    const int QM = p.Q * p.M, ntile = (QM + BT - 1) / BT;
    int64_t bx = blockIdx.x;
    const int jt = bx % ntile, h = (bx / ntile) % p.H, n = bx / ((int64_t)ntile * p.H), b = blockIdx.y;
    const int hpg = p.H / p.G, g = h / hpg, j0 = jt * BT;
    const int64_t cbase = (((int64_t)b * p.H + h) * p.NC + n) * p.Q;
    const float *cum = p.cum + cbase, *cs = p.cs + cbase, *gs = w.gs + cbase;
    const float aend = cum[p.Q - 1];
    const T* v = static_cast<const T*>(p.v);
    const T* bm_ = static_cast<const T*>(p.bmat);
    const T* cm = static_cast<const T*>(p.cmat);
    float* colacc = t.sc;  // [0..BT) dcs, [BT..2BT) -dcum, [2BT..3BT) dgs, [3BT..4BT) dw
    for (int e = tid; e < 4 * BT; e += kThreads) colacc[e] = 0.f;
    stage_rows(t.vJ, p.P + 1, v, p, b, n, h, p.H, p.P, j0, tid);
    stage_rows(t.bJ, p.R + 1, bm_, p, b, n, g, p.G, p.R, j0, tid);
    constexpr int MAXV = 16, MAXB = 32;  // per-thread outputs: BT*P/256 <= 16 (P <= 128), BT*R/256 <= 32 (R <= 256)
    float acc_v[MAXV], acc_b[MAXB];
#pragma unroll
    for (int k = 0; k < MAXV; ++k) acc_v[k] = 0.f;
#pragma unroll
    for (int k = 0; k < MAXB; ++k) acc_b[k] = 0.f;
    const int nv = BT * p.P, nb = BT * p.R;
    // target rows with t_i >= t_j: start at the tile holding the first fused index of time t(j0)
    // (a time step's M rows may straddle a tile boundary when M does not divide the tile size)
    for (int it = ((j0 / p.M) * p.M) / BT; it < ntile; ++it) {
        const int i0 = it * BT;
        __syncthreads();
        stage_rows(t.dyI, p.P + 1, dy, p, b, n, h, p.H, p.P, i0, tid);
        stage_rows(t.cI, p.R + 1, cm, p, b, n, g, p.G, p.R, i0, tid);
        __syncthreads();
        block_products(t, p, cum, cs, gs, i0, j0, tid);
        __syncthreads();
        // column scalars
        for (int e = tid; e < BT * BT; e += kThreads) {
            const int ii = e / BT, jj = e % BT, i = i0 + ii, j = j0 + jj;
            if (i < QM && j < QM) {
                const int ti = i / p.M, tj = j / p.M;
                const float dk = t.dKs[ii * (BT + 1) + jj];
                if (tj < ti) {
                    atomicAdd(&colacc[jj], dk * expf(cum[ti] - cum[tj]));
                    atomicAdd(&colacc[BT + jj], dk * t.Ks[ii * (BT + 1) + jj]);
                } else if (tj == ti) {
                    atomicAdd(&colacc[2 * BT + jj], dk);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int o = tid + k * kThreads;
            if (o < nv) {
                const int jj = o / p.P, x = o % p.P;
                float a = acc_v[k];
                for (int ii = 0; ii < BT; ++ii) a = fmaf(t.Ws[ii * (BT + 1) + jj], t.dyI[ii * (p.P + 1) + x], a);
                acc_v[k] = a;
            }
        }
#pragma unroll
        for (int k = 0; k < MAXB; ++k) {
            const int o = tid + k * kThreads;
            if (o < nb) {
                const int jj = o / p.R, x = o % p.R;
                float a = acc_b[k];
                for (int ii = 0; ii < BT; ++ii) a = fmaf(t.dCBs[ii * (BT + 1) + jj], t.cI[ii * (p.R + 1) + x], a);
                acc_b[k] = a;
            }
        }
    }
    // ---- chunk-state term: dS_n = dh_{n+1}
    __syncthreads();
    const float* dS = w.dstates + (((int64_t)b * p.NC + n) * p.H + h) * (int64_t)p.P * p.R;
    for (int e = tid; e < p.P * p.R; e += kThreads) t.big[e] = dS[e];
    // dy of the J tile for the skip term (reuses the dyI buffer)
    stage_rows(t.dyI, p.P + 1, dy, p, b, n, h, p.H, p.P, j0, tid);
    __syncthreads();
    float dd_part = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
        const int o = tid + k * kThreads;
        if (o < nv) {
            const int jj = o / p.P, x = o % p.P, j = j0 + jj, tj = j / p.M;
            const float wj = j < QM ? cs[tj] * expf(aend - cum[tj]) : 0.f;
            float t1 = 0.f;
            for (int r = 0; r < p.R; ++r) t1 = fmaf(t.big[x * p.R + r], t.bJ[jj * (p.R + 1) + r], t1);
            acc_v[k] = fmaf(wj, t1, acc_v[k]);
            atomicAdd(&colacc[3 * BT + jj], t.vJ[jj * (p.P + 1) + x] * t1);   // dw_j = v_j^T dS B_j
            const float dyv = t.dyI[jj * (p.P + 1) + x];
            if (p.d) {
                acc_v[k] = fmaf(p.d[h], dyv, acc_v[k]);
                dd_part = fmaf(dyv, t.vJ[jj * (p.P + 1) + x], dd_part);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < MAXB; ++k) {
        const int o = tid + k * kThreads;
        if (o < nb) {
            const int jj = o / p.R, x = o % p.R, j = j0 + jj, tj = j / p.M;
            const float wj = j < QM ? cs[tj] * expf(aend - cum[tj]) : 0.f;
            float t2 = 0.f;
            for (int pp = 0; pp < p.P; ++pp) t2 = fmaf(t.big[pp * p.R + x], t.vJ[jj * (p.P + 1) + pp], t2);
            acc_b[k] = fmaf(wj, t2, acc_b[k]);
        }
    }
    if (p.d && dd) {
        for (int off = 16; off > 0; off >>= 1) dd_part += __shfl_xor_sync(0xffffffffu, dd_part, off);
        if ((tid & 31) == 0) atomicAdd(&dd[h], dd_part);
    }
    __syncthreads();
    // ---- outputs
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
        const int o = tid + k * kThreads;
        if (o < nv) {
            const int jj = o / p.P, x = o % p.P, j = j0 + jj, tj = j / p.M, mu = j % p.M, s = n * p.Q + tj;
            if (j < QM && s < p.S) dv[((((int64_t)b * p.S + s) * p.M + mu) * p.H + h) * p.P + x] = acc_v[k];
        }
    }
#pragma unroll
    for (int k = 0; k < MAXB; ++k) {
        const int o = tid + k * kThreads;
        if (o < nb) {
            const int jj = o / p.R, x = o % p.R, j = j0 + jj, tj = j / p.M, mu = j % p.M, s = n * p.Q + tj;
            if (j < QM && s < p.S) {
                float* dst = db + ((((int64_t)b * p.S + s) * p.M + mu) * p.G + g) * p.R + x;
                if (hpg > 1) atomicAdd(dst, acc_b[k]); else *dst = acc_b[k];
            }
        }
    }
    for (int jj = tid; jj < BT; jj += kThreads) {
        const int j = j0 + jj;
        if (j < QM) {
            const int tj = j / p.M;
            const float e_end = expf(aend - cum[tj]), wj = cs[tj] * e_end, dw = colacc[3 * BT + jj];
            atomicAdd(&w.dcs[cbase + tj], colacc[jj] + dw * e_end);
            atomicAdd(&w.dcum[cbase + tj], -(colacc[BT + jj] + dw * wj));
            atomicAdd(&w.dgs[cbase + tj], colacc[2 * BT + jj]);
            atomicAdd(&w.daend[((int64_t)b * p.H + h) * p.NC + n], dw * wj);
        }
    }
}

// Row-tile kernel: everything that is a sum over source columns j for a tile I of target rows:
// dC_I and the positive half of dcum (intra-chunk term and state-readout term).
template <typename T>
__global__ void bwd_rows_kernel(Params p, BwdWork w, const T* dy, float* dc) {
    extern __shared__ float sm[];
    BwdTiles t = carve_tiles(sm, p.P, p.R);
    const int tid = threadIdx.x;
    const int QM = p.Q * p.M, ntile = (QM + BT - 1) / BT;
    int64_t bx = blockIdx.x;
    const int it = bx % ntile, h = (bx / ntile) % p.H, n = bx / ((int64_t)ntile * p.H), b = blockIdx.y;
    const int hpg = p.H / p.G, g = h / hpg, i0 = it * BT;
    const int64_t cbase = (((int64_t)b * p.H + h) * p.NC + n) * p.Q;
    const float *cum = p.cum + cbase, *cs = p.cs + cbase, *gs = w.gs + cbase;
    const T* v = static_cast<const T*>(p.v);
    const T* bm_ = static_cast<const T*>(p.bmat);
    const T* cm = static_cast<const T*>(p.cmat);
    float* rowacc = t.sc;  // [0..BT) +dcum
    for (int e = tid; e < 4 * BT; e += kThreads) rowacc[e] = 0.f;
    stage_rows(t.dyI, p.P + 1, dy, p, b, n, h, p.H, p.P, i0, tid);
    stage_rows(t.cI, p.R + 1, cm, p, b, n, g, p.G, p.R, i0, tid);
    constexpr int MAXC = 32;
    float acc_c[MAXC];
#pragma unroll
    for (int k = 0; k < MAXC; ++k) acc_c[k] = 0.f;
    const int nc_out = BT * p.R;
    // source columns with t_j <= t_i: up to the tile holding the last fused index of time t(i_last)
    const int i_last = min(i0 + BT, QM) - 1;
    const int jt_end = min(ntile - 1, (((i_last / p.M) + 1) * p.M - 1) / BT);
    for (int jt = 0; jt <= jt_end; ++jt) {
        const int j0 = jt * BT;
        __syncthreads();
        stage_rows(t.vJ, p.P + 1, v, p, b, n, h, p.H, p.P, j0, tid);
        stage_rows(t.bJ, p.R + 1, bm_, p, b, n, g, p.G, p.R, j0, tid);
        __syncthreads();
        block_products(t, p, cum, cs, gs, i0, j0, tid);
        __syncthreads();
        for (int e = tid; e < BT * BT; e += kThreads) {
            const int ii = e / BT, jj = e % BT, i = i0 + ii, j = j0 + jj;
            if (i < QM && j < QM && j / p.M < i / p.M)
                atomicAdd(&rowacc[ii], t.dKs[ii * (BT + 1) + jj] * t.Ks[ii * (BT + 1) + jj]);
        }
#pragma unroll
        for (int k = 0; k < MAXC; ++k) {
            const int o = tid + k * kThreads;
            if (o < nc_out) {
                const int ii = o / p.R, x = o % p.R;
                float a = acc_c[k];
                for (int jj = 0; jj < BT; ++jj) a = fmaf(t.dCBs[ii * (BT + 1) + jj], t.bJ[jj * (p.R + 1) + x], a);
                acc_c[k] = a;
            }
        }
    }
    // ---- state-readout term: dC_i += e_i h_n^T dy_i ; dcum_ti += C_i . (that)
    __syncthreads();
    const float* hin = p.states + (((int64_t)b * p.NC + n) * p.H + h) * (int64_t)p.P * p.R;
    for (int e = tid; e < p.P * p.R; e += kThreads) t.big[e] = hin[e];
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MAXC; ++k) {
        const int o = tid + k * kThreads;
        if (o < nc_out) {
            const int ii = o / p.R, x = o % p.R, i = i0 + ii;
            if (i < QM) {
                const float ei = expf(cum[i / p.M]);
                float t3 = 0.f;
                for (int pp = 0; pp < p.P; ++pp) t3 = fmaf(t.dyI[ii * (p.P + 1) + pp], t.big[pp * p.R + x], t3);
                t3 *= ei;
                acc_c[k] += t3;
                atomicAdd(&rowacc[ii], t.cI[ii * (p.R + 1) + x] * t3);
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MAXC; ++k) {
        const int o = tid + k * kThreads;
        if (o < nc_out) {
            const int ii = o / p.R, x = o % p.R, i = i0 + ii, ti = i / p.M, mu = i % p.M, s = n * p.Q + ti;
            if (i < QM && s < p.S) {
                float* dst = dc + ((((int64_t)b * p.S + s) * p.M + mu) * p.G + g) * p.R + x;
                if (hpg > 1) atomicAdd(dst, acc_c[k]); else *dst = acc_c[k];
            }
        }
    }
    for (int ii = tid; ii < BT; ii += kThreads) {
        const int i = i0 + ii;
        if (i < QM) atomicAdd(&w.dcum[cbase + i / p.M], rowacc[ii]);
    }
}

// Finalise: dcum[Q-1] += dAend; d_da = suffix sum of dcum over the chunk; scatter to [b, s, h] outputs.
__global__ void bwd_finalize_kernel(Params p, BwdWork w, float* d_da, float* d_cs, float* d_gs, float* d_dt, float* d_a) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t total = (int64_t)p.B * p.NC * p.H;
    if (idx >= total) return;
    const int h = idx % p.H, n = (idx / p.H) % p.NC, b = idx / ((int64_t)p.H * p.NC);
    const int64_t cbase = (((int64_t)b * p.H + h) * p.NC + n) * p.Q;
    float run = w.daend[((int64_t)b * p.H + h) * p.NC + n];
    float da_acc = 0.f;
    for (int l = p.Q - 1; l >= 0; --l) {
        run += w.dcum[cbase + l];
        const int s = n * p.Q + l;
        if (s < p.S) {
            const int64_t g = ((int64_t)b * p.S + s) * p.H + h;
            if (d_da) d_da[g] = run;
            if (d_cs) d_cs[g] = w.dcs[cbase + l];
            if (d_gs) d_gs[g] = w.dgs[cbase + l];
            if (d_dt) {   // Mamba-2: da = dt * A_h, cs = gs = dt
                const float dt = p.dsrc[g];
                d_dt[g] = run * p.a[h] + w.dcs[cbase + l] + w.dgs[cbase + l];
                da_acc = fmaf(run, dt, da_acc);
            }
        }
    }
    if (d_a) atomicAdd(&d_a[h], da_acc);
}

size_t bwd_workspace_bytes(int B, int S, int H, int P, int R, int Q, bool mamba2) {
    const int64_t nc = cdiv(S, Q);
    const size_t per = align_up((size_t)B * H * nc * Q * sizeof(float), 256);
    const size_t st = align_up((size_t)B * nc * H * P * R * sizeof(float), 256);
    const size_t fin = align_up((size_t)B * H * P * R * sizeof(float), 256);
    const size_t ae = align_up((size_t)B * H * nc * sizeof(float), 256);
    const size_t outs = mamba2 ? align_up((size_t)B * S * H * sizeof(float), 256) : 0;  // internal d_da of Mamba-2
    return 6 * per + 2 * st + fin + ae + outs;
}

template <typename T>
static int32_t launch_bwd(BwdParams bp, BwdWork w, cudaStream_t stream) {
    Params& p = bp.fwd;
    const T* dy = static_cast<const T*>(bp.dy);
    const size_t smem = bwd_smem_bytes(p.P, p.R);
    cudaError_t e = cudaFuncSetAttribute(bwd_columns_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(bwd_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(bwd)");
    {   // recompute K1 (with same-time weights), K3, K4
        int64_t total = (int64_t)p.B * p.NC * p.H;
        chunk_cumsum_kernel<<<(unsigned)cdiv(total, 128), 128, 0, stream>>>(p);
        if (int32_t er = check_launch("chunk_cumsum")) return er;
        dim3 grid(p.NC, p.H, p.B);
        size_t sm3 = (size_t)16 * (p.P + p.R) * sizeof(float);
        chunk_state_kernel<T><<<grid, kThreads, sm3, stream>>>(p);
        if (int32_t er = check_launch("chunk_state")) return er;
        dim3 grid4((unsigned)cdiv((int64_t)p.P * p.R, kThreads), p.H, p.B);
        state_passing_kernel<<<grid4, kThreads, 0, stream>>>(p);
        if (int32_t er = check_launch("state_passing")) return er;
        // readout gradient G_n = sum_i exp(cum_ti) dy_i (x) C_i : the K3 kernel with dy / C / exp(cum) weights
        Params q = p;
        q.v = bp.dy, q.bmat = p.cmat, q.states = w.dstates, q.state_weight_mode = 1, q.angles = nullptr;
        chunk_state_kernel<T><<<grid, kThreads, sm3, stream>>>(q);
        if (int32_t er = check_launch("chunk_state(readout gradient)")) return er;
        bwd_state_passing_kernel<<<grid4, kThreads, 0, stream>>>(p, w, bp.dh_final, bp.dh0);
        if (int32_t er = check_launch("bwd_state_passing")) return er;
    }
    const int64_t ntile = cdiv((int64_t)p.Q * p.M, BT);
    dim3 grid((unsigned)(ntile * p.H * p.NC), p.B);
    bwd_columns_kernel<T><<<grid, kThreads, smem, stream>>>(p, w, dy, bp.dv, bp.db, bp.dd);
    if (int32_t er = check_launch("bwd_columns")) return er;
    bwd_rows_kernel<T><<<grid, kThreads, smem, stream>>>(p, w, dy, bp.dc);
    if (int32_t er = check_launch("bwd_rows")) return er;
    int64_t total = (int64_t)p.B * p.NC * p.H;
    bwd_finalize_kernel<<<(unsigned)cdiv(total, 128), 128, 0, stream>>>(p, w, bp.d_da, bp.d_cs, bp.d_gs, bp.d_dt, bp.d_a);
    return check_launch("bwd_finalize");
}

int32_t run_bwd(BwdParams bp, void* workspace, size_t ws_bytes, cudaStream_t stream) {
    Params& p = bp.fwd;
    p.NC = (int)cdiv(p.S, p.Q);
    const bool mamba2 = bp.d_dt != nullptr;
    const size_t need = bwd_workspace_bytes(p.B, p.S, p.H, p.P, p.R, p.Q, mamba2);
    if (workspace == nullptr || ws_bytes < need)
        return fail(BM_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", ws_bytes, need);
    if (!aligned16(workspace)) return fail(BM_ERR_BAD_ALIGNMENT, "workspace is not 16-byte aligned");
    if (p.P > 128 || p.R > 256) return fail(BM_ERR_UNSUPPORTED, "backward supports headdim <= 128 and state_rank <= 256");
    if (bwd_smem_bytes(p.P, p.R) > 200 * 1024) return fail(BM_ERR_UNSUPPORTED, "headdim x state_rank too large for the backward tiles");
    if (p.B > 65535 || p.H > 65535) return fail(BM_ERR_UNSUPPORTED, "batch / nheads above 65535");
    const size_t per = align_up((size_t)p.B * p.H * p.NC * p.Q * sizeof(float), 256);
    const size_t st = align_up((size_t)p.B * p.NC * p.H * p.P * p.R * sizeof(float), 256);
    const size_t fin = align_up((size_t)p.B * p.H * p.P * p.R * sizeof(float), 256);
    const size_t ae = align_up((size_t)p.B * p.H * p.NC * sizeof(float), 256);
    char* wp = static_cast<char*>(workspace);
    BwdWork w;
    p.cum = reinterpret_cast<float*>(wp); wp += per;
    p.cs = reinterpret_cast<float*>(wp); wp += per;
    w.gs = reinterpret_cast<float*>(wp); wp += per;
    p.gs = w.gs;
    // accumulators, contiguous so that one memset clears them
    char* zero_begin = wp;
    w.dcum = reinterpret_cast<float*>(wp); wp += per;
    w.dcs = reinterpret_cast<float*>(wp); wp += per;
    w.dgs = reinterpret_cast<float*>(wp); wp += per;
    w.daend = reinterpret_cast<float*>(wp); wp += ae;
    const size_t zero_bytes = (size_t)(wp - zero_begin);
    p.states = reinterpret_cast<float*>(wp); wp += st;
    w.dstates = reinterpret_cast<float*>(wp); wp += st;
    p.h_final = reinterpret_cast<float*>(wp); wp += fin;
    if (mamba2 && bp.d_da == nullptr) bp.d_da = reinterpret_cast<float*>(wp);
    p.state_weight_mode = 0;
    if (int32_t e = check_cuda(cudaMemsetAsync(zero_begin, 0, zero_bytes, stream), "cudaMemsetAsync(accumulators)")) return e;
    const size_t bc_bytes = (size_t)p.B * p.S * p.M * p.G * p.R * sizeof(float);
    if (p.H / p.G > 1) {   // group sums are accumulated with atomics
        if (int32_t e = check_cuda(cudaMemsetAsync(bp.db, 0, bc_bytes, stream), "cudaMemsetAsync(db)")) return e;
        if (int32_t e = check_cuda(cudaMemsetAsync(bp.dc, 0, bc_bytes, stream), "cudaMemsetAsync(dc)")) return e;
    }
    if (bp.dd) if (int32_t e = check_cuda(cudaMemsetAsync(bp.dd, 0, p.H * sizeof(float), stream), "cudaMemsetAsync(dd)")) return e;
    if (bp.d_a) if (int32_t e = check_cuda(cudaMemsetAsync(bp.d_a, 0, p.H * sizeof(float), stream), "cudaMemsetAsync(da)")) return e;
    return p.dtype == BM_DTYPE_F32 ? launch_bwd<float>(bp, w, stream) : launch_bwd<__nv_bfloat16>(bp, w, stream);
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
