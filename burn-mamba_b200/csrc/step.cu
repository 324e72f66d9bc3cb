// Recurrent single-token kernels: Mamba-2 state update + readout, conv window step, Mamba-1 step,
// Mamba-3 step.  All are HBM-bound streaming passes over the recurrent state: 128-bit loads/stores,
// one warp (or a power-of-two slice of it) per state row, warp-shuffle reduction for the readout.
#include "common.cuh"

using namespace bm;

namespace {

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }

template <typename T>
__device__ __forceinline__ float4 ld4_act(const T* p);
template <>
__device__ __forceinline__ float4 ld4_act<float>(const float* p) { return ld4(p); }
template <>
__device__ __forceinline__ float4 ld4_act<__nv_bfloat16>(const __nv_bfloat16* p) {
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    __nv_bfloat162 lo = *reinterpret_cast<__nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
    float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
    return make_float4(a.x, a.y, b.x, b.y);
}

// ------------------------------------------------------------------------------------------
// Mamba-2 step.  Grid: one CTA per (b, h); each warp owns rows p = warp, warp + nwarps, ...
// LPR = lanes per state row (R / 4 when R <= 128, else 32 with a loop over 128-wide slabs).
// ------------------------------------------------------------------------------------------
template <typename T, int LPR>
__global__ void __launch_bounds__(256) step2_kernel(bm_step2_args a) {
    constexpr int ROWS_PER_WARP = 32 / LPR;
    const int bh = blockIdx.x, b = bh / a.nheads, h = bh % a.nheads;
    const int g = h / (a.nheads / a.ngroups);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int sub = lane / LPR, rl = lane % LPR;  // row slot inside the warp, lane inside the row
    const int R = a.state_rank, P = a.headdim;
    float dt = a.dt[bh];
    if (a.dt_bias) dt = fminf(fmaxf(softplus_f32(dt + a.dt_bias[h]), a.dt_min), a.dt_max);
    const float da = expf(dt * a.a[h]);
    const float dskip = a.d ? a.d[h] : 0.f;
    const T* bv = static_cast<const T*>(a.b) + ((int64_t)b * a.ngroups + g) * R;
    const T* cv = static_cast<const T*>(a.c) + ((int64_t)b * a.ngroups + g) * R;
    const T* xv = static_cast<const T*>(a.x) + (int64_t)bh * P;
    const T* zv = a.z ? static_cast<const T*>(a.z) + (int64_t)bh * P : nullptr;
    T* yv = static_cast<T*>(a.y) + (int64_t)bh * P;
    float* st = a.state + (int64_t)bh * P * R;
    const int slabs = (R + 4 * LPR - 1) / (4 * LPR);
    for (int p0 = warp * ROWS_PER_WARP; p0 < P; p0 += nwarps * ROWS_PER_WARP) {
        const int p = p0 + sub;
        const bool live = p < P;
        const float xp = live ? to_f32(xv[p]) : 0.f;
        const float dtx = dt * xp;
        float part = 0.f;
        for (int sl = 0; sl < slabs; ++sl) {
            const int r = (sl * LPR + rl) * 4;
            if (live && r < R) {
                float4 hv = ld4(st + (int64_t)p * R + r);
                float4 b4 = ld4_act(bv + r), c4 = ld4_act(cv + r);
                hv.x = fmaf(hv.x, da, dtx * b4.x);
                hv.y = fmaf(hv.y, da, dtx * b4.y);
                hv.z = fmaf(hv.z, da, dtx * b4.z);
                hv.w = fmaf(hv.w, da, dtx * b4.w);
                st4(st + (int64_t)p * R + r, hv);
                part += hv.x * c4.x + hv.y * c4.y + hv.z * c4.z + hv.w * c4.w;
            }
        }
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (live && rl == 0) {
            float y = fmaf(dskip, xp, part);
            if (zv) y *= silu_f32(to_f32(zv[p]));
            yv[p] = from_f32<T>(y);
        }
    }
}

// Any state_rank (not a multiple of 4): one thread per (b, h, p) row.
template <typename T>
__global__ void step2_scalar_kernel(bm_step2_args a) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int P = a.headdim, R = a.state_rank;
    if (idx >= (int64_t)a.batch * a.nheads * P) return;
    const int64_t bh = idx / P;
    const int h = bh % a.nheads, b = bh / a.nheads, g = h / (a.nheads / a.ngroups);
    float dt = a.dt[bh];
    if (a.dt_bias) dt = fminf(fmaxf(softplus_f32(dt + a.dt_bias[h]), a.dt_min), a.dt_max);
    const float da = expf(dt * a.a[h]);
    const T* bv = static_cast<const T*>(a.b) + ((int64_t)b * a.ngroups + g) * R;
    const T* cv = static_cast<const T*>(a.c) + ((int64_t)b * a.ngroups + g) * R;
    const float xp = to_f32(static_cast<const T*>(a.x)[idx]);
    float* st = a.state + idx * R;
    float part = 0.f;
    for (int r = 0; r < R; ++r) {
        float hv = fmaf(st[r], da, dt * xp * to_f32(bv[r]));
        st[r] = hv;
        part = fmaf(hv, to_f32(cv[r]), part);
    }
    float y = a.d ? fmaf(a.d[h], xp, part) : part;
    if (a.z) y *= silu_f32(to_f32(static_cast<const T*>(a.z)[idx]));
    static_cast<T*>(a.y)[idx] = from_f32<T>(y);
}

template <typename T>
int32_t launch_step2(const bm_step2_args& a, cudaStream_t st) {
    const int R = a.state_rank;
    const int64_t bh = (int64_t)a.batch * a.nheads;
    const bool vec = R % 4 == 0 && ((R / 4) <= 32 ? ((R / 4) & (R / 4 - 1)) == 0 : true);
    if (!vec) {
        int64_t total = bh * a.headdim;
        step2_scalar_kernel<T><<<(unsigned)cdiv(total, 256), 256, 0, st>>>(a);
        return check_launch("step2_scalar");
    }
    const int lpr = R / 4 >= 32 ? 32 : R / 4;
    const int rows_per_warp = 32 / lpr;
    int warps = (int)cdiv(a.headdim, rows_per_warp);
    warps = warps > 8 ? 8 : (warps < 1 ? 1 : warps);
    const unsigned grid = (unsigned)bh, block = warps * 32;
    switch (lpr) {
        case 32: step2_kernel<T, 32><<<grid, block, 0, st>>>(a); break;
        case 16: step2_kernel<T, 16><<<grid, block, 0, st>>>(a); break;
        case 8: step2_kernel<T, 8><<<grid, block, 0, st>>>(a); break;
        case 4: step2_kernel<T, 4><<<grid, block, 0, st>>>(a); break;
        case 2: step2_kernel<T, 2><<<grid, block, 0, st>>>(a); break;
        default: step2_kernel<T, 1><<<grid, block, 0, st>>>(a); break;
    }
    return check_launch("step2");
}

// ------------------------------------------------------------------------------------------
// Conv window step: window[b, v, :] := [window[b, v, 1:], xin[b, v]]; out = silu(window . w + bias).
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void conv_step_kernel(bm_conv_step_args a) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)a.batch * a.channels) return;
    const int v = idx % a.channels, K = a.kernel;
    const int64_t b = idx / a.channels;
    float* win = a.window + idx * K;
    const float* w = a.weight + (int64_t)v * K;
    const int64_t xs = a.xin_stride > 0 ? a.xin_stride : a.channels;
    const float xn = to_f32(static_cast<const T*>(a.xin)[b * xs + v]);
    float acc = a.bias ? a.bias[v] : 0.f;
    if (K == 4) {
        float4 wv = ld4(win), ww = ld4(w);
        float4 nw = make_float4(wv.y, wv.z, wv.w, xn);
        st4(win, nw);
        acc += nw.x * ww.x + nw.y * ww.y + nw.z * ww.z + nw.w * ww.w;
    } else {
        for (int k = 0; k < K; ++k) {
            float val = k + 1 < K ? win[k + 1] : xn;
            win[k] = val;
            acc = fmaf(val, w[k], acc);
        }
    }
    const T o = from_f32<T>(silu_f32(acc));
    if (a.out_b == nullptr) {
        static_cast<T*>(a.out)[idx] = o;
    } else if (v < a.split_x) {   // the three tensors the state step reads: x [b, split_x], B / C [b, split_bc]
        static_cast<T*>(a.out)[b * a.split_x + v] = o;
    } else if (v < a.split_x + a.split_bc) {
        static_cast<T*>(a.out_b)[b * a.split_bc + (v - a.split_x)] = o;
    } else {
        static_cast<T*>(a.out_c)[b * a.split_bc + (v - a.split_x - a.split_bc)] = o;
    }
}

// ------------------------------------------------------------------------------------------
// Mamba-1 step: one thread per (b, i) channel, state row of R floats.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void step1_kernel(bm_step1_args a) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int I = a.d_inner, R = a.state_rank;
    if (idx >= (int64_t)a.batch * I) return;
    const int i = idx % I, b = idx / I;
    float delta = to_f32(static_cast<const T*>(a.delta)[idx]);
    if (a.delta_softplus) delta = softplus_stock(delta + (a.delta_bias ? a.delta_bias[i] : 0.f));
    const float u = to_f32(static_cast<const T*>(a.u)[idx]);
    const T* bv = static_cast<const T*>(a.b) + (int64_t)b * R;
    const T* cv = static_cast<const T*>(a.c) + (int64_t)b * R;
    const float* arow = a.a + (int64_t)i * R;
    float* st = a.state + idx * R;
    float part = 0.f;
    const float du = delta * u;
    if (R % 4 == 0) {
        for (int r = 0; r < R; r += 4) {
            float4 hv = ld4(st + r), av = ld4(arow + r);
            hv.x = fmaf(hv.x, expf(delta * av.x), du * to_f32(bv[r]));
            hv.y = fmaf(hv.y, expf(delta * av.y), du * to_f32(bv[r + 1]));
            hv.z = fmaf(hv.z, expf(delta * av.z), du * to_f32(bv[r + 2]));
            hv.w = fmaf(hv.w, expf(delta * av.w), du * to_f32(bv[r + 3]));
            st4(st + r, hv);
            part += hv.x * to_f32(cv[r]) + hv.y * to_f32(cv[r + 1]) + hv.z * to_f32(cv[r + 2]) + hv.w * to_f32(cv[r + 3]);
        }
    } else {
        for (int r = 0; r < R; ++r) {
            float hv = fmaf(st[r], expf(delta * arow[r]), du * to_f32(bv[r]));
            st[r] = hv;
            part = fmaf(hv, to_f32(cv[r]), part);
        }
    }
    float y = a.d ? fmaf(a.d[i], u, part) : part;
    if (a.z) y *= silu_f32(to_f32(static_cast<const T*>(a.z)[idx]));
    static_cast<T*>(a.y)[idx] = from_f32<T>(y);
}

// ------------------------------------------------------------------------------------------
// Mamba-3 step.  One CTA per (b, h): (1) new wrapped angle, rotated B / C and the previous B into
// shared memory; (2) state rows streamed once, warp per row; (3) cache roll.
// ------------------------------------------------------------------------------------------
constexpr int kStep3MaxM = 8;

// One rotated B/C element from the cos/sin tables of the new angle (src/modules/misc/rope.rs:50-170).
__device__ __forceinline__ float rot_elem(const float* row, const float* cs_sm, const float* sn_sm, int r, int R, int rope_dim,
                                          bool pairwise) {
    float self = row[r];
    if (rope_dim == 0) return self;
    if (pairwise) {
        if (r >= rope_dim) return self;
        const float c = cs_sm[r >> 1], s = sn_sm[r >> 1], other = row[r ^ 1];
        return (r & 1) ? (s * other + c * self) : (c * self - s * other);
    }
    int half = R >> 1, na = rope_dim >> 1;
    if (r < na) return cs_sm[r] * self - sn_sm[r] * row[r + half];
    if (r >= half && r < half + na) return sn_sm[r - half] * row[r - half] + cs_sm[r - half] * self;
    return self;
}

// kM: the MIMO rank when it is 1, 2 or 4 (the loops over m are then resolved at compile time), 0 for any other rank.
template <int kM>
__global__ void __launch_bounds__(256, 2) step3_kernel(bm_step3_args a) {
    extern __shared__ float sm[];
    const int R = a.state_rank, P = a.headdim, M = kM ? kM : a.mimo_rank, H = a.nheads;
    const int na_alloc = max(a.rope_dim / 2, 1), na = a.rope_dim / 2;
    float* ang = sm;                 // [na_alloc] new wrapped angle
    float* cosv = ang + na_alloc;    // [na_alloc]
    float* sinv = cosv + na_alloc;   // [na_alloc]
    float* bs = sm + ((3 * na_alloc + 3) & ~3);  // [M][R] rotated B (16-byte aligned for 128-bit reads)
    float* cs = bs + M * R;          // [M][R] rotated C
    float* bp = cs + M * R;          // [M][R] previous rotated B
    float* braw = bp + M * R;        // [M][R] this step's B as given
    float* craw = braw + M * R;      // [M][R] this step's C as given
    const int bh = blockIdx.x, b = bh / H, h = bh % H, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const bool pairwise = M == 1;
    float* st = a.state + (int64_t)bh * P * R;
    const bool fast = R % 4 == 0 && R <= 128 && M <= 4;
    constexpr int NB = 8;
    const int r4 = lane * 4;
    const bool act = r4 < R;
    // (0) Everything the step reads from global memory is requested before anything waits on it: the first batch of
    // state rows of this warp (with P <= 64 the only one) and its per-row scalars, the raw B / C rows, the previous B,
    // the angle inputs.  The rotation below then works from shared memory, so the CTA pays one memory latency, not
    // one per phase.
    float4 hv[NB];
    float xl = 0.f, xpl = 0.f, mxl[4] = {1.f, 1.f, 1.f, 1.f};
    auto fetch_rows = [&](int p0) {
#pragma unroll
        for (int j = 0; j < NB; ++j)
            hv[j] = (p0 + j < P && act) ? ld4(st + (int64_t)(p0 + j) * R + r4) : make_float4(0.f, 0.f, 0.f, 0.f);
        // per-row scalars: lane j of the warp fetches those of row p0 + j, later they are broadcast
        const int prow = p0 + (lane & (NB - 1));
        const bool plive = prow < P;
        xl = plive ? a.x[(int64_t)bh * P + prow] : 0.f;
        xpl = plive ? a.v_state[(int64_t)bh * P + prow] : 0.f;
#pragma unroll
        for (int m = 0; m < 4; ++m)
            mxl[m] = (m < M && plive && a.mimo_x) ? a.mimo_x[((int64_t)h * M + m) * P + prow] : 1.f;
    };
    if (fast && warp * NB < P) fetch_rows(warp * NB);
    const float dt = a.dt[bh];
    const float alpha = a.alpha[bh], beta = a.beta[bh], gamma = a.gamma[bh];
    // (row m, column r) loops run m outside and r over the threads: no division by the runtime R per element
    for (int m = 0; m < M; ++m) {
        const int64_t row = (((int64_t)b * M + m) * H + h) * R;
        for (int r = tid; r < R; r += blockDim.x) {
            braw[m * R + r] = a.b[row + r];
            craw[m * R + r] = a.c[row + r];
            bp[m * R + r] = a.k_state[row + r];
        }
    }
    // (1a) angle := wrap(angle + dt * range * pi * tanh(rot)) (src/mamba3/rotation/mod.rs:559-567, :744-747)
    for (int j = tid; j < na_alloc; j += blockDim.x) {
        float inc = dt * (tanhf(a.rot[(int64_t)b * na_alloc + j]) * (a.range * 3.14159265358979323846f));
        float th = wrap_angle(a.angle[(int64_t)bh * na_alloc + j] + inc);
        ang[j] = th;
        sincosf(th, &sinv[j], &cosv[j]);
    }
    __syncthreads();
    // (1b) rotate B and C
    for (int m = 0; m < M; ++m)
        for (int r = tid; r < R; r += blockDim.x) {
            bs[m * R + r] = rot_elem(braw + m * R, cosv, sinv, r, R, na * 2, pairwise);
            cs[m * R + r] = rot_elem(craw + m * R, cosv, sinv, r, R, na * 2, pairwise);
        }
    __syncthreads();
    // (2) state rows
    if (fast) {
        // Fast path: a lane owns 4 consecutive state columns of every row (one 128-bit load / store per
        // row) and keeps its slice of the rotated B / C and of the previous B in registers.  The warp
        // works on NB rows at a time: all NB row loads are issued before the first is used, so that each
        // warp keeps NB x 512 bytes in flight, and the NB x 4 per-lane partial outputs are reduced with
        // one transposing butterfly (31 shuffles instead of 5 per value); lane 4 j + m then holds
        // y[row j][m].
        float4 bq[4], cq[4], pq[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const bool on = act && m < M;
            bq[m] = on ? ld4(bs + m * R + r4) : make_float4(0.f, 0.f, 0.f, 0.f);
            cq[m] = on ? ld4(cs + m * R + r4) : make_float4(0.f, 0.f, 0.f, 0.f);
            pq[m] = on ? ld4(bp + m * R + r4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int p0 = warp * NB; p0 < P; p0 += NB * nwarps) {
            if (p0 != warp * NB) fetch_rows(p0);
            const int prow = p0 + (lane & (NB - 1));
            const bool plive = prow < P;
            // the row's input coefficients, formed once by the lane that fetched its scalars
            float gl[4], btl[4];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                gl[m] = gamma * xl * mxl[m];
                btl[m] = beta * xpl * mxl[m];
            }
            float v[NB * 4];
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                float4 h4 = make_float4(alpha * hv[j].x, alpha * hv[j].y, alpha * hv[j].z, alpha * hv[j].w);
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    if (m < M) {
                        const float g = __shfl_sync(0xffffffffu, gl[m], j), bt = __shfl_sync(0xffffffffu, btl[m], j);
                        h4.x = fmaf(g, bq[m].x, fmaf(bt, pq[m].x, h4.x));
                        h4.y = fmaf(g, bq[m].y, fmaf(bt, pq[m].y, h4.y));
                        h4.z = fmaf(g, bq[m].z, fmaf(bt, pq[m].z, h4.z));
                        h4.w = fmaf(g, bq[m].w, fmaf(bt, pq[m].w, h4.w));
                    }
                }
                if (p0 + j < P && act) st4(st + (int64_t)(p0 + j) * R + r4, h4);
#pragma unroll
                for (int m = 0; m < 4; ++m)
                    v[j * 4 + m] = h4.x * cq[m].x + h4.y * cq[m].y + h4.z * cq[m].z + h4.w * cq[m].w;
            }
            // transposing butterfly: after the round with offset o a lane keeps the half of its values
            // whose index bit matches its own lane bit, summed with the partner's copy of that half
#pragma unroll
            for (int o = 16, n = NB * 2; o > 0; o >>= 1, n >>= 1) {
                const bool up = (lane & o) != 0;
#pragma unroll
                for (int k = 0; k < n; ++k) {
                    const float send = up ? v[k] : v[k + n];
                    const float keep = up ? v[k + n] : v[k];
                    v[k] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
            // v[0] of lane l is the total of value index l = 4 * row + m
            const int yrow = p0 + (lane >> 2), ym = lane & 3;
            if (yrow < P && ym < M) a.y[(((int64_t)b * M + ym) * H + h) * P + yrow] = v[0];
            if (plive && lane < NB) a.v_state[(int64_t)bh * P + prow] = xl;
        }
    } else {
    for (int p = warp; p < P; p += nwarps) {
        const float x = a.x[(int64_t)bh * P + p], xprev = a.v_state[(int64_t)bh * P + p];
        float cg[kStep3MaxM], cb[kStep3MaxM], part[kStep3MaxM];
#pragma unroll
        for (int m = 0; m < kStep3MaxM; ++m) {
            float mx = (m < M && a.mimo_x) ? a.mimo_x[((int64_t)h * M + m) * P + p] : 1.f;
            cg[m] = gamma * x * mx;
            cb[m] = beta * xprev * mx;
            part[m] = 0.f;
        }
        for (int r = lane; r < R; r += 32) {
            float hv = alpha * st[(int64_t)p * R + r];
#pragma unroll
            for (int m = 0; m < kStep3MaxM; ++m)
                if (m < M) hv = fmaf(cg[m], bs[m * R + r], fmaf(cb[m], bp[m * R + r], hv));
            st[(int64_t)p * R + r] = hv;
#pragma unroll
            for (int m = 0; m < kStep3MaxM; ++m)
                if (m < M) part[m] = fmaf(hv, cs[m * R + r], part[m]);
        }
#pragma unroll
        for (int m = 0; m < kStep3MaxM; ++m) {
            if (m < M) {
                float s = part[m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0) a.y[(((int64_t)b * M + m) * H + h) * P + p] = s;
            }
        }
        if (lane == 0) a.v_state[(int64_t)bh * P + p] = x;
    }
    }
    // (3) cache roll: k_state := rotated B, angle := new angle (all reads of the old values are done:
    // bp / ang were staged before the barrier above)
    for (int m = 0; m < M; ++m)
        for (int r = tid; r < R; r += blockDim.x) a.k_state[(((int64_t)b * M + m) * H + h) * R + r] = bs[m * R + r];
    for (int j = tid; j < na_alloc; j += blockDim.x) a.angle[(int64_t)bh * na_alloc + j] = ang[j];
}

}  // namespace

extern "C" int32_t bm_step2(const bm_step2_args* a, void* stream) {
    clear_error();
    if (a == nullptr) return fail(BM_ERR_NULL_POINTER, "args is NULL");
    BM_REQUIRE(a->batch > 0 && a->nheads > 0 && a->headdim > 0 && a->state_rank > 0, BM_ERR_BAD_SHAPE,
               "batch, nheads, headdim, state_rank must be positive");
    BM_REQUIRE(a->ngroups > 0 && a->nheads % a->ngroups == 0, BM_ERR_BAD_SHAPE, "nheads must be divisible by ngroups");
    BM_REQUIRE(a->dtype == BM_DTYPE_F32 || a->dtype == BM_DTYPE_BF16, BM_ERR_UNSUPPORTED, "dtype must be f32 or bf16");
    BM_REQUIRE_PTR(a->state);
    BM_REQUIRE_PTR(a->x);
    BM_REQUIRE_PTR(a->dt);
    BM_REQUIRE_PTR(a->a);
    BM_REQUIRE_PTR(a->b);
    BM_REQUIRE_PTR(a->c);
    BM_REQUIRE_PTR(a->y);
    BM_OPTIONAL_PTR(a->d);
    BM_OPTIONAL_PTR(a->dt_bias);
    BM_OPTIONAL_PTR(a->z);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return a->dtype == BM_DTYPE_F32 ? launch_step2<float>(*a, st) : launch_step2<__nv_bfloat16>(*a, st);
}

extern "C" int32_t bm_conv_step(const bm_conv_step_args* a, void* stream) {
    clear_error();
    if (a == nullptr) return fail(BM_ERR_NULL_POINTER, "args is NULL");
    BM_REQUIRE(a->batch > 0 && a->channels > 0 && a->kernel > 0, BM_ERR_BAD_SHAPE, "batch, channels, kernel must be positive");
    BM_REQUIRE(a->dtype == BM_DTYPE_F32 || a->dtype == BM_DTYPE_BF16, BM_ERR_UNSUPPORTED, "dtype must be f32 or bf16");
    BM_REQUIRE_PTR(a->window);
    BM_REQUIRE_PTR(a->xin);
    BM_REQUIRE_PTR(a->weight);
    BM_REQUIRE_PTR(a->out);
    BM_OPTIONAL_PTR(a->bias);
    BM_REQUIRE(a->xin_stride == 0 || a->xin_stride >= a->channels, BM_ERR_BAD_SHAPE, "xin_stride must be 0 (dense) or >= channels");
    if (a->out_b != nullptr || a->out_c != nullptr) {
        BM_REQUIRE_PTR(a->out_b);
        BM_REQUIRE_PTR(a->out_c);
        BM_REQUIRE(a->split_x > 0 && a->split_bc > 0 && a->split_x + 2 * a->split_bc == a->channels, BM_ERR_BAD_SHAPE,
                   "split_x + 2 split_bc must equal channels");
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int64_t total = (int64_t)a->batch * a->channels;
    if (a->dtype == BM_DTYPE_F32) conv_step_kernel<float><<<(unsigned)cdiv(total, 256), 256, 0, st>>>(*a);
    else conv_step_kernel<__nv_bfloat16><<<(unsigned)cdiv(total, 256), 256, 0, st>>>(*a);
    return check_launch("conv_step");
}

extern "C" int32_t bm_step1(const bm_step1_args* a, void* stream) {
    clear_error();
    if (a == nullptr) return fail(BM_ERR_NULL_POINTER, "args is NULL");
    BM_REQUIRE(a->batch > 0 && a->d_inner > 0 && a->state_rank > 0, BM_ERR_BAD_SHAPE,
               "batch, d_inner, state_rank must be positive");
    BM_REQUIRE(a->dtype == BM_DTYPE_F32 || a->dtype == BM_DTYPE_BF16, BM_ERR_UNSUPPORTED, "dtype must be f32 or bf16");
    BM_REQUIRE_PTR(a->state);
    BM_REQUIRE_PTR(a->u);
    BM_REQUIRE_PTR(a->delta);
    BM_REQUIRE_PTR(a->a);
    BM_REQUIRE_PTR(a->b);
    BM_REQUIRE_PTR(a->c);
    BM_REQUIRE_PTR(a->y);
    BM_OPTIONAL_PTR(a->d);
    BM_OPTIONAL_PTR(a->delta_bias);
    BM_OPTIONAL_PTR(a->z);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int64_t total = (int64_t)a->batch * a->d_inner;
    if (a->dtype == BM_DTYPE_F32) step1_kernel<float><<<(unsigned)cdiv(total, 128), 128, 0, st>>>(*a);
    else step1_kernel<__nv_bfloat16><<<(unsigned)cdiv(total, 128), 128, 0, st>>>(*a);
    return check_launch("step1");
}

extern "C" int32_t bm_step3(const bm_step3_args* a, void* stream) {
    clear_error();
    if (a == nullptr) return fail(BM_ERR_NULL_POINTER, "args is NULL");
    BM_REQUIRE(a->batch > 0 && a->nheads > 0 && a->headdim > 0 && a->state_rank > 0 && a->mimo_rank > 0,
               BM_ERR_BAD_SHAPE, "batch, nheads, headdim, state_rank, mimo_rank must be positive");
    BM_REQUIRE(a->mimo_rank <= kStep3MaxM, BM_ERR_UNSUPPORTED, "mimo_rank above %d", kStep3MaxM);
    BM_REQUIRE(a->rope_dim >= 0 && a->rope_dim % 2 == 0 && a->rope_dim <= a->state_rank, BM_ERR_BAD_SHAPE,
               "rope_dim must be even and <= state_rank");
    BM_REQUIRE(a->rope_dim == 0 || a->state_rank % 2 == 0, BM_ERR_BAD_SHAPE, "state_rank must be even when rotating");
    BM_REQUIRE_PTR(a->state);
    BM_REQUIRE_PTR(a->k_state);
    BM_REQUIRE_PTR(a->v_state);
    BM_REQUIRE_PTR(a->angle);
    BM_REQUIRE_PTR(a->x);
    BM_REQUIRE_PTR(a->b);
    BM_REQUIRE_PTR(a->c);
    BM_REQUIRE_PTR(a->rot);
    BM_REQUIRE_PTR(a->dt);
    BM_REQUIRE_PTR(a->alpha);
    BM_REQUIRE_PTR(a->beta);
    BM_REQUIRE_PTR(a->gamma);
    BM_REQUIRE_PTR(a->y);
    BM_OPTIONAL_PTR(a->mimo_x);
    size_t smem = (((3 * (size_t)(a->rope_dim / 2 > 1 ? a->rope_dim / 2 : 1) + 3) & ~(size_t)3) + 5 * (size_t)a->mimo_rank * a->state_rank) * sizeof(float);
    BM_REQUIRE(smem <= 48 * 1024, BM_ERR_UNSUPPORTED, "mimo_rank * state_rank too large for the step kernel");
    int64_t bh = (int64_t)a->batch * a->nheads;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (a->mimo_rank) {
        case 1: step3_kernel<1><<<(unsigned)bh, 256, smem, st>>>(*a); break;
        case 2: step3_kernel<2><<<(unsigned)bh, 256, smem, st>>>(*a); break;
        case 4: step3_kernel<4><<<(unsigned)bh, 256, smem, st>>>(*a); break;
        default: step3_kernel<0><<<(unsigned)bh, 256, smem, st>>>(*a); break;
    }
    return check_launch("step3");
}
