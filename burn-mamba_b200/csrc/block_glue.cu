// Pre- and post-SSD kernels of the Mamba-2 block (HBM-bound elementwise passes):
//   bm_conv1d_silu_fwd  causal depthwise conv (k taps) + bias + SiLU over the [b, s, v] projection columns,
//                       left context from the cache window, outputs written as the three tensors the SSD reads
//                       (src/mamba2/mamba2.rs:618-654: the window slide, Conv1d, SiLU and the x / B / C split);
//   bm_rmsnorm_gated    RmsNormGated (src/modules/norm/rms_norm_gated.rs:70-135) and, with z = NULL, the plain
//                       RmsNorm of the layer stack (src/modules/norm/rms_norm.rs:53-98).
// Both take a row stride for the tensors that are column slices of the in-projection's output, so that no
// slice is materialised.
#include "common.cuh"
#include "tc_common.cuh"

#include <algorithm>

using namespace bm;

namespace {

constexpr int TL = 4;         // tokens per thread in the conv kernel
constexpr int VEC = 8;        // channels per thread (16 bytes of bf16, 32 of f32)

template <typename T>
struct Vec8 {
    float v[VEC];
    __device__ __forceinline__ void load(const T* p);
    __device__ __forceinline__ void store(T* p) const;
};
template <>
__device__ __forceinline__ void Vec8<float>::load(const float* p) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
template <>
__device__ __forceinline__ void Vec8<float>::store(float* p) const {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void Vec8<__nv_bfloat16>::load(const __nv_bfloat16* p) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
        v[2 * j] = f.x, v[2 * j + 1] = f.y;
    }
}
template <>
__device__ __forceinline__ void Vec8<__nv_bfloat16>::store(__nv_bfloat16* p) const {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// One thread: 8 adjacent channels x TL consecutive tokens.  All TL + K - 1 input rows of the thread are fetched
// before anything is computed (the loads are independent, so they are all in flight together).
// Consecutive threads take consecutive channel vectors, so every row access of a warp is one contiguous run.
template <typename T, int K>
__global__ void __launch_bounds__(128, 6) conv1d_silu_kernel(bm_conv1d_silu_args a) {
    const int V = a.channels, S = a.seqlen;
    const int nvec = V / VEC;
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int vec = gid % nvec;
    const int nchunk = (S + TL - 1) / TL;
    const int chunk = (gid / nvec) % nchunk;
    const int b = gid / ((int64_t)nvec * nchunk);
    if (b >= a.batch) return;
    const int c0 = vec * VEC, t0 = chunk * TL;
    const T* xin = static_cast<const T*>(a.xin) + (int64_t)b * S * a.xin_stride + c0;
    Vec8<T> in[TL + K - 1];
#pragma unroll
    for (int r = 0; r < TL + K - 1; ++r) {
        const int t = t0 - (K - 1) + r;
        if (t >= 0 && t < S) {
            in[r].load(xin + (int64_t)t * a.xin_stride);
        } else {
            // before the sequence: the cache window's column K + t (its last K - 1 columns are tokens -K+1 .. -1)
#pragma unroll
            for (int j = 0; j < VEC; ++j)
                in[r].v[j] = (t < 0 && a.window) ? a.window[((int64_t)b * V + c0 + j) * K + (K + t)] : 0.f;
        }
    }
    float w[K][VEC], bias[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        bias[j] = a.bias ? a.bias[c0 + j] : 0.f;
        if (K == 4) {   // one 16-byte load per channel (rows of the [v, 4] weight are 16-byte aligned)
            const float4 wv = *reinterpret_cast<const float4*>(a.weight + (int64_t)(c0 + j) * 4);
            w[0][j] = wv.x, w[1 % K][j] = wv.y, w[2 % K][j] = wv.z, w[3 % K][j] = wv.w;
        } else {
#pragma unroll
            for (int k = 0; k < K; ++k) w[k][j] = a.weight[(int64_t)(c0 + j) * K + k];
        }
    }
    // which output tensor this channel vector belongs to
    T* dst;
    int64_t dstride;
    if (a.out_b == nullptr) {
        dst = static_cast<T*>(a.out_x) + (int64_t)b * S * V + c0, dstride = V;
    } else if (c0 < a.split_x) {
        dst = static_cast<T*>(a.out_x) + (int64_t)b * S * a.split_x + c0, dstride = a.split_x;
    } else if (c0 < a.split_x + a.split_bc) {
        dst = static_cast<T*>(a.out_b) + (int64_t)b * S * a.split_bc + (c0 - a.split_x), dstride = a.split_bc;
    } else {
        dst = static_cast<T*>(a.out_c) + (int64_t)b * S * a.split_bc + (c0 - a.split_x - a.split_bc), dstride = a.split_bc;
    }
#pragma unroll
    for (int i = 0; i < TL; ++i) {
        if (t0 + i < S) {
            Vec8<T> o;
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
                float acc = bias[j];
#pragma unroll
                for (int k = 0; k < K; ++k) acc = fmaf(in[i + k].v[j], w[k][j], acc);
                o.v[j] = silu_fast(acc);
            }
            o.store(dst + (int64_t)(t0 + i) * dstride);
        }
    }
}

// The same conv for bf16 with the input staged by TMA: a persistent CTA walks tiles of 64 tokens x 128 channels
// (+ K - 1 halo rows, zero-filled by the copy where they lie before the sequence) and keeps the copies of its
// next two tiles in flight, so the latency of the strided row reads is paid by the copy engine, not by registers.
// A thread computes 8 tokens of one 8-channel vector from shared memory.  The first K - 1 tokens of a sequence
// take their left context from the float32 cache window, as above.  A wait on a copy is bounded; if it ever ran
// out, the tile's rows would be read straight from global memory instead.
constexpr int kCtTok = 64, kCtCh = 128, kCtStages = 3, kCtThreads = 128;
constexpr int kCtRowsMax = kCtTok + 3;
constexpr int kCtStageBytes = kCtRowsMax * kCtCh * 2;   // 17152

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
            tc::smem_u32(dst)),
        "l"(m), "r"(tc::smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

template <int K>
__global__ void __launch_bounds__(kCtThreads, 4) conv1d_silu_tma_kernel(bm_conv1d_silu_args a, const __grid_constant__ CUtensorMap tm,
                                                                         int n_ctile, int n_ttile, int ntiles) {
    using T = __nv_bfloat16;
    extern __shared__ __align__(128) unsigned char ctraw[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(ctraw + kCtStages * kCtStageBytes);
    const int V = a.channels, S = a.seqlen, tid = threadIdx.x;
    constexpr int ROWS = kCtTok + K - 1;
    if (tid == 0) {
        for (int i = 0; i < kCtStages; ++i) tc::mbar_init(&bars[i], 1);
        tc::fence_mbar_init();
        tc::tma_prefetch_desc(&tm);
    }
    __syncthreads();
    auto coords = [&](int tile, int& ct, int& tt, int& b) {   // channel tile fastest
        ct = tile % n_ctile;
        tt = (tile / n_ctile) % n_ttile;
        b = tile / (n_ctile * n_ttile);
    };
    auto issue = [&](int k) {
        const int tile = blockIdx.x + k * gridDim.x;
        if (tid == 0 && tile < ntiles) {
            int ct, tt, b;
            coords(tile, ct, tt, b);
            const int sidx = k % kCtStages;
            tc::mbar_expect_tx(&bars[sidx], ROWS * kCtCh * 2);
            tma_load_3d(ctraw + sidx * kCtStageBytes, &tm, &bars[sidx], ct * kCtCh, tt * kCtTok - (K - 1), b);
        }
    };
    issue(0);
    issue(1);
    const int cg = tid & 15, tg = tid >> 4;   // 8-channel vector inside the tile, group of 8 tokens
    float w[K][VEC], bias[VEC];
    int ct_loaded = -1;
    for (int k = 0;; ++k) {
        const int tile = blockIdx.x + k * gridDim.x;
        if (tile >= ntiles) break;
        issue(k + 2);   // its stage was last read two tiles ago, before that tile's closing barrier
        int ct, tt, b;
        coords(tile, ct, tt, b);
        const int c0 = ct * kCtCh + cg * VEC, t0 = tt * kCtTok;
        const bool live = c0 < V;
        const int cc = live ? c0 : 0;
        // taps and bias of this thread's 8 channels: fetched when the channel tile changes.  The host sizes the grid as a
        // multiple of the channel tiles per row where it can, so that a CTA keeps one channel tile for all its tiles
        // (fetched per tile, these scalar reads at a 128-byte stride between threads were 7/8 of the kernel's L1 traffic).
        if (ct != ct_loaded) {
            ct_loaded = ct;
#pragma unroll
            for (int j = 0; j < VEC; ++j) {
                bias[j] = a.bias ? a.bias[cc + j] : 0.f;
#pragma unroll
                for (int kk = 0; kk < K; ++kk) w[kk][j] = a.weight[(int64_t)(cc + j) * K + kk];
            }
        }
        T* dst;
        int64_t dstride;
        if (a.out_b == nullptr) {
            dst = static_cast<T*>(a.out_x) + (int64_t)b * S * V + cc, dstride = V;
        } else if (cc < a.split_x) {
            dst = static_cast<T*>(a.out_x) + (int64_t)b * S * a.split_x + cc, dstride = a.split_x;
        } else if (cc < a.split_x + a.split_bc) {
            dst = static_cast<T*>(a.out_b) + (int64_t)b * S * a.split_bc + (cc - a.split_x), dstride = a.split_bc;
        } else {
            dst = static_cast<T*>(a.out_c) + (int64_t)b * S * a.split_bc + (cc - a.split_x - a.split_bc), dstride = a.split_bc;
        }
        bool landed = true;
        {
            uint32_t n = 0;
#pragma unroll 1
            while (!tc::mbar_try_wait(&bars[k % kCtStages], (k / kCtStages) & 1))
                if (++n >= tc::kWaitBudget) {
                    landed = false;
                    break;
                }
            landed = __all_sync(0xffffffffu, landed);
        }
        const unsigned char* stage = ctraw + (k % kCtStages) * kCtStageBytes;
        const T* grow = static_cast<const T*>(a.xin) + (int64_t)b * S * a.xin_stride + cc;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r0 = tg * 8 + half * TL;            // first token of this pass inside the tile
            Vec8<T> in[TL + K - 1];
#pragma unroll
            for (int r = 0; r < TL + K - 1; ++r) {
                const int t = t0 + r0 - (K - 1) + r;      // token of the row
                if (t < 0) {
#pragma unroll
                    for (int j = 0; j < VEC; ++j)
                        in[r].v[j] = a.window ? a.window[((int64_t)b * V + cc + j) * K + (K + t)] : 0.f;
                } else if (landed) {
                    in[r].load(reinterpret_cast<const T*>(stage + (r0 + r) * (kCtCh * 2) + cg * 16));
                } else if (t < S) {
                    in[r].load(grow + (int64_t)t * a.xin_stride);
                } else {
#pragma unroll
                    for (int j = 0; j < VEC; ++j) in[r].v[j] = 0.f;
                }
            }
#pragma unroll
            for (int i = 0; i < TL; ++i) {
                if (live && t0 + r0 + i < S) {
                    Vec8<T> o;
#pragma unroll
                    for (int j = 0; j < VEC; ++j) {
                        float acc = bias[j];
#pragma unroll
                        for (int kk = 0; kk < K; ++kk) acc = fmaf(in[i + kk].v[j], w[kk][j], acc);
                        o.v[j] = silu_fast(acc);
                    }
                    o.store(dst + (int64_t)(t0 + r0 + i) * dstride);
                }
            }
        }
        __syncthreads();   // the stage is free for the tile after next
    }
}

// New cache window: the last K columns of [old window columns 1.. | the sequence's raw inputs].
template <typename T>
__global__ void conv_window_kernel(bm_conv1d_silu_args a) {
    const int V = a.channels, S = a.seqlen, K = a.kernel;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // (b, j, c): c fastest, so the reads run along channels
    if (idx >= (int64_t)a.batch * K * V) return;
    const int c = idx % V, j = (idx / V) % K, b = idx / ((int64_t)V * K);
    const int t = S - K + j;   // token that lands in column j
    float val;
    if (t >= 0) val = to_f32(static_cast<const T*>(a.xin)[((int64_t)b * S + t) * a.xin_stride + c]);
    else val = a.window ? a.window[((int64_t)b * V + c) * K + (K + t)] : 0.f;
    a.new_window[((int64_t)b * V + c) * K + j] = val;
}

// ---------------------------------------------------------------------------------------------
// gated RMS norm: one CTA per row, the row in registers, one pass.
// ---------------------------------------------------------------------------------------------
constexpr int NT = 128;            // threads per row
constexpr int MAXV = 8;            // vectors of 8 per thread: rows up to 8192 wide

// Eight consecutive elements as they come from memory (16 bytes of bf16, 32 of float32): what a thread holds of a
// row whose loads are all issued before the first is used.
template <typename T>
struct Raw8;
template <>
struct Raw8<__nv_bfloat16> {
    uint4 w;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { w = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void unpack(float (&v)[VEC]) const {
        const uint32_t q[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q[j]));
            v[2 * j] = f.x, v[2 * j + 1] = f.y;
        }
    }
};
template <>
struct Raw8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) {
        a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    }
    __device__ __forceinline__ void unpack(float (&v)[VEC]) const {
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    }
};

// NV = vectors of 8 per thread the row needs (ceil(width / (8 NT))), so that nothing is held for columns the row
// does not have.  Every load of the row (x, the gate, the weight) is issued before the first value is used: the CTA
// waits on memory once, not once per vector and again after the reduction.
template <typename T, int NV>
__global__ void __launch_bounds__(NT) rmsnorm_gated_kernel(bm_rmsnorm_gated_args a) {
    __shared__ float red[NT / 32];
    const int64_t row = blockIdx.x;
    const int D = a.width;
    const T* xr = static_cast<const T*>(a.x) + row * a.x_stride;
    const T* zr = a.z ? static_cast<const T*>(a.z) + row * a.z_stride : nullptr;
    const T* gr = static_cast<const T*>(a.gamma);
    T* orow = static_cast<T*>(a.out) + row * (int64_t)D;
    const bool gate = zr != nullptr, gate_first = gate && !a.norm_before_gate;
    Raw8<T> xraw[NV], zraw[NV], graw[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = min((i * NT + (int)threadIdx.x) * VEC, D - VEC);   // the last vector is fetched again where the row ends
        xraw[i].load(xr + c);
        if (gate) zraw[i].load(zr + c);
        graw[i].load(gr + c);
    }
    float xv[NV][VEC];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        xraw[i].unpack(xv[i]);
        if ((i * NT + (int)threadIdx.x) * VEC < D) {
            if (gate_first) {
                float zv[VEC];
                zraw[i].unpack(zv);
#pragma unroll
                for (int j = 0; j < VEC; ++j) xv[i][j] *= silu_fast(zv[j]);
            }
#pragma unroll
            for (int j = 0; j < VEC; ++j) ss = fmaf(xv[i][j], xv[i][j], ss);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < NT / 32; ++i) tot += red[i];
    const float inv = rsqrtf(tot / (float)D + a.eps);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * NT + threadIdx.x) * VEC;
        if (c < D) {
            float gv[VEC];
            graw[i].unpack(gv);
            Vec8<T> ov;
#pragma unroll
            for (int j = 0; j < VEC; ++j) ov.v[j] = xv[i][j] * inv * gv[j];
            if (gate && !gate_first) {
                float zv[VEC];
                zraw[i].unpack(zv);
#pragma unroll
                for (int j = 0; j < VEC; ++j) ov.v[j] *= silu_fast(zv[j]);
            }
            ov.store(orow + c);
        }
    }
}

template <typename T>
void launch_rmsnorm(const bm_rmsnorm_gated_args& a, cudaStream_t st) {
    const unsigned rows = (unsigned)a.rows;
    switch ((a.width + NT * VEC - 1) / (NT * VEC)) {
        case 1: rmsnorm_gated_kernel<T, 1><<<rows, NT, 0, st>>>(a); break;
        case 2: rmsnorm_gated_kernel<T, 2><<<rows, NT, 0, st>>>(a); break;
        case 3: rmsnorm_gated_kernel<T, 3><<<rows, NT, 0, st>>>(a); break;
        case 4: rmsnorm_gated_kernel<T, 4><<<rows, NT, 0, st>>>(a); break;
        case 5: rmsnorm_gated_kernel<T, 5><<<rows, NT, 0, st>>>(a); break;
        case 6: rmsnorm_gated_kernel<T, 6><<<rows, NT, 0, st>>>(a); break;
        case 7: rmsnorm_gated_kernel<T, 7><<<rows, NT, 0, st>>>(a); break;
        default: rmsnorm_gated_kernel<T, 8><<<rows, NT, 0, st>>>(a); break;
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Mamba-3: everything between the in-projection and the SSD slot for B and C, in one pass
// (src/mamba3/helpers.rs:82-95 qk_norm_expand_bias: RMS norm over r, group -> head expansion, + bias[h, m, r];
//  src/mamba3/rotation/mod.rs:653-679 + src/modules/misc/rope.rs:50-170: rotation of the leading rope_dim entries
//  by the cumulative angles, pairs (2j, 2j+1) when `pairwise`, else (j, j + r/2)).
// One CTA per token.  The raw rows [m, g, r] of B and C (a few KB) are normalised once into shared memory; then
// one thread per (head, group of 4 pairs) forms cos / sin of its angles once and writes its 8 entries of every
// rank of both tensors, consecutive threads on consecutive chunks.
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void store4(T* dst, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* dst, const float (&v)[4]) {
    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, const float (&v)[4]) {
    __nv_bfloat162 p[2] = {__floats2bfloat162_rn(v[0], v[1]), __floats2bfloat162_rn(v[2], v[3])};
    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<uint2*>(p);
}

template <typename T>
__global__ void __launch_bounds__(256, 4) mamba3_bc_prep_kernel(bm_mamba3_bc_prep_args a) {
    extern __shared__ float nrm[];   // [2][m * g][r]: normalised B rows, then C rows
    const int M = a.mimo_rank, G = a.ngroups, H = a.nheads, Rk = a.state_rank;
    const int rows = M * G, half = Rk / 2, na = a.rope_dim / 2, ngrp = half / 4;
    const int64_t tok = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    // ---- RMS norm of the 2 m g raw rows, one warp per row
    for (int rw = warp; rw < 2 * rows; rw += nwarps) {
        const bool isc = rw >= rows;
        const int r0 = isc ? rw - rows : rw;
        const T* src = static_cast<const T*>(isc ? a.c_raw : a.b_raw) + tok * a.raw_stride + (int64_t)r0 * Rk;
        const float* gam = isc ? a.c_gamma : a.b_gamma;
        float ss = 0.f;
        for (int e = lane; e < Rk; e += 32) {
            const float v = to_f32(src[e]);
            nrm[(int64_t)rw * Rk + e] = v;
            ss = fmaf(v, v, ss);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = 1.f / sqrtf(ss / (float)Rk + a.eps);
        for (int e = lane; e < Rk; e += 32) nrm[(int64_t)rw * Rk + e] *= inv * gam[e];
    }
    __syncthreads();
    // ---- heads: bias, rotation, store.  A thread takes 4 pairs of one head: one 16-byte read per half of the normalised
    // row and of the bias, so that the 16 threads of a head read 256 contiguous bytes with each instruction (at 8 pairs
    // per thread every 16-byte read skipped the next 16 bytes and a warp's read spread over twice the lines).
    const int hpg = H / G;
    for (int idx = threadIdx.x; idx < H * ngrp; idx += blockDim.x) {
        const int h = idx / ngrp, j0 = (idx % ngrp) * 4, g = h / hpg;
        float cs[4], sn[4], th[4];
        if (a.angles != nullptr && j0 + 4 <= na && (na & 3) == 0) {
            const float4 t0 = *reinterpret_cast<const float4*>(a.angles + (tok * H + h) * na + j0);
            th[0] = t0.x, th[1] = t0.y, th[2] = t0.z, th[3] = t0.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) th[j] = (a.angles != nullptr && j0 + j < na) ? a.angles[(tok * H + h) * na + j0 + j] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) __sincosf(wrap_angle(th[j]), &sn[j], &cs[j]);
        const int o_lo = a.pairwise ? 2 * j0 : j0, o_hi = a.pairwise ? 2 * j0 + 4 : j0 + half;
        for (int m = 0; m < M; ++m) {
#pragma unroll
            for (int isc = 0; isc < 2; ++isc) {
                const float* nr = nrm + ((int64_t)isc * rows + m * G + g) * Rk;
                const float* bias = (isc ? a.c_bias : a.b_bias) + ((int64_t)h * M + m) * Rk;
                const float4 nl = *reinterpret_cast<const float4*>(nr + o_lo), nh = *reinterpret_cast<const float4*>(nr + o_hi);
                const float4 bl = __ldg(reinterpret_cast<const float4*>(bias + o_lo));
                const float4 bh = __ldg(reinterpret_cast<const float4*>(bias + o_hi));
                const float lo[4] = {nl.x + bl.x, nl.y + bl.y, nl.z + bl.z, nl.w + bl.w};
                const float hi[4] = {nh.x + bh.x, nh.y + bh.y, nh.z + bh.z, nh.w + bh.w};
                float olo[4], ohi[4];
                if (a.pairwise) {   // lo, hi hold 8 consecutive entries: pair j = entries (2j, 2j + 1)
                    olo[0] = cs[0] * lo[0] - sn[0] * lo[1], olo[1] = sn[0] * lo[0] + cs[0] * lo[1];
                    olo[2] = cs[1] * lo[2] - sn[1] * lo[3], olo[3] = sn[1] * lo[2] + cs[1] * lo[3];
                    ohi[0] = cs[2] * hi[0] - sn[2] * hi[1], ohi[1] = sn[2] * hi[0] + cs[2] * hi[1];
                    ohi[2] = cs[3] * hi[2] - sn[3] * hi[3], ohi[3] = sn[3] * hi[2] + cs[3] * hi[3];
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        olo[j] = cs[j] * lo[j] - sn[j] * hi[j];
                        ohi[j] = sn[j] * lo[j] + cs[j] * hi[j];
                    }
                }
                T* dst = static_cast<T*>(isc ? a.c_out : a.b_out) + ((tok * M + m) * H + h) * Rk;
                store4<T>(dst + o_lo, olo);
                store4<T>(dst + o_hi, ohi);
            }
        }
    }
}

extern "C" int32_t bm_conv1d_silu_fwd(const bm_conv1d_silu_args* a, void* stream) {
    clear_error();
    if (a == nullptr) return fail(BM_ERR_NULL_POINTER, "args is NULL");
    BM_REQUIRE(a->batch > 0 && a->seqlen > 0 && a->channels > 0, BM_ERR_BAD_SHAPE, "batch, seqlen, channels must be positive");
    BM_REQUIRE(a->kernel == 4 || a->kernel == 2 || a->kernel == 3, BM_ERR_UNSUPPORTED, "conv kernel must be 2, 3 or 4 taps");
    BM_REQUIRE(a->dtype == BM_DTYPE_F32 || a->dtype == BM_DTYPE_BF16, BM_ERR_UNSUPPORTED, "dtype must be f32 or bf16");
    const int esz = a->dtype == BM_DTYPE_F32 ? 4 : 2;
    BM_REQUIRE(a->channels % VEC == 0 && ((int64_t)a->xin_stride * esz) % 16 == 0 && a->xin_stride >= a->channels, BM_ERR_BAD_SHAPE,
               "channels must be a multiple of 8 and input rows must start 16-byte aligned, stride >= channels");
    BM_REQUIRE_PTR(a->xin);
    BM_REQUIRE_PTR(a->weight);
    BM_REQUIRE_PTR(a->out_x);
    BM_OPTIONAL_PTR(a->bias);
    BM_OPTIONAL_PTR(a->window);
    BM_OPTIONAL_PTR(a->new_window);
    if (a->out_b != nullptr || a->out_c != nullptr) {
        BM_REQUIRE_PTR(a->out_b);
        BM_REQUIRE_PTR(a->out_c);
        BM_REQUIRE(a->split_x > 0 && a->split_bc > 0 && a->split_x + 2 * a->split_bc == a->channels &&
                       a->split_x % VEC == 0 && a->split_bc % VEC == 0,
                   BM_ERR_BAD_SHAPE, "split_x + 2 split_bc must equal channels, both multiples of 8");
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    bool staged = false;
    if (a->dtype == BM_DTYPE_BF16 && aligned16(a->xin)) {
        // TMA-staged kernel: 3-D map over [b][s][channels] with the projection's row stride
        CUtensorMap tm;
        const char* err = nullptr;
        const uint64_t dims[3] = {(uint64_t)a->channels, (uint64_t)a->seqlen, (uint64_t)a->batch};
        const uint64_t strides[2] = {(uint64_t)a->xin_stride * 2, (uint64_t)a->seqlen * a->xin_stride * 2};
        const uint32_t box[3] = {(uint32_t)kCtCh, (uint32_t)(kCtTok + a->kernel - 1), 1};
        if (tc::make_tensor_map_bf16(&tm, a->xin, 3, dims, strides, box, 0, &err)) {
            const int n_ctile = (int)cdiv(a->channels, kCtCh), n_ttile = (int)cdiv(a->seqlen, kCtTok);
            const int64_t ntiles = (int64_t)a->batch * n_ctile * n_ttile;
            if (ntiles <= INT32_MAX / 2) {
                static int sms = 0;
                if (sms == 0) {
                    int dev = 0;
                    cudaGetDevice(&dev);
                    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
                    if (sms <= 0) sms = 148;
                }
                int grid2 = (int)std::min<int64_t>(ntiles, 4 * (int64_t)sms);
                if (grid2 > n_ctile) grid2 -= grid2 % n_ctile;   // a CTA then keeps one channel tile (tile index = CTA + k * grid)
                const size_t smem = (size_t)kCtStages * kCtStageBytes + kCtStages * sizeof(uint64_t);
                cudaError_t e = cudaSuccess;
                switch (a->kernel) {
                    case 2:
                        e = cudaFuncSetAttribute(conv1d_silu_tma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                        if (e == cudaSuccess) conv1d_silu_tma_kernel<2><<<grid2, kCtThreads, smem, st>>>(*a, tm, n_ctile, n_ttile, (int)ntiles);
                        break;
                    case 3:
                        e = cudaFuncSetAttribute(conv1d_silu_tma_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                        if (e == cudaSuccess) conv1d_silu_tma_kernel<3><<<grid2, kCtThreads, smem, st>>>(*a, tm, n_ctile, n_ttile, (int)ntiles);
                        break;
                    default:
                        e = cudaFuncSetAttribute(conv1d_silu_tma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                        if (e == cudaSuccess) conv1d_silu_tma_kernel<4><<<grid2, kCtThreads, smem, st>>>(*a, tm, n_ctile, n_ttile, (int)ntiles);
                        break;
                }
                if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(conv1d_silu_tma_kernel)");
                if (int32_t e2 = check_launch("conv1d_silu_tma")) return e2;
                staged = true;
            }
        }
    }
    const int64_t threads = (int64_t)a->batch * cdiv(a->seqlen, TL) * (a->channels / VEC);
    const unsigned grid = (unsigned)cdiv(threads, 128);
    const bool f32 = a->dtype == BM_DTYPE_F32;
    if (!staged) switch (a->kernel) {
        case 2: f32 ? conv1d_silu_kernel<float, 2><<<grid, 128, 0, st>>>(*a) : conv1d_silu_kernel<__nv_bfloat16, 2><<<grid, 128, 0, st>>>(*a); break;
        case 3: f32 ? conv1d_silu_kernel<float, 3><<<grid, 128, 0, st>>>(*a) : conv1d_silu_kernel<__nv_bfloat16, 3><<<grid, 128, 0, st>>>(*a); break;
        default: f32 ? conv1d_silu_kernel<float, 4><<<grid, 128, 0, st>>>(*a) : conv1d_silu_kernel<__nv_bfloat16, 4><<<grid, 128, 0, st>>>(*a); break;
    }
    if (int32_t e = check_launch("conv1d_silu")) return e;
    if (a->new_window != nullptr) {
        BM_REQUIRE(a->new_window != a->window, BM_ERR_UNSUPPORTED, "new_window must not alias window");
        const int64_t total = (int64_t)a->batch * a->kernel * a->channels;
        if (f32) conv_window_kernel<float><<<(unsigned)cdiv(total, 256), 256, 0, st>>>(*a);
        else conv_window_kernel<__nv_bfloat16><<<(unsigned)cdiv(total, 256), 256, 0, st>>>(*a);
        return check_launch("conv_window");
    }
    return BM_OK;
}

extern "C" int32_t bm_rmsnorm_gated(const bm_rmsnorm_gated_args* a, void* stream) {
    clear_error();
    if (a == nullptr) return fail(BM_ERR_NULL_POINTER, "args is NULL");
    BM_REQUIRE(a->rows > 0 && a->width > 0, BM_ERR_BAD_SHAPE, "rows and width must be positive");
    BM_REQUIRE(a->dtype == BM_DTYPE_F32 || a->dtype == BM_DTYPE_BF16, BM_ERR_UNSUPPORTED, "dtype must be f32 or bf16");
    BM_REQUIRE(a->width % VEC == 0 && a->width <= NT * MAXV * VEC, BM_ERR_UNSUPPORTED, "width must be a multiple of 8, at most %d",
               NT * MAXV * VEC);
    const int esz = a->dtype == BM_DTYPE_F32 ? 4 : 2;
    BM_REQUIRE(((int64_t)a->x_stride * esz) % 16 == 0 && a->x_stride >= a->width &&
                   (a->z == nullptr || (((int64_t)a->z_stride * esz) % 16 == 0 && a->z_stride >= a->width)),
               BM_ERR_BAD_SHAPE, "rows must start 16-byte aligned and strides be at least the width");
    BM_REQUIRE_PTR(a->x);
    BM_REQUIRE_PTR(a->gamma);
    BM_REQUIRE_PTR(a->out);
    BM_OPTIONAL_PTR(a->z);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (a->dtype == BM_DTYPE_F32) launch_rmsnorm<float>(*a, st);
    else launch_rmsnorm<__nv_bfloat16>(*a, st);
    return check_launch("rmsnorm_gated");
}

extern "C" int32_t bm_mamba3_bc_prep(const bm_mamba3_bc_prep_args* a, void* stream) {
    clear_error();
    if (a == nullptr) return fail(BM_ERR_NULL_POINTER, "args is NULL");
    BM_REQUIRE(a->batch > 0 && a->seqlen > 0 && a->mimo_rank > 0 && a->ngroups > 0 && a->nheads > 0 && a->state_rank > 0,
               BM_ERR_BAD_SHAPE, "batch, seqlen, mimo_rank, ngroups, nheads, state_rank must be positive");
    BM_REQUIRE(a->nheads % a->ngroups == 0, BM_ERR_BAD_SHAPE, "nheads must be divisible by ngroups");
    BM_REQUIRE(a->state_rank % 16 == 0, BM_ERR_UNSUPPORTED, "state_rank must be a multiple of 16");
    BM_REQUIRE(a->rope_dim >= 0 && a->rope_dim <= a->state_rank && a->rope_dim % 2 == 0, BM_ERR_BAD_SHAPE,
               "rope_dim must be even and at most state_rank");
    BM_REQUIRE(a->dtype == BM_DTYPE_F32 || a->dtype == BM_DTYPE_BF16, BM_ERR_UNSUPPORTED, "dtype must be f32 or bf16");
    const int esz = a->dtype == BM_DTYPE_F32 ? 4 : 2;
    const int64_t row = (int64_t)a->mimo_rank * a->ngroups * a->state_rank;
    BM_REQUIRE(a->raw_stride >= row && ((int64_t)a->raw_stride * esz) % 16 == 0, BM_ERR_BAD_SHAPE,
               "raw_stride must cover m g r entries and keep rows 16-byte aligned");
    BM_REQUIRE_PTR(a->b_raw); BM_REQUIRE_PTR(a->c_raw); BM_REQUIRE_PTR(a->b_gamma); BM_REQUIRE_PTR(a->c_gamma);
    BM_REQUIRE_PTR(a->b_bias); BM_REQUIRE_PTR(a->c_bias); BM_REQUIRE_PTR(a->b_out); BM_REQUIRE_PTR(a->c_out);
    BM_OPTIONAL_PTR(a->angles);
    const size_t smem = 2 * (size_t)row * sizeof(float);
    BM_REQUIRE(smem <= 48 * 1024, BM_ERR_UNSUPPORTED, "m g r too large for the staging buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = (unsigned)((int64_t)a->batch * a->seqlen);
    if (a->dtype == BM_DTYPE_F32) mamba3_bc_prep_kernel<float><<<grid, 256, smem, st>>>(*a);
    else mamba3_bc_prep_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>(*a);
    return check_launch("mamba3_bc_prep");
}
