// Cumulative data-dependent rotation angles of Mamba-3's Complex2D rotation
// (src/mamba3/rotation/mod.rs:559-567, :653-679):
//   theta[b, s, h, j] = prev[b, h, j] + sum_{t <= s} dt[b, t, h] * range * pi * tanh(rot[b, t, j]).
// HBM-bound on the theta write (b*s*h*a*4 bytes).  The sequence is cut into chunks of kChunk tokens and
// scanned in three passes without any scratch memory: theta itself carries the chunk totals between them.
//   pass A  one thread per (b, chunk, block of kHB heads, j): the chunk's sums -> theta[b, last row of chunk, h, j]
//   pass B  one thread per (b, h, j): exclusive scan of those totals over the chunks, in place
//           (+ prev), and the wrapped final angle -> last
//   pass C  same threads as pass A: each reads its carries from the row pass B left them in, then walks the
//           chunk writing theta (the carry row is the last row it overwrites)
// A thread of passes A and C owns one rotation lane j for kHB heads, so tanh(rot) is evaluated once per
// kHB heads, dt[b, t, h] is a warp-uniform (broadcast) load, and every theta
// store is a full 128-byte line across the lanes of a warp.
#include "common.cuh"

using namespace bm;

namespace {

constexpr int kChunk = 64;   // tokens per chunk
constexpr int kHB = 8;       // heads per thread

__device__ __forceinline__ int chunk_last_row(int c, int S) { return min((c + 1) * kChunk, S) - 1; }

template <bool kWrite>
__global__ void angle_chunk_kernel(bm_angle_cumsum_args a, int nchunks, int nhb) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int A = a.nangles, H = a.nheads, S = a.seqlen;
    if (idx >= (int64_t)a.batch * nchunks * nhb * A) return;
    const int j = idx % A, hb = (idx / A) % nhb, c = (idx / ((int64_t)A * nhb)) % nchunks;
    const int b = idx / ((int64_t)A * nhb * nchunks);
    const int h0 = hb * kHB;
    const float scale = a.range * 3.14159265358979323846f;
    const int t0 = c * kChunk, t1 = min(t0 + kChunk, S);
    const float* rot = a.rot + (int64_t)b * S * A + j;
    const float* dt = a.dt + (int64_t)b * S * H + h0;
    float* th = a.theta + (int64_t)b * S * H * A + (int64_t)h0 * A + j;
    const int64_t carry_row = (int64_t)chunk_last_row(c, S) * H * A;
    float run[kHB];
#pragma unroll
    for (int k = 0; k < kHB; ++k) run[k] = (kWrite && h0 + k < H) ? th[carry_row + (int64_t)k * A] : 0.f;
    constexpr int U = 4;   // tokens whose loads are issued together
    int t = t0;
    for (; t + U <= t1; t += U) {
        float r[U], d[U][kHB];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            r[u] = rot[(int64_t)(t + u) * A];
#pragma unroll
            for (int k = 0; k < kHB; ++k) d[u][k] = h0 + k < H ? dt[(int64_t)(t + u) * H + k] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const float v = tanhf(r[u]) * scale;
            float* tr = th + (int64_t)(t + u) * H * A;
#pragma unroll
            for (int k = 0; k < kHB; ++k) {
                run[k] = fmaf(d[u][k], v, run[k]);
                if (kWrite && h0 + k < H) tr[(int64_t)k * A] = run[k];
            }
        }
    }
    for (; t < t1; ++t) {
        const float v = tanhf(rot[(int64_t)t * A]) * scale;
        float* tr = th + (int64_t)t * H * A;
#pragma unroll
        for (int k = 0; k < kHB; ++k) {
            if (h0 + k < H) {
                run[k] = fmaf(dt[(int64_t)t * H + k], v, run[k]);
                if (kWrite) tr[(int64_t)k * A] = run[k];
            }
        }
    }
    if (!kWrite) {
#pragma unroll
        for (int k = 0; k < kHB; ++k)
            if (h0 + k < H) th[carry_row + (int64_t)k * A] = run[k];
    }
}

__global__ void angle_carry_kernel(bm_angle_cumsum_args a, int nchunks) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int A = a.nangles, H = a.nheads, S = a.seqlen;
    if (idx >= (int64_t)a.batch * H * A) return;
    const int j = idx % A, h = (idx / A) % H, b = idx / ((int64_t)A * H);
    float* th = a.theta + ((int64_t)b * S * H + h) * A + j;
    float run = a.prev ? a.prev[idx] : 0.f;
    // the totals of up to 32 chunks are fetched together (independent loads), then scanned in registers
    constexpr int G = 32;
    for (int c0 = 0; c0 < nchunks; c0 += G) {
        float tot[G];
#pragma unroll
        for (int g = 0; g < G; ++g) tot[g] = c0 + g < nchunks ? th[(int64_t)chunk_last_row(c0 + g, S) * H * A] : 0.f;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            if (c0 + g < nchunks) {
                th[(int64_t)chunk_last_row(c0 + g, S) * H * A] = run;   // carry entering chunk c0 + g
                run += tot[g];
            }
        }
    }
    if (a.last) a.last[idx] = wrap_angle(run);
}

// Passes A and C with the chunk's inputs staged in shared memory: one CTA per (b, chunk) loads the chunk's
// rot rows (tanh and the range factor applied once per entry) and dt rows with coalesced reads, then a thread
// per (block of kHB heads, j) walks the tokens from shared memory, so the serial walk waits on no global load.
constexpr int kStThreads = 256;

template <bool kWrite>
__global__ void __launch_bounds__(kStThreads) angle_chunk_staged_kernel(bm_angle_cumsum_args a, int nchunks, int nhb) {
    extern __shared__ float ash[];
    const int A = a.nangles, H = a.nheads, S = a.seqlen;
    const int Hp = (H + 3) & ~3;                        // dt rows padded to 16 bytes
    const int Ap = (A + 3) & ~3;                        // so that the dt block starts 16-byte aligned
    float* vs = ash;                                    // [kChunk][A]  range * pi * tanh(rot)
    float* ds = ash + kChunk * Ap;                      // [kChunk][Hp] dt
    const int c = blockIdx.x % nchunks, b = blockIdx.x / nchunks;
    const int t0 = c * kChunk, nt = min(kChunk, S - t0);
    const float scale = a.range * 3.14159265358979323846f;
    const float* rot = a.rot + ((int64_t)b * S + t0) * A;
    const float* dt = a.dt + ((int64_t)b * S + t0) * H;
    for (int e = threadIdx.x; e < nt * A; e += kStThreads) vs[e] = tanhf(rot[e]) * scale;
    // dt rows: a warp per token row, so the padded layout needs no division per element
    for (int t = threadIdx.x >> 5; t < nt; t += kStThreads / 32)
        for (int h = threadIdx.x & 31; h < Hp; h += 32) ds[t * Hp + h] = h < H ? dt[t * H + h] : 0.f;
    __syncthreads();
    const int j = threadIdx.x % A, ngrp = kStThreads / A;
    if ((int)threadIdx.x >= ngrp * A) return;
    const int64_t carry_row = (int64_t)chunk_last_row(c, S) * H * A;
    const uint32_t Au = (uint32_t)A, row_stride = (uint32_t)H * Au;
    for (int hb = threadIdx.x / A; hb < nhb; hb += ngrp) {
        const int h0 = hb * kHB;
        float* th = a.theta + (int64_t)b * S * H * A + (int64_t)h0 * A + j;
        float run[kHB];
#pragma unroll
        for (int k = 0; k < kHB; ++k) run[k] = (kWrite && h0 + k < H) ? th[carry_row + (int64_t)k * A] : 0.f;
        float* tr = th + (int64_t)t0 * H * A;           // row of the token being written, advanced by one row per token
        const float* vp = vs + j;
        const float* dp = ds + h0;                      // h0 is a multiple of kHB = 8 and Hp of 4: 16-byte aligned
        if (h0 + kHB <= H) {
            // whole block of heads: two 128-bit broadcast reads of dt per token, no guards, stores at fixed offsets
#pragma unroll 4
            for (int t = 0; t < nt; ++t) {
                const float v = vp[t * A];
                const float4 d0 = *reinterpret_cast<const float4*>(dp + t * Hp);
                const float4 d1 = *reinterpret_cast<const float4*>(dp + t * Hp + 4);
                run[0] = fmaf(d0.x, v, run[0]), run[1] = fmaf(d0.y, v, run[1]);
                run[2] = fmaf(d0.z, v, run[2]), run[3] = fmaf(d0.w, v, run[3]);
                run[4] = fmaf(d1.x, v, run[4]), run[5] = fmaf(d1.y, v, run[5]);
                run[6] = fmaf(d1.z, v, run[6]), run[7] = fmaf(d1.w, v, run[7]);
                if (kWrite) {
#pragma unroll
                    for (int k = 0; k < kHB; ++k) tr[k * Au] = run[k];
                    tr += row_stride;
                }
            }
        } else {
            for (int t = 0; t < nt; ++t) {
                const float v = vp[t * A];
#pragma unroll
                for (int k = 0; k < kHB; ++k) {
                    if (h0 + k < H) {
                        run[k] = fmaf(dp[t * Hp + k], v, run[k]);
                        if (kWrite) tr[k * Au] = run[k];
                    }
                }
                tr += row_stride;
            }
        }
        if (!kWrite) {
#pragma unroll
            for (int k = 0; k < kHB; ++k)
                if (h0 + k < H) th[carry_row + (int64_t)k * A] = run[k];
        }
    }
}

}  // namespace

extern "C" int32_t bm_angle_cumsum(const bm_angle_cumsum_args* a, void* stream) {
    clear_error();
    if (a == nullptr) return fail(BM_ERR_NULL_POINTER, "args is NULL");
    BM_REQUIRE(a->batch > 0 && a->seqlen > 0 && a->nheads > 0 && a->nangles > 0, BM_ERR_BAD_SHAPE,
               "batch, seqlen, nheads, nangles must be positive");
    BM_REQUIRE_PTR(a->rot);
    BM_REQUIRE_PTR(a->dt);
    BM_REQUIRE_PTR(a->theta);
    BM_OPTIONAL_PTR(a->prev);
    BM_OPTIONAL_PTR(a->last);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int nchunks = (a->seqlen + kChunk - 1) / kChunk;
    const int nhb = (a->nheads + kHB - 1) / kHB;
    const int64_t per_chunk = (int64_t)a->batch * nchunks * nhb * a->nangles;
    const int64_t per_lane = (int64_t)a->batch * a->nheads * a->nangles;
    const size_t smem = (size_t)kChunk * (((a->nangles + 3) & ~3) + ((a->nheads + 3) & ~3)) * sizeof(float);
    const bool staged = a->nangles <= kStThreads && smem <= 48 * 1024 && (int64_t)a->batch * nchunks <= INT32_MAX;
    const unsigned sgrid = (unsigned)((int64_t)a->batch * nchunks);
    if (staged) angle_chunk_staged_kernel<false><<<sgrid, kStThreads, smem, st>>>(*a, nchunks, nhb);
    else angle_chunk_kernel<false><<<(unsigned)cdiv(per_chunk, 128), 128, 0, st>>>(*a, nchunks, nhb);
    if (int32_t e = check_launch("angle_cumsum (chunk totals)")) return e;
    angle_carry_kernel<<<(unsigned)cdiv(per_lane, 128), 128, 0, st>>>(*a, nchunks);
    if (int32_t e = check_launch("angle_cumsum (carries)")) return e;
    if (staged) angle_chunk_staged_kernel<true><<<sgrid, kStThreads, smem, st>>>(*a, nchunks, nhb);
    else angle_chunk_kernel<true><<<(unsigned)cdiv(per_chunk, 128), 128, 0, st>>>(*a, nchunks, nhb);
    return check_launch("angle_cumsum (write)");
}
