// Mamba-2 chunked SSD backward on the Blackwell tensor cores (tcgen05 / TMEM / TMA): bf16 operands,
// float32 accumulation, float32 gradient of the recurrent state carried in registers.
//
// Gradients of combined_backward (src/mamba2/ssd/serial_recalculated/combined_backward.rs:126-590) with the
// 128-token tile as the chunk.  One CTA per SM; the tiles of all (batch, head) units, laid end to end, are
// cut into one contiguous range per CTA; inside a unit a CTA walks its tiles in REVERSE order with dh, the
// gradient of the state leaving the tile, in registers.  A unit that straddles two ranges is walked by two
// CTAs: the one with the later tiles does them first thing and hands dh over through the workspace, the
// other one reaches its earlier tiles of that unit as the last thing it does.  The state entering
// every tile comes from a forward pass of the tensor-core kernel run first (chunk states at tile
// granularity).  Per tile, with c_t the inclusive cumulative log decay inside the tile, f[t,s] =
// exp(c_t - c_s) [s <= t], e_t = exp(c_t), k_s = exp(c_end - c_s) (every factor <= 1, so any decay is safe):
//     CB  = C B^T                 dM = dY (dt X)^T                         tcgen05, phase 1
//     M   = bf16(CB f)            dCB = bf16(dM f)                         mask pass, TMEM -> shared memory
//     dC  = dCB B   + (e dY) h_in^T                                        tcgen05, phase 2
//     dB  = dCB^T C + (k dt X) dh^T
//     G   = M^T dY        Gi = B dh        dhC = C^T (e dY)        Y2 = C h_in^T
//     dx  = dt (G + k Gi) + D dy          ddt (direct) = sum_p x (G + k Gi)
//     d(dt A)_k = sum_{t >= k} [rowsum_t(W) - colsum_t(W) + e_t dy_t . Y2_t] + sum_{s < k} k_s dt_s x_s . Gi_s
//                 + exp(c_end) <dh, h_in>,   W = (CB f) o dM in float32
//            (the pair terms cancel exactly between the row and the column sums of the same W; the state terms
//             are arranged so that no two large sums cancel)
//     dh <- exp(c_end) dh + dhC
// The kernel is phase-synchronous (all 512 threads walk the same phases, one elected thread issues the MMAs
// of a phase and everybody waits for their commit); thread (row = tid % 128, quarter = tid / 128) owns one
// row and one quarter of the columns of every accumulator.  Gradients leave through shared-memory staging
// and per-row bulk copies (dx) or bulk reduce-adds (dB, dC: summed over the heads of a group).  Every
// wait is bounded; a wait that runs out stores BM_ERR_TIMEOUT in the workspace status word and the CTA leaves.
#include "ssd2_tc.cuh"
#include "tc_common.cuh"

namespace bm {
namespace tc {

namespace {

constexpr int T = 128, P = 64, R = 128;
constexpr int kThreads = 512;
constexpr uint32_t kPanel = 16384;            // [128 rows x 128 B]

// shared-memory map (bytes from a 1024-aligned base)
constexpr uint32_t kOffX = 0;                 // X -> dt X (Xd) -> k dt X (Xw), one panel
constexpr uint32_t kOffDy = 1 * kPanel;       // dY
constexpr uint32_t kOffDye = 2 * kPanel;      // e dY
constexpr uint32_t kOffB = 3 * kPanel;        // 2 panels
constexpr uint32_t kOffC = 5 * kPanel;        // 2 panels
constexpr uint32_t kOffM = 7 * kPanel;        // masked CB, 2 panels [t][s]
constexpr uint32_t kOffDcb = 9 * kPanel;      // masked dM, 2 panels [t][s]
constexpr uint32_t kOffH = 11 * kPanel;       // h_in bf16 [r][p]
constexpr uint32_t kOffDh = 12 * kPanel;      // dh bf16 [r][p]
constexpr uint32_t kOperandBytes = 13 * kPanel;   // 208 KB
// output staging aliases the operand area once the MMAs of phase 2 have completed
constexpr uint32_t kRowC = 528, kRowX = 272;  // padded row strides (bytes) of the float32 staging tiles
constexpr uint32_t kOffStC = 0, kOffStB = 128 * kRowC, kOffStX = 2 * 128 * kRowC;
static_assert(kOffStX + 128 * kRowX <= kOperandBytes, "staging does not fit the operand area");
constexpr uint32_t kOffSc = kOperandBytes;    // per-tile scalars, float[128] each
enum { kScCum = 0, kScDt, kScK, kScE, kScColk, kScColW, kScPa, kScPb = kScPa + 4, kScPd = kScPb + 4, kScCount = kScPd + 4 };
constexpr uint32_t kOffRed = kOffSc + kScCount * 128 * 4;   // 8 floats of block reductions
constexpr uint32_t kOffBar = kOffRed + 64;
constexpr uint32_t kSmemBytes = kOffBar + 64 + 1024;
static_assert(kSmemBytes <= 232448, "over the 227 KB shared-memory limit of a CTA");

// TMEM columns
constexpr uint32_t kColCB = 0, kColDM = 128, kColDC = 256, kColDB = 384;   // phase 1 / phase 2 accumulators
constexpr uint32_t kColG = 0, kColGi = 64, kColDhC = 128, kColY2 = 192;    // phase 2, over the consumed CB / dM

struct Bars {
    uint64_t ld_full, mma1, mma2;
    uint32_t tmem_base;
    uint32_t failed;
};

struct alignas(64) BwdParams {
    CUtensorMap tm_x, tm_dy, tm_b, tm_c;
    const float* dt;
    const float* a;
    const float* d;
    const float* chunk_states;   // [b, n, h, p, r] state entering every tile (from the forward pass)
    const float* dh_final;
    const __nv_bfloat16* x;      // raw pointers for the row-local products
    const __nv_bfloat16* dy;
    float* dx;
    float* ddt;
    float* da;
    float* db;
    float* dc;
    float* dd;
    float* dh0;
    int* status;
    int* handoff_flags;          // [grid] warps of CTA c that have stored the dh its first piece ends with
    float* handoff;              // [grid][P][R]
    int B, S, H, G, NT, num_units;
    int share_q, share_r;        // (num_units * NT) / grid and the remainder
};

__device__ __forceinline__ void bulk_store_row(float* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_add_row(float* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes)
                 : "memory");
}

// Bounded wait of the whole CTA on one mbarrier phase, followed by a CTA-wide agreement: true when any
// thread's budget ran out (every thread then leaves together).
__device__ __forceinline__ bool cta_wait_failed(uint64_t* bar, uint32_t parity) {
    uint32_t n = 0;
    bool ok = true;
#pragma unroll 1
    while (!mbar_try_wait(bar, parity))
        if (++n >= kWaitBudget) {
            ok = false;
            break;
        }
    return __syncthreads_or(!ok) != 0;
}

__global__ void __launch_bounds__(kThreads, 1) ssd2_bwd_tc_kernel(const __grid_constant__ BwdParams prm) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    Bars* bars = reinterpret_cast<Bars*>(smem + kOffBar);
    float* sc = reinterpret_cast<float*>(smem + kOffSc);
    float* red = reinterpret_cast<float*>(smem + kOffRed);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = tid & 127, pq = tid >> 7;   // the accumulator row and column quarter this thread owns

    if (tid == 0) {
        mbar_init(&bars->ld_full, 1);
        mbar_init(&bars->mma1, 1);
        mbar_init(&bars->mma2, 1);
        bars->failed = 0;
        fence_mbar_init();
        tma_prefetch_desc(&prm.tm_x);
        tma_prefetch_desc(&prm.tm_dy);
        tma_prefetch_desc(&prm.tm_b);
        tma_prefetch_desc(&prm.tm_c);
    }
    if (warp == 2) {
        tmem_alloc(&bars->tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const int hpg = prm.H / prm.G;
    const float log2e = 1.4426950408889634f;
    uint32_t phase = 0;   // every barrier completes once per tile

    // tiles [lo, hi) of the global (unit-major) tile sequence: share_q per CTA, one more for the first share_r
    const int cta = blockIdx.x, extra = cta < prm.share_r ? cta : prm.share_r;
    const int lo = cta * prm.share_q + extra, hi = lo + prm.share_q + (cta < prm.share_r ? 1 : 0);
    const int u_first = lo / prm.NT, u_last = (hi - 1) / prm.NT;

    for (int unit = u_first; unit <= u_last; ++unit) {
        const int b = unit / prm.H, h = unit - b * prm.H, g = h / hpg;
        const int i_lo = unit == u_first ? lo - u_first * prm.NT : 0;          // this CTA's tiles of the unit
        const int i_hi = unit == u_last ? hi - u_last * prm.NT : prm.NT;
        const int64_t state_base = ((int64_t)b * prm.H + h) * P * R;
        const float ah = prm.a[h], dskip = prm.d ? prm.d[h] : 0.f;
        // dh = gradient of the state leaving the current tile: the caller's at the end of the unit, else what
        // the next CTA stored when it finished the later tiles of this unit
        float dh[16];
        {
            const float* src = prm.dh_final ? prm.dh_final + state_base : nullptr;
            if (i_hi != prm.NT) {
                const int* flag = prm.handoff_flags + cta + 1;
                uint32_t n = 0;
                bool ok = true;
#pragma unroll 1
                while (ld_acquire_gpu(flag) < kThreads / 32)
                    if (++n >= kWaitBudget) {
                        ok = false;
                        break;
                    }
                if (__syncthreads_or(!ok)) goto timed_out;
                src = prm.handoff + (int64_t)(cta + 1) * P * R;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) dh[j] = src ? src[(int64_t)(16 * pq + j) * R + row] : 0.f;
        }
        float da_acc = 0.f, dd_acc = 0.f;   // meaningful in thread 0 (dA) and as per-thread partials (dD)

        for (int i = i_hi - 1; i >= i_lo; --i, phase ^= 1) {
            const int s0 = i * T, left = prm.S - s0;
            // ---- loads of the tile
            if (tid == 0) {
                mbar_expect_tx(&bars->ld_full, 6 * kPanel);
                tma_load_4d(smem + kOffX, &prm.tm_x, &bars->ld_full, 0, h, s0, b);
                tma_load_4d(smem + kOffDy, &prm.tm_dy, &bars->ld_full, 0, h, s0, b);
                tma_load_4d(smem + kOffB, &prm.tm_b, &bars->ld_full, 0, g, s0, b);
                tma_load_4d(smem + kOffB + kPanel, &prm.tm_b, &bars->ld_full, 64, g, s0, b);
                tma_load_4d(smem + kOffC, &prm.tm_c, &bars->ld_full, 0, g, s0, b);
                tma_load_4d(smem + kOffC + kPanel, &prm.tm_c, &bars->ld_full, 64, g, s0, b);
            }
            // ---- per-token scalars (warp 1): log2-domain cumulative decay and the factors derived from it
            if (warp == 1) {
                float d4[4], c4[4], run = 0.f;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int t = lane * 4 + k;
                    d4[k] = t < left ? prm.dt[((int64_t)b * prm.S + s0 + t) * prm.H + h] : 0.f;
                    run = fmaf(d4[k], ah * log2e, run);
                    c4[k] = run;
                }
                float incl = run;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += up;
                }
                const float excl = incl - run;
                const float cend = __shfl_sync(0xffffffffu, incl, 31);
                const float cblk = __shfl_sync(0xffffffffu, incl, (lane & ~7) | 7);   // end of the 32-token block
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int t = lane * 4 + k;
                    const float c = excl + c4[k];
                    sc[kScCum * 128 + t] = c;
                    sc[kScDt * 128 + t] = d4[k];
                    sc[kScK * 128 + t] = ex2(cend - c);
                    sc[kScE * 128 + t] = ex2(c);
                    sc[kScColk * 128 + t] = ex2(cblk - c);
                    sc[kScColW * 128 + t] = 0.f;
                }
            }
            // ---- the state entering the tile -> bf16 operand [r][p]; dh -> bf16 operand [r][p]; <dh, h_in> over
            // this thread's 16 elements
            float dot = 0.f;
            {
                float hin[16];
                const float* cs = prm.chunk_states + (((int64_t)b * prm.NT + i) * prm.H + h) * P * R;
#pragma unroll
                for (int j = 0; j < 16; ++j) hin[j] = cs[(int64_t)(16 * pq + j) * R + row];
#pragma unroll
                for (int j = 0; j < 16; ++j) dot = fmaf(dh[j], hin[j], dot);
                uint4 v0, v1, w0, w1;
                v0 = make_uint4(pack_bf16x2(hin[0], hin[1]), pack_bf16x2(hin[2], hin[3]), pack_bf16x2(hin[4], hin[5]), pack_bf16x2(hin[6], hin[7]));
                v1 = make_uint4(pack_bf16x2(hin[8], hin[9]), pack_bf16x2(hin[10], hin[11]), pack_bf16x2(hin[12], hin[13]), pack_bf16x2(hin[14], hin[15]));
                w0 = make_uint4(pack_bf16x2(dh[0], dh[1]), pack_bf16x2(dh[2], dh[3]), pack_bf16x2(dh[4], dh[5]), pack_bf16x2(dh[6], dh[7]));
                w1 = make_uint4(pack_bf16x2(dh[8], dh[9]), pack_bf16x2(dh[10], dh[11]), pack_bf16x2(dh[12], dh[13]), pack_bf16x2(dh[14], dh[15]));
                *reinterpret_cast<uint4*>(smem + kOffH + sw128_offset(row, 2 * pq)) = v0;
                *reinterpret_cast<uint4*>(smem + kOffH + sw128_offset(row, 2 * pq + 1)) = v1;
                *reinterpret_cast<uint4*>(smem + kOffDh + sw128_offset(row, 2 * pq)) = w0;
                *reinterpret_cast<uint4*>(smem + kOffDh + sw128_offset(row, 2 * pq + 1)) = w1;
            }
            if (cta_wait_failed(&bars->ld_full, phase)) goto timed_out;   // also publishes the scalars
            // ---- operand scaling: X -> dt X, e dY (this thread: 16 elements of row `row`)
            uint4 xr[2], dyr[2];   // the unscaled x and dy of this thread's 16 elements, packed bf16
            {
                const float dts = sc[kScDt * 128 + row], et = sc[kScE * 128 + row];
#pragma unroll
                for (int c2 = 0; c2 < 2; ++c2) {
                    const uint32_t off = sw128_offset(row, 2 * pq + c2);
                    xr[c2] = *reinterpret_cast<const uint4*>(smem + kOffX + off);
                    dyr[c2] = *reinterpret_cast<const uint4*>(smem + kOffDy + off);
                    const uint32_t* xs = &xr[c2].x;
                    const uint32_t* ys = &dyr[c2].x;
                    uint32_t xo[4], yo[4];
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const float2 xf = unpack_bf16x2(xs[m]), yf = unpack_bf16x2(ys[m]);
                        xo[m] = pack_bf16x2(xf.x * dts, xf.y * dts);
                        yo[m] = pack_bf16x2(yf.x * et, yf.y * et);
                    }
                    *reinterpret_cast<uint4*>(smem + kOffX + off) = make_uint4(xo[0], xo[1], xo[2], xo[3]);
                    *reinterpret_cast<uint4*>(smem + kOffDye + off) = make_uint4(yo[0], yo[1], yo[2], yo[3]);
                }
            }
            fence_proxy_async_smem();
            __syncthreads();
            // ---- phase 1: CB = C B^T, dM = dY (dt X)^T
            if (tid == 0) {
                tc_fence_after();
                const uint32_t id128 = umma_idesc_bf16(128, 128, false, false);
                const uint64_t dc_ = umma_desc_kmajor(smem_u32(smem + kOffC)), db_ = umma_desc_kmajor(smem_u32(smem + kOffB));
#pragma unroll 1
                for (int k = 0; k < 8; ++k) {
                    const uint32_t off = (k >> 2) * kPanel + (k & 3) * 32;
                    umma_ss(tmem + kColCB, desc_advance(dc_, off), desc_advance(db_, off), id128, k > 0);
                }
                const uint64_t ddy = umma_desc_kmajor(smem_u32(smem + kOffDy)), dxd = umma_desc_kmajor(smem_u32(smem + kOffX));
#pragma unroll 1
                for (int k = 0; k < 4; ++k) umma_ss(tmem + kColDM, desc_advance(ddy, k * 32), desc_advance(dxd, k * 32), id128, k > 0);
                umma_commit(&bars->mma1);
            }
            if (cta_wait_failed(&bars->mma1, phase)) goto timed_out;
            tc_fence_after();
            // ---- mask pass: columns [32 pq, 32 pq + 32) of row `row`; X: dt X -> k dt X for the state terms
            {
                const int q = row >> 5;                       // 32-row block of this row
                uint32_t om[16], od[16];
                float wrow = 0.f;
                if (pq <= q) {
                    uint32_t cb[32], dm[32];
                    tmem_ld32(lane_addr + kColCB + 32 * pq, cb);
                    tmem_ld32(lane_addr + kColDM + 32 * pq, dm);
                    tmem_wait_ld();
                    const float ct = sc[kScCum * 128 + row];
                    if (pq < q) {
                        const float rf = ex2(ct - sc[kScCum * 128 + 32 * pq + 31]);
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float f0 = rf * sc[kScColk * 128 + 32 * pq + 2 * j], f1 = rf * sc[kScColk * 128 + 32 * pq + 2 * j + 1];
                            const float m0 = __uint_as_float(cb[2 * j]) * f0, m1 = __uint_as_float(cb[2 * j + 1]) * f1;
                            om[j] = pack_bf16x2(m0, m1);
                            od[j] = pack_bf16x2(__uint_as_float(dm[2 * j]) * f0, __uint_as_float(dm[2 * j + 1]) * f1);
                            cb[2 * j] = __float_as_uint(m0 * __uint_as_float(dm[2 * j]));          // W
                            cb[2 * j + 1] = __float_as_uint(m1 * __uint_as_float(dm[2 * j + 1]));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int s_ = 32 * pq + 2 * j;
                            const float f0 = s_ <= row ? ex2(ct - sc[kScCum * 128 + s_]) : 0.f;
                            const float f1 = s_ + 1 <= row ? ex2(ct - sc[kScCum * 128 + s_ + 1]) : 0.f;
                            const float m0 = __uint_as_float(cb[2 * j]) * f0, m1 = __uint_as_float(cb[2 * j + 1]) * f1;
                            om[j] = pack_bf16x2(m0, m1);
                            od[j] = pack_bf16x2(__uint_as_float(dm[2 * j]) * f0, __uint_as_float(dm[2 * j + 1]) * f1);
                            cb[2 * j] = __float_as_uint(m0 * __uint_as_float(dm[2 * j]));
                            cb[2 * j + 1] = __float_as_uint(m1 * __uint_as_float(dm[2 * j + 1]));
                        }
                    }
                    // W = M o dM: row sum (this thread's 32 columns) and, through a transposing butterfly over
                    // the warp's 32 rows, the column sums of the same values
#pragma unroll
                    for (int j = 0; j < 32; ++j) wrow += __uint_as_float(cb[j]);
#pragma unroll
                    for (int o = 16; o >= 1; o >>= 1) {
#pragma unroll
                        for (int j = 0; j < o; ++j) {
                            const bool up = (lane & o) != 0;
                            const float send = up ? __uint_as_float(cb[j]) : __uint_as_float(cb[j + o]);
                            const float keep = up ? __uint_as_float(cb[j + o]) : __uint_as_float(cb[j]);
                            cb[j] = __float_as_uint(keep + __shfl_xor_sync(0xffffffffu, send, o));
                        }
                    }
                    atomicAdd(&sc[kScColW * 128 + 32 * pq + lane], __uint_as_float(cb[0]));
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) om[j] = od[j] = 0u;
                }
                sc[(kScPa + pq) * 128 + row] = wrow;
                const uint32_t pan = (pq >> 1) * kPanel;
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    const uint32_t off = pan + sw128_offset(row, (pq & 1) * 4 + c4);
                    *reinterpret_cast<uint4*>(smem + kOffM + off) = make_uint4(om[4 * c4], om[4 * c4 + 1], om[4 * c4 + 2], om[4 * c4 + 3]);
                    *reinterpret_cast<uint4*>(smem + kOffDcb + off) = make_uint4(od[4 * c4], od[4 * c4 + 1], od[4 * c4 + 2], od[4 * c4 + 3]);
                }
                // the scaled input of the state terms: k_s dt_s x_s (dM has been formed from dt_s x_s already)
                const float ks = sc[kScK * 128 + row];
#pragma unroll
                for (int c2 = 0; c2 < 2; ++c2) {
                    const uint32_t off = sw128_offset(row, 2 * pq + c2);
                    uint4 v = *reinterpret_cast<const uint4*>(smem + kOffX + off);
                    uint32_t* w = &v.x;
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const float2 f = unpack_bf16x2(w[m]);
                        w[m] = pack_bf16x2(f.x * ks, f.y * ks);
                    }
                    *reinterpret_cast<uint4*>(smem + kOffX + off) = v;
                }
            }
            tc_fence_before();
            fence_proxy_async_smem();
            __syncthreads();
            // ---- phase 2
            if (tid == 0) {
                tc_fence_after();
                const uint32_t b_sm = smem_u32(smem + kOffB), c_sm = smem_u32(smem + kOffC), m_sm = smem_u32(smem + kOffM);
                const uint32_t dcb_sm = smem_u32(smem + kOffDcb), x_sm = smem_u32(smem + kOffX), dy_sm = smem_u32(smem + kOffDy);
                const uint32_t dye_sm = smem_u32(smem + kOffDye), h_sm = smem_u32(smem + kOffH), dh_sm = smem_u32(smem + kOffDh);
                const uint32_t id_kk = umma_idesc_bf16(128, 128, false, false), id_kmn = umma_idesc_bf16(128, 128, false, true);
                const uint32_t id_mm = umma_idesc_bf16(128, 128, true, true);
                const uint32_t id64_mm = umma_idesc_bf16(128, 64, true, true), id64_kmn = umma_idesc_bf16(128, 64, false, true);
                // dC = dCB B + (e dY) h_in^T
                {
                    const uint64_t da_ = umma_desc_kmajor(dcb_sm), db_ = umma_desc_mnmajor(b_sm, kPanel);
#pragma unroll 1
                    for (int k = 0; k < 8; ++k)
                        umma_ss(tmem + kColDC, desc_advance(da_, (k >> 2) * kPanel + (k & 3) * 32), desc_advance(db_, k * 2048), id_kmn, k > 0);
                    const uint64_t dy_ = umma_desc_kmajor(dye_sm), dh_ = umma_desc_kmajor(h_sm);
#pragma unroll 1
                    for (int k = 0; k < 4; ++k) umma_ss(tmem + kColDC, desc_advance(dy_, k * 32), desc_advance(dh_, k * 32), id_kk, true);
                }
                // dB = dCB^T C + (k dt X) dh^T
                {
                    const uint64_t da_ = umma_desc_mnmajor(dcb_sm, kPanel), dc_ = umma_desc_mnmajor(c_sm, kPanel);
#pragma unroll 1
                    for (int k = 0; k < 8; ++k) umma_ss(tmem + kColDB, desc_advance(da_, k * 2048), desc_advance(dc_, k * 2048), id_mm, k > 0);
                    const uint64_t dx_ = umma_desc_kmajor(x_sm), dh_ = umma_desc_kmajor(dh_sm);
#pragma unroll 1
                    for (int k = 0; k < 4; ++k) umma_ss(tmem + kColDB, desc_advance(dx_, k * 32), desc_advance(dh_, k * 32), id_kk, true);
                }
                // G = M^T dY, Gi = B dh, dhC = C^T (e dY)
                {
                    const uint64_t dm_ = umma_desc_mnmajor(m_sm, kPanel), dy_ = umma_desc_mnmajor(dy_sm, kPanel);
#pragma unroll 1
                    for (int k = 0; k < 8; ++k) umma_ss(tmem + kColG, desc_advance(dm_, k * 2048), desc_advance(dy_, k * 2048), id64_mm, k > 0);
                    const uint64_t db_ = umma_desc_kmajor(b_sm), dh_ = umma_desc_mnmajor(dh_sm, kPanel);
#pragma unroll 1
                    for (int k = 0; k < 8; ++k)
                        umma_ss(tmem + kColGi, desc_advance(db_, (k >> 2) * kPanel + (k & 3) * 32), desc_advance(dh_, k * 2048), id64_kmn, k > 0);
                    const uint64_t dc_ = umma_desc_mnmajor(c_sm, kPanel), de_ = umma_desc_mnmajor(dye_sm, kPanel);
#pragma unroll 1
                    for (int k = 0; k < 8; ++k) umma_ss(tmem + kColDhC, desc_advance(dc_, k * 2048), desc_advance(de_, k * 2048), id64_mm, k > 0);
                    const uint64_t dck = umma_desc_kmajor(c_sm), dhm = umma_desc_mnmajor(h_sm, kPanel);
#pragma unroll 1
                    for (int k = 0; k < 8; ++k)
                        umma_ss(tmem + kColY2, desc_advance(dck, (k >> 2) * kPanel + (k & 3) * 32), desc_advance(dhm, k * 2048), id64_kmn, k > 0);
                }
                umma_commit(&bars->mma2);
            }
            if (cta_wait_failed(&bars->mma2, phase)) goto timed_out;
            tc_fence_after();
            // ---- epilogue (operand buffers are free now: staging aliases them)
            {
                uint32_t acc[32];
                tmem_ld32(lane_addr + kColDC + 32 * pq, acc);
                tmem_wait_ld();
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4)
                    *reinterpret_cast<uint4*>(smem + kOffStC + row * kRowC + pq * 128 + c4 * 16) =
                        make_uint4(acc[4 * c4], acc[4 * c4 + 1], acc[4 * c4 + 2], acc[4 * c4 + 3]);
                tmem_ld32(lane_addr + kColDB + 32 * pq, acc);
                tmem_wait_ld();
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4)
                    *reinterpret_cast<uint4*>(smem + kOffStB + row * kRowC + pq * 128 + c4 * 16) =
                        make_uint4(acc[4 * c4], acc[4 * c4 + 1], acc[4 * c4 + 2], acc[4 * c4 + 3]);
                // dx and the direct part of ddt: 16 columns of row `row`
                uint32_t gg[16], gi[16], dc16[16], y2[16];
                tmem_ld16(lane_addr + kColG + 16 * pq, gg);
                tmem_ld16(lane_addr + kColGi + 16 * pq, gi);
                tmem_ld16(lane_addr + kColDhC + 16 * pq, dc16);
                tmem_ld16(lane_addr + kColY2 + 16 * pq, y2);
                tmem_wait_ld();
                const float dts = sc[kScDt * 128 + row], ks = sc[kScK * 128 + row];
                float pd = 0.f, pin = 0.f, pgi = 0.f, dxo[16];   // direct ddt; dy . Y2; x . Gi
#pragma unroll
                for (int c2 = 0; c2 < 2; ++c2) {
                    const uint32_t* xs = &xr[c2].x;
                    const uint32_t* ys = &dyr[c2].x;
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const float2 xf = unpack_bf16x2(xs[m]), yf = unpack_bf16x2(ys[m]);
                        const int j = 8 * c2 + 2 * m;
                        const float g0 = fmaf(ks, __uint_as_float(gi[j]), __uint_as_float(gg[j]));
                        const float g1 = fmaf(ks, __uint_as_float(gi[j + 1]), __uint_as_float(gg[j + 1]));
                        pd = fmaf(xf.x, g0, pd);
                        pd = fmaf(xf.y, g1, pd);
                        pin = fmaf(yf.x, __uint_as_float(y2[j]), pin);
                        pin = fmaf(yf.y, __uint_as_float(y2[j + 1]), pin);
                        pgi = fmaf(xf.x, __uint_as_float(gi[j]), pgi);
                        pgi = fmaf(xf.y, __uint_as_float(gi[j + 1]), pgi);
                        dxo[j] = fmaf(dts, g0, dskip * yf.x);
                        dxo[j + 1] = fmaf(dts, g1, dskip * yf.y);
                        dd_acc = fmaf(xf.x, yf.x, dd_acc);
                        dd_acc = fmaf(xf.y, yf.y, dd_acc);
                    }
                }
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4)
                    *reinterpret_cast<float4*>(smem + kOffStX + row * kRowX + pq * 64 + c4 * 16) =
                        make_float4(dxo[4 * c4], dxo[4 * c4 + 1], dxo[4 * c4 + 2], dxo[4 * c4 + 3]);
                // the readout term joins the row sum of W this thread stored in the mask pass
                sc[(kScPa + pq) * 128 + row] += sc[kScE * 128 + row] * pin;
                sc[(kScPb + pq) * 128 + row] = ks * dts * pgi;
                sc[(kScPd + pq) * 128 + row] = pd;
                // the state gradient entering the tile
                const float decay = ex2(sc[kScCum * 128 + 127]);
#pragma unroll
                for (int j = 0; j < 16; ++j) dh[j] = fmaf(decay, dh[j], __uint_as_float(dc16[j]));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                if (tid == 0) red[0] = 0.f;
                tc_fence_before();
                fence_proxy_async_smem();
                __syncthreads();
                if (lane == 0) atomicAdd(&red[0], dot * decay);
                // gradient rows leave: dx by a bulk copy, dB / dC by a bulk reduce-add into the group's rows
                if (tid < 128 && tid < left) {
                    const int64_t tok = (int64_t)b * prm.S + s0 + tid;
                    bulk_store_row(prm.dx + (tok * prm.H + h) * P, smem + kOffStX + tid * kRowX, P * 4);
                    bulk_add_row(prm.dc + (tok * prm.G + g) * R, smem + kOffStC + tid * kRowC, R * 4);
                    bulk_add_row(prm.db + (tok * prm.G + g) * R, smem + kOffStB + tid * kRowC, R * 4);
                    tma_store_commit();
                }
                __syncthreads();
                // ---- suffix sum of dc over the tile -> d(dt A); ddt and dA (warp 0)
                if (warp == 0) {
                    float v[4], u[4], run = 0.f, prun = 0.f;
#pragma unroll
                    for (int k = 3; k >= 0; --k) {
                        const int t = lane * 4 + k;
                        float dcv = -sc[kScColW * 128 + t];
#pragma unroll
                        for (int w = 0; w < 4; ++w) dcv += sc[(kScPa + w) * 128 + t];
                        run += dcv;
                        v[k] = run;
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {   // exclusive prefix of the state-input terms
                        const int t = lane * 4 + k;
                        u[k] = prun;
#pragma unroll
                        for (int w = 0; w < 4; ++w) prun += sc[(kScPb + w) * 128 + t];
                    }
                    float incl = run, pincl = prun;   // suffix / prefix over lanes
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const float dn = __shfl_down_sync(0xffffffffu, incl, o);
                        const float up = __shfl_up_sync(0xffffffffu, pincl, o);
                        if (lane + o < 32) incl += dn;
                        if (lane >= o) pincl += up;
                    }
                    const float after = incl - run + (pincl - prun) + red[0];   // lanes above, lanes below, exp(c_end) <dh, h_in>
                    float dal = 0.f;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int t = lane * 4 + k;
                        const float dda = v[k] + u[k] + after;
                        const float dts2 = sc[kScDt * 128 + t];
                        float pdv = 0.f;
#pragma unroll
                        for (int w = 0; w < 4; ++w) pdv += sc[(kScPd + w) * 128 + t];
                        if (t < left) prm.ddt[((int64_t)b * prm.S + s0 + t) * prm.H + h] = fmaf(ah, dda, pdv);
                        dal = fmaf(dts2, dda, dal);
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) dal += __shfl_xor_sync(0xffffffffu, dal, o);
                    da_acc += dal;
                }
                // the staging tiles must have been read before the next tile's loads overwrite them
                if (tid < 128) tma_store_wait_read<0>();
                __syncthreads();
            }
        }
        // ---- end of this CTA's tiles of the unit: dh0 at the start of the unit, else the hand-over; dA, dD
        {
            float* dst = i_lo == 0 ? prm.dh0 + state_base : prm.handoff + (int64_t)cta * P * R;
#pragma unroll
            for (int j = 0; j < 16; ++j) dst[(int64_t)(16 * pq + j) * R + row] = dh[j];
            if (i_lo != 0) {
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicAdd(prm.handoff_flags + cta, 1);
            }
        }
        if (tid == 0) atomicAdd(prm.da + h, da_acc);
        if (prm.dd != nullptr) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dd_acc += __shfl_xor_sync(0xffffffffu, dd_acc, o);
            if (lane == 0) atomicAdd(prm.dd + h, dd_acc);
        }
    }
    goto done;
timed_out:
    if (tid == 0) {
        atomicExch(prm.status, (int)BM_ERR_TIMEOUT);
        // what this thread may still have in flight (loads, MMAs of the current tile) before shared memory and
        // TMEM go back; bounded again
        uint64_t* bs[3] = {&bars->ld_full, &bars->mma1, &bars->mma2};
        for (int k = 0; k < 3; ++k)
            for (uint32_t n = 0; n < kWaitBudget && !mbar_try_wait(bs[k], phase); ++n) {}
    }
done:
    if (tid < 128) tma_store_wait_all<0>();
    tc_fence_before();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem, 512);
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

struct BwdLayout {
    size_t off_fwd, off_cs, off_y, off_hf, off_flags, off_slots, total;
};

BwdLayout bwd_layout(const bm_ssd2_bwd_args* a, const bm_ssd2_fwd_args* f) {
    BwdLayout l{};
    const size_t nt = (size_t)cdiv(a->seqlen, T);
    l.off_fwd = 0;   // the forward kernel's status word doubles as this pass's
    l.off_cs = align_up(l.off_fwd + ssd2_workspace_bytes(f), 256);
    l.off_y = align_up(l.off_cs + (size_t)a->batch * nt * a->nheads * P * R * sizeof(float), 256);
    l.off_hf = align_up(l.off_y + (size_t)a->batch * a->seqlen * a->nheads * P * 2, 256);
    l.off_flags = align_up(l.off_hf + (size_t)a->batch * a->nheads * P * R * sizeof(float), 256);
    l.off_slots = l.off_flags + align_up((size_t)(sm_count() + 1) * sizeof(int), 256);
    l.total = l.off_slots + (size_t)(sm_count() + 1) * P * R * sizeof(float);
    return l;
}

bm_ssd2_fwd_args forward_args(const bm_ssd2_bwd_args* a) {
    bm_ssd2_fwd_args f{};
    f.batch = a->batch, f.seqlen = a->seqlen, f.nheads = a->nheads, f.headdim = a->headdim, f.state_rank = a->state_rank;
    f.ngroups = a->ngroups, f.chunk_len = T, f.dtype = a->dtype, f.path = BM_PATH_TENSOR_SINGLE;
    f.x = a->x, f.dt = a->dt, f.a = a->a, f.b = a->b, f.c = a->c, f.d = a->d, f.h0 = a->h0;
    return f;
}

}  // namespace

const char* ssd2_bwd_why_not(const bm_ssd2_bwd_args* a) {
    if (a->dtype != BM_DTYPE_BF16) return "activations must be bf16";
    if (a->headdim != P) return "headdim must be 64";
    if (a->state_rank != R) return "state_rank must be 128";
    return nullptr;
}

bool ssd2_bwd_supported(const bm_ssd2_bwd_args* a) { return ssd2_bwd_why_not(a) == nullptr; }

size_t ssd2_bwd_workspace_bytes(const bm_ssd2_bwd_args* a) {
    const bm_ssd2_fwd_args f = forward_args(a);
    return bwd_layout(a, &f).total;
}

int32_t ssd2_bwd_run(const bm_ssd2_bwd_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    bm_ssd2_fwd_args f = forward_args(a);
    const BwdLayout l = bwd_layout(a, &f);
    if (workspace == nullptr || workspace_bytes < l.total)
        return fail(BM_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", workspace_bytes, l.total);
    char* w = static_cast<char*>(workspace);
    // forward pass for the state entering every tile (and the final state)
    f.y = w + l.off_y;
    f.h_final = reinterpret_cast<float*>(w + l.off_hf);
    f.chunk_states = reinterpret_cast<float*>(w + l.off_cs);
    if (int32_t e = ssd2_run(&f, w + l.off_fwd, l.off_cs - l.off_fwd, stream)) return e;

    BwdParams prm{};
    const char* err = nullptr;
    const uint64_t S = a->seqlen, H = a->nheads, G = a->ngroups, B = a->batch;
    const uint32_t box[4] = {64, 1, (uint32_t)T, 1};
    {
        const uint64_t dims[4] = {(uint64_t)P, H, S, B};
        const uint64_t strides[3] = {(uint64_t)P * 2, H * P * 2, S * H * P * 2};
        if (!make_tensor_map_bf16(&prm.tm_x, a->x, 4, dims, strides, box, 128, &err) ||
            !make_tensor_map_bf16(&prm.tm_dy, a->dy, 4, dims, strides, box, 128, &err))
            return fail(BM_ERR_CUDA, "tensor map (x/dy): %s", err);
    }
    {
        const uint64_t dims[4] = {(uint64_t)R, G, S, B};
        const uint64_t strides[3] = {(uint64_t)R * 2, G * R * 2, S * G * R * 2};
        if (!make_tensor_map_bf16(&prm.tm_b, a->b, 4, dims, strides, box, 128, &err) ||
            !make_tensor_map_bf16(&prm.tm_c, a->c, 4, dims, strides, box, 128, &err))
            return fail(BM_ERR_CUDA, "tensor map (b/c): %s", err);
    }
    prm.dt = a->dt, prm.a = a->a, prm.d = a->d;
    prm.chunk_states = f.chunk_states, prm.dh_final = a->dh_final;
    prm.x = static_cast<const __nv_bfloat16*>(a->x), prm.dy = static_cast<const __nv_bfloat16*>(a->dy);
    prm.dx = a->dx, prm.ddt = a->ddt, prm.da = a->da, prm.db = a->db, prm.dc = a->dc, prm.dd = a->dd, prm.dh0 = a->dh0;
    prm.status = reinterpret_cast<int*>(w);
    prm.B = a->batch, prm.S = a->seqlen, prm.H = a->nheads, prm.G = a->ngroups;
    prm.NT = (int)cdiv(a->seqlen, T);
    prm.num_units = a->batch * a->nheads;
    cudaError_t e = cudaFuncSetAttribute(ssd2_bwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(ssd2_bwd_tc_kernel)");
    const size_t grp = (size_t)a->batch * a->seqlen * a->ngroups * R * sizeof(float);
    if (int32_t r = check_cuda(cudaMemsetAsync(a->db, 0, grp, stream), "cudaMemsetAsync(db)")) return r;
    if (int32_t r = check_cuda(cudaMemsetAsync(a->dc, 0, grp, stream), "cudaMemsetAsync(dc)")) return r;
    if (int32_t r = check_cuda(cudaMemsetAsync(a->da, 0, (size_t)a->nheads * sizeof(float), stream), "cudaMemsetAsync(da)")) return r;
    if (a->dd != nullptr)
        if (int32_t r = check_cuda(cudaMemsetAsync(a->dd, 0, (size_t)a->nheads * sizeof(float), stream), "cudaMemsetAsync(dd)")) return r;
    const int grid = prm.num_units < sm_count() ? prm.num_units : sm_count();
    if ((int64_t)prm.num_units * prm.NT > INT32_MAX) return fail(BM_ERR_UNSUPPORTED, "more than 2^31 tiles");
    prm.share_q = (int)((int64_t)prm.num_units * prm.NT / grid);
    prm.share_r = (int)((int64_t)prm.num_units * prm.NT % grid);
    prm.handoff_flags = reinterpret_cast<int*>(w + l.off_flags);
    prm.handoff = reinterpret_cast<float*>(w + l.off_slots);
    if (int32_t r = check_cuda(cudaMemsetAsync(prm.handoff_flags, 0, l.off_slots - l.off_flags, stream), "cudaMemsetAsync(flags)")) return r;
    ssd2_bwd_tc_kernel<<<grid, kThreads, kSmemBytes, stream>>>(prm);
    return check_launch("ssd2_bwd_tc_kernel");
}

}  // namespace tc
}  // namespace bm
