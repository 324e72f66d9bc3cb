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
// output staging aliases the operand area once the MMAs of phase 2 have completed: float32 tiles as TMA boxes of
// [128 rows x 32 floats] with 128-byte swizzle (one panel each): 4 for dC, 4 for dB, 2 for dx
// dx (written while the dC / dB MMAs still run) goes where only M lived, which G has finished reading by then; dC
// and dB (written after all MMAs) take the X, dY, e dY, B, C and dCB buffers
constexpr uint32_t kOffStC = 0, kOffStX = kOffM;
__host__ __device__ constexpr uint32_t stage_b_box(int k) { return k < 3 ? (4 + k) * kPanel : kOffDcb; }
static_assert(kOffM == 7 * kPanel && kOffDcb == 9 * kPanel, "staging map assumes this operand layout");
// the float32 state entering the tile is bulk-copied into the (not yet written) M area and read from there
constexpr uint32_t kOffHin = kOffM;
constexpr uint32_t kOffSc = kOperandBytes;    // per-tile scalars, float[128] each
enum { kScCum = 0, kScSc, kScSame, kScK, kScE, kScColk, kScColZ, kScPgs, kScPa, kScPgi = kScPa + 4, kScCount = kScPgi + 4 };
constexpr uint32_t kOffRed = kOffSc + kScCount * 128 * 4;   // 8 floats of block reductions
constexpr uint32_t kOffBar = kOffRed + 64;
constexpr uint32_t kSmemBytes = kOffBar + 64 + 1024;
static_assert(kSmemBytes <= 232448, "over the 227 KB shared-memory limit of a CTA");

// TMEM columns
constexpr uint32_t kColCB = 0, kColDM = 128, kColDC = 256, kColDB = 384;   // phase 1 / phase 2 accumulators
constexpr uint32_t kColG = 0, kColGi = 64, kColDhC = 128, kColY2 = 192;    // phase 2, over the consumed CB / dM

// Optional phase timeline (development builds only, -DBM_BWD_TRACE): thread 0 of CTA 0 records clock64() at the
// phase boundaries of its first tiles into prm.trace[tile][event].
#ifdef BM_BWD_TRACE
#define BWD_TRACE(ev)                                                                    \
    do {                                                                                 \
        if (blockIdx.x == 0 && tid == 0 && ntile < 64) prm.trace[ntile * 16 + (ev)] = clock64(); \
    } while (0)
#else
#define BWD_TRACE(ev) do { } while (0)
#endif

struct Bars {
    uint64_t ld_full, mma1, mma2, mma3;
    uint32_t tmem_base;
};

struct alignas(64) BwdParams {
    CUtensorMap tm_x, tm_dy, tm_b, tm_c;
    CUtensorMap tm_dx, tm_db, tm_dc;   // float32 gradient tiles, boxes of [128 rows x 32 floats]
    const float* sc;             // [b, s, h] column scale: dt (Mamba-2), scale (Mamba-3 single), NULL = 1
    const float* a;              // [h] (Mamba-2: the step's log decay is dt a)
    const float* da;             // [b, s, h] log decay per step (Mamba-3)
    const float* gamma;          // [b, s, h] same-step weight (Mamba-3 single), NULL = 1
    const float* d;
    const float* chunk_states;   // [b, n, h, p, r] state entering every tile (from the forward pass)
    const float* dh_final;
    float* dx;                   // [b, rows, h, p]
    float* ddt;                  // Mamba-2: [b, s, h]
    float* d_a;                  // Mamba-2: [h]
    float* dda;                  // Mamba-3: [b, s, h]
    float* dgamma;               // Mamba-3 single: [b, s, h]
    float* dscale;               // Mamba-3 single: [b, s, h]
    float* db;
    float* dc;
    float* dd;
    float* dh0;
    int* status;
    long long* trace;            // development builds only
    int* handoff_flags;          // [grid] warps of CTA c that have stored the dh its first piece ends with
    float* handoff;              // [grid][P][R]
    int B, S, St, H, G, NT, num_units, log2m;   // S counts fused (time x rank) rows, St time steps
    int share_q, share_r;        // (num_units * NT) / grid and the remainder
    int plain_bc;                // one head per group: dB / dC rows are stored, not reduce-added
};

// L2 prefetch of one tile of a 4-D tensor map.
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap* m, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(m), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}

// One float32 box [128 rows x 32 floats] from shared memory to its place in a gradient tensor: plain store, or
// reduce-add (rows past the end of the tensor are clipped by the copy engine).
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, const void* src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(m),
                 "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}
__device__ __forceinline__ void bulk_load_1d(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
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

// kMode 0: Mamba-2 (rows are tokens; column scale and same-step weight are both dt; skip term D).
// kMode 1: the Mamba-3 cores on the fused (time x rank) axis, 1 << log2m rows per step: strict-in-time decay
//          kernel with column scale `sc`, same-step block weighted by gamma (both 1 for the generic core).
template <int kMode>
__global__ void __launch_bounds__(kThreads, 1) ssd_bwd_tc_kernel(const __grid_constant__ BwdParams prm) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    Bars* bars = reinterpret_cast<Bars*>(smem + kOffBar);
    float* sc = reinterpret_cast<float*>(smem + kOffSc);
    float* red = reinterpret_cast<float*>(smem + kOffRed);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = tid & 127, pq = tid >> 7;   // the accumulator row and column quarter this thread owns
    const int log2m = kMode == 0 ? 0 : prm.log2m;

    if (tid == 0) {
        mbar_init(&bars->ld_full, 1);
        mbar_init(&bars->mma1, 1);
        mbar_init(&bars->mma2, 1);
        mbar_init(&bars->mma3, 1);
        fence_mbar_init();
        tma_prefetch_desc(&prm.tm_x);
        tma_prefetch_desc(&prm.tm_dy);
        tma_prefetch_desc(&prm.tm_b);
        tma_prefetch_desc(&prm.tm_c);
        tma_prefetch_desc(&prm.tm_dx);
        tma_prefetch_desc(&prm.tm_db);
        tma_prefetch_desc(&prm.tm_dc);
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
    int ntile = 0;        // tiles this CTA has started (trace index)

    // tiles [lo, hi) of the global (unit-major) tile sequence: share_q per CTA, one more for the first share_r
    const int cta = blockIdx.x, extra = cta < prm.share_r ? cta : prm.share_r;
    const int lo = cta * prm.share_q + extra, hi = lo + prm.share_q + (cta < prm.share_r ? 1 : 0);
    const int u_first = lo / prm.NT, u_last = (hi - 1) / prm.NT;

    for (int unit = u_first; unit <= u_last; ++unit) {
        const int b = unit / prm.H, h = unit - b * prm.H, g = h / hpg;
        const int i_lo = unit == u_first ? lo - u_first * prm.NT : 0;          // this CTA's tiles of the unit
        const int i_hi = unit == u_last ? hi - u_last * prm.NT : prm.NT;
        const int64_t state_base = ((int64_t)b * prm.H + h) * P * R;
        const float ah = kMode == 0 ? prm.a[h] : 1.f, dskip = (kMode == 0 && prm.d) ? prm.d[h] : 0.f;
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
        float da_acc = 0.f, dd_acc = 0.f;   // Mamba-2: dA (warp 0) and per-thread partials of dD

        for (int i = i_hi - 1; i >= i_lo; --i, phase ^= 1, ++ntile) {
            const int s0 = i * T, left = prm.S - s0;
            BWD_TRACE(0);
            // ---- loads of the tile
            if (tid == 0) {
                mbar_expect_tx(&bars->ld_full, 6 * kPanel + P * R * 4);
                bulk_load_1d(smem + kOffHin, prm.chunk_states + (((int64_t)b * prm.NT + i) * prm.H + h) * P * R, P * R * 4, &bars->ld_full);
                tma_load_4d(smem + kOffX, &prm.tm_x, &bars->ld_full, 0, h, s0, b);
                tma_load_4d(smem + kOffDy, &prm.tm_dy, &bars->ld_full, 0, h, s0, b);
                tma_load_4d(smem + kOffB, &prm.tm_b, &bars->ld_full, 0, g, s0, b);
                tma_load_4d(smem + kOffB + kPanel, &prm.tm_b, &bars->ld_full, 64, g, s0, b);
                tma_load_4d(smem + kOffC, &prm.tm_c, &bars->ld_full, 0, g, s0, b);
                tma_load_4d(smem + kOffC + kPanel, &prm.tm_c, &bars->ld_full, 64, g, s0, b);
                if (i > i_lo) {   // the tile this CTA walks next: into L2 while this one is worked on
                    tma_prefetch_4d(&prm.tm_x, 0, h, s0 - T, b);
                    tma_prefetch_4d(&prm.tm_dy, 0, h, s0 - T, b);
                    tma_prefetch_4d(&prm.tm_b, 0, g, s0 - T, b);
                    tma_prefetch_4d(&prm.tm_b, 64, g, s0 - T, b);
                    tma_prefetch_4d(&prm.tm_c, 0, g, s0 - T, b);
                    tma_prefetch_4d(&prm.tm_c, 64, g, s0 - T, b);
                }
            }
            // ---- per-row scalars (warp 1): log2-domain cumulative decay and the factors derived from it
            if (warp == 1) {
                float d4[4], g4[4], c4[4], run = 0.f;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int t = lane * 4 + k;
                    const bool live = t < left;
                    if (kMode == 0) {
                        d4[k] = live ? prm.sc[((int64_t)b * prm.S + s0 + t) * prm.H + h] : 0.f;
                        g4[k] = d4[k];
                        run = fmaf(d4[k], ah * log2e, run);
                    } else {
                        const int rrow = s0 + t;
                        const int64_t o = ((int64_t)b * prm.St + (rrow >> log2m)) * prm.H + h;
                        d4[k] = live ? (prm.sc ? prm.sc[o] : 1.f) : 0.f;
                        g4[k] = live ? (prm.gamma ? prm.gamma[o] : 1.f) : 0.f;
                        // the step's decay enters at its first rank, so every rank of a step sees it
                        if (live && (rrow & ((1 << log2m) - 1)) == 0) run = fmaf(prm.da[o], log2e, run);
                    }
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
                const float cblk = __shfl_sync(0xffffffffu, incl, (lane & ~7) | 7);   // end of the 32-row block
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int t = lane * 4 + k;
                    const float c = excl + c4[k];
                    sc[kScCum * 128 + t] = c;
                    sc[kScSc * 128 + t] = d4[k];
                    sc[kScSame * 128 + t] = g4[k];
                    sc[kScK * 128 + t] = ex2(cend - c);
                    sc[kScE * 128 + t] = ex2(c);
                    sc[kScColk * 128 + t] = ex2(cblk - c);
                    sc[kScColZ * 128 + t] = 0.f;
                    sc[kScPgs * 128 + t] = 0.f;
                }
            }
            // ---- dh -> bf16 operand [r][p]
            {
                const uint4 w0 = make_uint4(pack_bf16x2(dh[0], dh[1]), pack_bf16x2(dh[2], dh[3]), pack_bf16x2(dh[4], dh[5]), pack_bf16x2(dh[6], dh[7]));
                const uint4 w1 = make_uint4(pack_bf16x2(dh[8], dh[9]), pack_bf16x2(dh[10], dh[11]), pack_bf16x2(dh[12], dh[13]), pack_bf16x2(dh[14], dh[15]));
                *reinterpret_cast<uint4*>(smem + kOffDh + sw128_offset(row, 2 * pq)) = w0;
                *reinterpret_cast<uint4*>(smem + kOffDh + sw128_offset(row, 2 * pq + 1)) = w1;
            }
            BWD_TRACE(1);
            if (cta_wait_failed(&bars->ld_full, phase)) goto timed_out;   // also publishes the scalars
            BWD_TRACE(2);
            // ---- the state entering the tile (float32 [p][r], just landed) -> bf16 operand [r][p]; <dh, h_in> over this
            // thread's 16 elements
            float dot = 0.f;
            {
                const float* hs32 = reinterpret_cast<const float*>(smem + kOffHin);
                float hin[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) hin[j] = hs32[(16 * pq + j) * R + row];
#pragma unroll
                for (int j = 0; j < 16; ++j) dot = fmaf(dh[j], hin[j], dot);
                const uint4 v0 = make_uint4(pack_bf16x2(hin[0], hin[1]), pack_bf16x2(hin[2], hin[3]), pack_bf16x2(hin[4], hin[5]), pack_bf16x2(hin[6], hin[7]));
                const uint4 v1 = make_uint4(pack_bf16x2(hin[8], hin[9]), pack_bf16x2(hin[10], hin[11]), pack_bf16x2(hin[12], hin[13]), pack_bf16x2(hin[14], hin[15]));
                *reinterpret_cast<uint4*>(smem + kOffH + sw128_offset(row, 2 * pq)) = v0;
                *reinterpret_cast<uint4*>(smem + kOffH + sw128_offset(row, 2 * pq + 1)) = v1;
            }
            // ---- e dY (this thread: 16 elements of row `row`); x and dy of those elements stay in registers
            uint4 xr[2], dyr[2];
            {
                const float et = sc[kScE * 128 + row];
#pragma unroll
                for (int c2 = 0; c2 < 2; ++c2) {
                    const uint32_t off = sw128_offset(row, 2 * pq + c2);
                    xr[c2] = *reinterpret_cast<const uint4*>(smem + kOffX + off);
                    dyr[c2] = *reinterpret_cast<const uint4*>(smem + kOffDy + off);
                    const uint32_t* ys = &dyr[c2].x;
                    uint32_t yo[4];
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const float2 yf = unpack_bf16x2(ys[m]);
                        yo[m] = pack_bf16x2(yf.x * et, yf.y * et);
                    }
                    *reinterpret_cast<uint4*>(smem + kOffDye + off) = make_uint4(yo[0], yo[1], yo[2], yo[3]);
                }
            }
            fence_proxy_async_smem();
            __syncthreads();
            // ---- phase 1: CB = C B^T, dM = dY X^T
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
            BWD_TRACE(3);
            if (cta_wait_failed(&bars->mma1, phase)) goto timed_out;
            BWD_TRACE(4);
            tc_fence_after();
            // ---- mask pass: columns [32 pq, 32 pq + 32) of row `row`.  Entry (t, s): an earlier step takes
            // w = exp(c_t - c_s) sc_s, the same step takes the row's same-step weight, later steps 0.
            //   M = CB w, dCB = dM w (bf16, to shared memory);  Z = CB dM exp(c_t - c_s) over earlier steps:
            //   its row sums weighted by sc_s and its column sums feed the decay and scale gradients; the
            //   same-step sum of CB dM is the gradient of the same-step weight.
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
                            const int s_ = 32 * pq + 2 * j;
                            const float f0 = rf * sc[kScColk * 128 + s_], f1 = rf * sc[kScColk * 128 + s_ + 1];
                            const float w0 = f0 * sc[kScSc * 128 + s_], w1 = f1 * sc[kScSc * 128 + s_ + 1];
                            const float c0 = __uint_as_float(cb[2 * j]), c1 = __uint_as_float(cb[2 * j + 1]);
                            const float d0 = __uint_as_float(dm[2 * j]), d1 = __uint_as_float(dm[2 * j + 1]);
                            om[j] = pack_bf16x2(c0 * w0, c1 * w1);
                            od[j] = pack_bf16x2(d0 * w0, d1 * w1);
                            const float z0 = c0 * d0 * f0, z1 = c1 * d1 * f1;
                            wrow = fmaf(z0, sc[kScSc * 128 + s_], wrow);
                            wrow = fmaf(z1, sc[kScSc * 128 + s_ + 1], wrow);
                            cb[2 * j] = __float_as_uint(z0);
                            cb[2 * j + 1] = __float_as_uint(z1);
                        }
                    } else {
                        const float same = sc[kScSame * 128 + row];
                        const int tstep = row >> log2m;
                        float gs = 0.f;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            float mv[2], dcv[2], zv[2];
#pragma unroll
                            for (int e = 0; e < 2; ++e) {
                                const int s_ = 32 * pq + 2 * j + e, sstep = s_ >> log2m;
                                const float cv = __uint_as_float(cb[2 * j + e]), dv = __uint_as_float(dm[2 * j + e]);
                                float w = 0.f, z = 0.f;
                                if (sstep < tstep) {
                                    const float f = ex2(ct - sc[kScCum * 128 + s_]);
                                    w = f * sc[kScSc * 128 + s_];
                                    z = cv * dv * f;
                                    wrow = fmaf(z, sc[kScSc * 128 + s_], wrow);
                                } else if (sstep == tstep) {
                                    w = same;
                                    gs = fmaf(cv, dv, gs);
                                }
                                mv[e] = cv * w, dcv[e] = dv * w, zv[e] = z;
                            }
                            om[j] = pack_bf16x2(mv[0], mv[1]);
                            od[j] = pack_bf16x2(dcv[0], dcv[1]);
                            cb[2 * j] = __float_as_uint(zv[0]);
                            cb[2 * j + 1] = __float_as_uint(zv[1]);
                        }
                        sc[kScPgs * 128 + row] = gs;
                    }
                    // column sums of Z over the warp's 32 rows through a transposing butterfly
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
                    atomicAdd(&sc[kScColZ * 128 + 32 * pq + lane], __uint_as_float(cb[0]));
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
                // the scaled input of the state terms: k_s sc_s x_s (dM has been formed from x_s already)
                const float ks = sc[kScK * 128 + row] * sc[kScSc * 128 + row];
#pragma unroll
                for (int c2 = 0; c2 < 2; ++c2) {
                    const uint32_t* xs = &xr[c2].x;
                    uint32_t w[4];
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const float2 f = unpack_bf16x2(xs[m]);
                        w[m] = pack_bf16x2(f.x * ks, f.y * ks);
                    }
                    *reinterpret_cast<uint4*>(smem + kOffX + sw128_offset(row, 2 * pq + c2)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            tc_fence_before();
            fence_proxy_async_smem();
            __syncthreads();
            BWD_TRACE(5);
            // ---- phase 2
            if (tid == 0) {
                tc_fence_after();
                const uint32_t b_sm = smem_u32(smem + kOffB), c_sm = smem_u32(smem + kOffC), m_sm = smem_u32(smem + kOffM);
                const uint32_t dcb_sm = smem_u32(smem + kOffDcb), x_sm = smem_u32(smem + kOffX), dy_sm = smem_u32(smem + kOffDy);
                const uint32_t dye_sm = smem_u32(smem + kOffDye), h_sm = smem_u32(smem + kOffH), dh_sm = smem_u32(smem + kOffDh);
                const uint32_t id_kk = umma_idesc_bf16(128, 128, false, false), id_kmn = umma_idesc_bf16(128, 128, false, true);
                const uint32_t id_mm = umma_idesc_bf16(128, 128, true, true);
                const uint32_t id64_mm = umma_idesc_bf16(128, 64, true, true), id64_kmn = umma_idesc_bf16(128, 64, false, true);
                // G = M^T dY, Gi = B dh, dhC = C^T (e dY), Y2 = C h_in^T
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
                umma_commit(&bars->mma2);   // the four 64-wide products: their epilogue runs while dC / dB are computed
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
                // dB = dCB^T C + (k sc X) dh^T
                {
                    const uint64_t da_ = umma_desc_mnmajor(dcb_sm, kPanel), dc_ = umma_desc_mnmajor(c_sm, kPanel);
#pragma unroll 1
                    for (int k = 0; k < 8; ++k) umma_ss(tmem + kColDB, desc_advance(da_, k * 2048), desc_advance(dc_, k * 2048), id_mm, k > 0);
                    const uint64_t dx_ = umma_desc_kmajor(x_sm), dh_ = umma_desc_kmajor(dh_sm);
#pragma unroll 1
                    for (int k = 0; k < 4; ++k) umma_ss(tmem + kColDB, desc_advance(dx_, k * 32), desc_advance(dh_, k * 32), id_kk, true);
                }
                umma_commit(&bars->mma3);
            }
            BWD_TRACE(6);
            if (cta_wait_failed(&bars->mma2, phase)) goto timed_out;
            BWD_TRACE(7);
            tc_fence_after();
            // ---- epilogue of the 64-wide products (dC / dB are still being computed: only the M buffer is free yet)
            {
                // dx: 16 columns of row `row`; dy . Y2 and x . Gi for the decay / scale gradients
                uint32_t gg[16], gi[16], dc16[16], y2[16];
                tmem_ld16(lane_addr + kColG + 16 * pq, gg);
                tmem_ld16(lane_addr + kColGi + 16 * pq, gi);
                tmem_ld16(lane_addr + kColDhC + 16 * pq, dc16);
                tmem_ld16(lane_addr + kColY2 + 16 * pq, y2);
                tmem_wait_ld();
                const float ks = sc[kScK * 128 + row] * sc[kScSc * 128 + row];
                float pin = 0.f, pgi = 0.f, dxo[16];
#pragma unroll
                for (int c2 = 0; c2 < 2; ++c2) {
                    const uint32_t* xs = &xr[c2].x;
                    const uint32_t* ys = &dyr[c2].x;
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        const float2 xf = unpack_bf16x2(xs[m]), yf = unpack_bf16x2(ys[m]);
                        const int j = 8 * c2 + 2 * m;
                        pin = fmaf(yf.x, __uint_as_float(y2[j]), pin);
                        pin = fmaf(yf.y, __uint_as_float(y2[j + 1]), pin);
                        pgi = fmaf(xf.x, __uint_as_float(gi[j]), pgi);
                        pgi = fmaf(xf.y, __uint_as_float(gi[j + 1]), pgi);
                        dxo[j] = fmaf(ks, __uint_as_float(gi[j]), __uint_as_float(gg[j]));
                        dxo[j + 1] = fmaf(ks, __uint_as_float(gi[j + 1]), __uint_as_float(gg[j + 1]));
                        if (kMode == 0) {
                            dxo[j] = fmaf(dskip, yf.x, dxo[j]);
                            dxo[j + 1] = fmaf(dskip, yf.y, dxo[j + 1]);
                            dd_acc = fmaf(xf.x, yf.x, dd_acc);
                            dd_acc = fmaf(xf.y, yf.y, dd_acc);
                        }
                    }
                }
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4)
                    *reinterpret_cast<float4*>(smem + kOffStX + (pq >> 1) * kPanel + sw128_offset(row, (pq & 1) * 4 + c4)) =
                        make_float4(dxo[4 * c4], dxo[4 * c4 + 1], dxo[4 * c4 + 2], dxo[4 * c4 + 3]);
                // the readout term joins the weighted row sum of Z this thread stored in the mask pass
                sc[(kScPa + pq) * 128 + row] += sc[kScE * 128 + row] * pin;
                sc[(kScPgi + pq) * 128 + row] = pgi;
                // the state gradient entering the tile
                const float decay = ex2(sc[kScCum * 128 + 127]);
#pragma unroll
                for (int j = 0; j < 16; ++j) dh[j] = fmaf(decay, dh[j], __uint_as_float(dc16[j]));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                // ---- dC and dB, once their MMAs have completed
                if (cta_wait_failed(&bars->mma3, phase)) goto timed_out;
                tc_fence_after();
                uint32_t acc[32];
                tmem_ld32(lane_addr + kColDC + 32 * pq, acc);
                tmem_wait_ld();
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4)
                    *reinterpret_cast<uint4*>(smem + kOffStC + pq * kPanel + sw128_offset(row, c4)) =
                        make_uint4(acc[4 * c4], acc[4 * c4 + 1], acc[4 * c4 + 2], acc[4 * c4 + 3]);
                tmem_ld32(lane_addr + kColDB + 32 * pq, acc);
                tmem_wait_ld();
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4)
                    *reinterpret_cast<uint4*>(smem + stage_b_box(pq) + sw128_offset(row, c4)) =
                        make_uint4(acc[4 * c4], acc[4 * c4 + 1], acc[4 * c4 + 2], acc[4 * c4 + 3]);
                if (tid == 0) red[0] = 0.f;
                tc_fence_before();
                fence_proxy_async_smem();
                __syncthreads();
                BWD_TRACE(8);
                if (lane == 0) atomicAdd(&red[0], dot * decay);
                // gradient tiles leave as TMA boxes: dx stored, dB / dC reduce-added into the group's rows (stored when
                // every head has its own); ten copies per tile, issued by one thread
                if (tid == 32) {
#pragma unroll
                    for (int k = 0; k < 2; ++k) tma_store_4d(&prm.tm_dx, smem + kOffStX + k * kPanel, 32 * k, h, s0, b);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (prm.plain_bc) {
                            tma_store_4d(&prm.tm_dc, smem + kOffStC + k * kPanel, 32 * k, g, s0, b);
                            tma_store_4d(&prm.tm_db, smem + stage_b_box(k), 32 * k, g, s0, b);
                        } else {
                            tma_reduce_add_4d(&prm.tm_dc, smem + kOffStC + k * kPanel, 32 * k, g, s0, b);
                            tma_reduce_add_4d(&prm.tm_db, smem + stage_b_box(k), 32 * k, g, s0, b);
                        }
                    }
                    tma_store_commit();
                }
                __syncthreads();
                BWD_TRACE(9);
                // ---- scalar gradients (warp 0, four consecutive rows per lane):
                //   d(log decay)_row = sum_{t >= row} [rowsum_t - sc_t colZ_t] + sum_{s < row} k_s sc_s (x_s . Gi_s)
                //                      + exp(c_end) <dh, h_in>
                //   d(column scale)_row = colZ_row + k_row (x_row . Gi_row);  d(same-step weight)_row = Pgs_row
                if (warp == 0) {
                    float v[4], u[4], ds[4], run = 0.f, prun = 0.f;
#pragma unroll
                    for (int k = 3; k >= 0; --k) {
                        const int t = lane * 4 + k;
                        float dcv = -sc[kScSc * 128 + t] * sc[kScColZ * 128 + t];
#pragma unroll
                        for (int w = 0; w < 4; ++w) dcv += sc[(kScPa + w) * 128 + t];
                        run += dcv;
                        v[k] = run;
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {   // exclusive prefix of the state-input terms
                        const int t = lane * 4 + k;
                        float pg = 0.f;
#pragma unroll
                        for (int w = 0; w < 4; ++w) pg += sc[(kScPgi + w) * 128 + t];
                        pg *= sc[kScK * 128 + t];
                        ds[k] = sc[kScColZ * 128 + t] + pg;
                        u[k] = prun;
                        prun = fmaf(sc[kScSc * 128 + t], pg, prun);
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
                    if (kMode == 0) {
                        float dal = 0.f;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int t = lane * 4 + k;
                            const float dda = v[k] + u[k] + after;
                            if (t < left)
                                prm.ddt[((int64_t)b * prm.S + s0 + t) * prm.H + h] = fmaf(ah, dda, ds[k] + sc[kScPgs * 128 + t]);
                            dal = fmaf(sc[kScSc * 128 + t], dda, dal);
                        }
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) dal += __shfl_xor_sync(0xffffffffu, dal, o);
                        da_acc += dal;
                    } else {
                        // rows of a step are consecutive and never straddle lanes (1, 2 or 4 rows per step)
                        const int m = 1 << log2m;
#pragma unroll
                        for (int k0 = 0; k0 < 4; ++k0) {
                            if ((k0 & (m - 1)) != 0) continue;
                            const int t = lane * 4 + k0;
                            if (t >= left) continue;
                            float dsc = 0.f, dg = 0.f;
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                if (k >= k0 && k < k0 + m) {
                                    dsc += ds[k];
                                    dg += sc[kScPgs * 128 + lane * 4 + k];
                                }
                            const int64_t o = ((int64_t)b * prm.St + ((s0 + t) >> log2m)) * prm.H + h;
                            prm.dda[o] = v[k0] + u[k0] + after;
                            if (prm.dscale) prm.dscale[o] = dsc;
                            if (prm.dgamma) prm.dgamma[o] = dg;
                        }
                    }
                }
                // the staging tiles must have been read before the next tile's loads overwrite them
                BWD_TRACE(10);
                if (tid == 32) tma_store_wait_read<0>();
                __syncthreads();
                BWD_TRACE(11);
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
        if (kMode == 0) {
            if (tid == 0) atomicAdd(prm.d_a + h, da_acc);
            if (prm.dd != nullptr) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) dd_acc += __shfl_xor_sync(0xffffffffu, dd_acc, o);
                if (lane == 0) atomicAdd(prm.dd + h, dd_acc);
            }
        }
    }
    goto done;
timed_out:
    if (tid == 0) {
        atomicExch(prm.status, (int)BM_ERR_TIMEOUT);
        // what this thread may still have in flight (loads, MMAs of the current tile) before shared memory and
        // TMEM go back; bounded again
        uint64_t* bs[4] = {&bars->ld_full, &bars->mma1, &bars->mma2, &bars->mma3};
        for (int k = 0; k < 4; ++k)
            for (uint32_t n = 0; n < kWaitBudget && !mbar_try_wait(bs[k], phase); ++n) {}
    }
done:
    if (tid == 32) tma_store_wait_all<0>();
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

// rows = sequence length of the kernel's row axis (tokens, or fused time x rank rows)
BwdLayout bwd_layout(int batch, int64_t rows, int nheads, size_t fwd_bytes) {
    BwdLayout l{};
    const size_t nt = (size_t)cdiv(rows, T);
    l.off_fwd = 0;   // the forward kernel's status word doubles as this pass's
    l.off_cs = align_up(l.off_fwd + fwd_bytes, 256);
    l.off_y = align_up(l.off_cs + (size_t)batch * nt * nheads * P * R * sizeof(float), 256);
    l.off_hf = align_up(l.off_y + (size_t)batch * rows * nheads * P * 2, 256);
    l.off_flags = align_up(l.off_hf + (size_t)batch * nheads * P * R * sizeof(float), 256);
    l.off_slots = l.off_flags + align_up((size_t)(sm_count() + 1) * sizeof(int), 256);
    l.total = l.off_slots + (size_t)(sm_count() + 1) * P * R * sizeof(float) + 64 * 16 * sizeof(long long);
    return l;
}

bm_ssd2_fwd_args forward_args(const bm_ssd2_bwd_args* a) {
    bm_ssd2_fwd_args f{};
    f.batch = a->batch, f.seqlen = a->seqlen, f.nheads = a->nheads, f.headdim = a->headdim, f.state_rank = a->state_rank;
    f.ngroups = a->ngroups, f.chunk_len = T, f.dtype = a->dtype, f.path = BM_PATH_TENSOR_SINGLE;
    f.x = a->x, f.dt = a->dt, f.a = a->a, f.b = a->b, f.c = a->c, f.d = a->d, f.h0 = a->h0;
    return f;
}

bm_ssd3_fwd_args forward_args3(const bm_ssd3_bwd_args* a) {
    bm_ssd3_fwd_args f{};
    f.batch = a->batch, f.seqlen = a->seqlen, f.nheads = a->nheads, f.headdim = a->headdim, f.state_rank = a->state_rank;
    f.mimo_rank = a->mimo_rank, f.chunk_len = a->chunk_len, f.dtype = a->dtype, f.path = BM_PATH_TENSOR;
    f.v = a->v, f.da = a->da, f.b = a->b, f.c = a->c, f.gamma = a->gamma, f.scale = a->scale, f.h0 = a->h0;
    return f;
}

int log2_of(int v) {
    int l = 0;
    while ((1 << l) < v) ++l;
    return (1 << l) == v ? l : -1;
}

// Tensor maps, shares and the launch, common to both families.  `rows` = length of the row axis.
template <int kMode>
int32_t launch(BwdParams& prm, const void* x, const void* dy, const void* bmat, const void* cmat, int batch, int64_t rows,
               int nheads, int ngroups, char* w, const BwdLayout& l, cudaStream_t stream) {
    const char* err = nullptr;
    const uint64_t S = rows, H = nheads, G = ngroups, B = batch;
    const uint32_t box[4] = {64, 1, (uint32_t)T, 1};
    {
        const uint64_t dims[4] = {(uint64_t)P, H, S, B};
        const uint64_t strides[3] = {(uint64_t)P * 2, H * P * 2, S * H * P * 2};
        if (!make_tensor_map_bf16(&prm.tm_x, x, 4, dims, strides, box, 128, &err) ||
            !make_tensor_map_bf16(&prm.tm_dy, dy, 4, dims, strides, box, 128, &err))
            return fail(BM_ERR_CUDA, "tensor map (x/dy): %s", err);
    }
    {
        const uint64_t dims[4] = {(uint64_t)R, G, S, B};
        const uint64_t strides[3] = {(uint64_t)R * 2, G * R * 2, S * G * R * 2};
        if (!make_tensor_map_bf16(&prm.tm_b, bmat, 4, dims, strides, box, 128, &err) ||
            !make_tensor_map_bf16(&prm.tm_c, cmat, 4, dims, strides, box, 128, &err))
            return fail(BM_ERR_CUDA, "tensor map (b/c): %s", err);
    }
    {
        const uint32_t box32[4] = {32, 1, (uint32_t)T, 1};
        const uint64_t dx_dims[4] = {(uint64_t)P, H, S, B}, dx_str[3] = {(uint64_t)P * 4, H * P * 4, S * H * P * 4};
        const uint64_t bc_dims[4] = {(uint64_t)R, G, S, B}, bc_str[3] = {(uint64_t)R * 4, G * R * 4, S * G * R * 4};
        if (!make_tensor_map_f32(&prm.tm_dx, prm.dx, 4, dx_dims, dx_str, box32, 128, &err) ||
            !make_tensor_map_f32(&prm.tm_db, prm.db, 4, bc_dims, bc_str, box32, 128, &err) ||
            !make_tensor_map_f32(&prm.tm_dc, prm.dc, 4, bc_dims, bc_str, box32, 128, &err))
            return fail(BM_ERR_CUDA, "tensor map (gradients): %s", err);
    }
    prm.status = reinterpret_cast<int*>(w);
    prm.B = batch, prm.S = (int)rows, prm.H = nheads, prm.G = ngroups;
    prm.NT = (int)cdiv(rows, T);
    prm.num_units = batch * nheads;
    prm.plain_bc = ngroups == nheads ? 1 : 0;
    cudaError_t e = cudaFuncSetAttribute(ssd_bwd_tc_kernel<kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(ssd_bwd_tc_kernel)");
    if (!prm.plain_bc) {
        const size_t grp = (size_t)batch * rows * ngroups * R * sizeof(float);
        if (int32_t r = check_cuda(cudaMemsetAsync(prm.db, 0, grp, stream), "cudaMemsetAsync(db)")) return r;
        if (int32_t r = check_cuda(cudaMemsetAsync(prm.dc, 0, grp, stream), "cudaMemsetAsync(dc)")) return r;
    }
    const int grid = prm.num_units < sm_count() ? prm.num_units : sm_count();
    if ((int64_t)prm.num_units * prm.NT > INT32_MAX) return fail(BM_ERR_UNSUPPORTED, "more than 2^31 tiles");
    prm.share_q = (int)((int64_t)prm.num_units * prm.NT / grid);
    prm.share_r = (int)((int64_t)prm.num_units * prm.NT % grid);
    prm.handoff_flags = reinterpret_cast<int*>(w + l.off_flags);
    prm.handoff = reinterpret_cast<float*>(w + l.off_slots);
    prm.trace = reinterpret_cast<long long*>(w + l.total - 64 * 16 * sizeof(long long));
    if (int32_t r = check_cuda(cudaMemsetAsync(prm.handoff_flags, 0, l.off_slots - l.off_flags, stream), "cudaMemsetAsync(flags)")) return r;
    ssd_bwd_tc_kernel<kMode><<<grid, kThreads, kSmemBytes, stream>>>(prm);
    return check_launch("ssd_bwd_tc_kernel");
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
    return bwd_layout(a->batch, a->seqlen, a->nheads, ssd2_workspace_bytes(&f)).total;
}

int32_t ssd2_bwd_run(const bm_ssd2_bwd_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    bm_ssd2_fwd_args f = forward_args(a);
    const BwdLayout l = bwd_layout(a->batch, a->seqlen, a->nheads, ssd2_workspace_bytes(&f));
    if (workspace == nullptr || workspace_bytes < l.total)
        return fail(BM_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", workspace_bytes, l.total);
    char* w = static_cast<char*>(workspace);
    // forward pass for the state entering every tile
    f.y = w + l.off_y;
    f.h_final = reinterpret_cast<float*>(w + l.off_hf);
    f.chunk_states = reinterpret_cast<float*>(w + l.off_cs);
    if (int32_t e = ssd2_run(&f, w + l.off_fwd, l.off_cs - l.off_fwd, stream)) return e;

    BwdParams prm{};
    prm.sc = a->dt, prm.a = a->a, prm.d = a->d;
    prm.chunk_states = f.chunk_states, prm.dh_final = a->dh_final;
    prm.dx = a->dx, prm.ddt = a->ddt, prm.d_a = a->da, prm.db = a->db, prm.dc = a->dc, prm.dd = a->dd, prm.dh0 = a->dh0;
    prm.St = a->seqlen, prm.log2m = 0;
    if (int32_t r = check_cuda(cudaMemsetAsync(a->da, 0, (size_t)a->nheads * sizeof(float), stream), "cudaMemsetAsync(da)")) return r;
    if (a->dd != nullptr)
        if (int32_t r = check_cuda(cudaMemsetAsync(a->dd, 0, (size_t)a->nheads * sizeof(float), stream), "cudaMemsetAsync(dd)")) return r;
    return launch<0>(prm, a->x, a->dy, a->b, a->c, a->batch, a->seqlen, a->nheads, a->ngroups, w, l, stream);
}

const char* ssd3_bwd_why_not(const bm_ssd3_bwd_args* a) {
    if (a->dtype != BM_DTYPE_BF16) return "activations must be bf16";
    if (a->headdim != P) return "headdim must be 64";
    if (a->state_rank != R) return "state_rank must be 128";
    if (log2_of(a->mimo_rank) < 0 || a->mimo_rank > 4) return "mimo_rank must be 1, 2 or 4";
    return nullptr;
}

bool ssd3_bwd_supported(const bm_ssd3_bwd_args* a) { return ssd3_bwd_why_not(a) == nullptr; }

size_t ssd3_bwd_workspace_bytes(const bm_ssd3_bwd_args* a) {
    const bm_ssd3_fwd_args f = forward_args3(a);
    return bwd_layout(a->batch, (int64_t)a->seqlen * a->mimo_rank, a->nheads, ssd3_workspace_bytes(&f)).total;
}

int32_t ssd3_bwd_run(const bm_ssd3_bwd_args* a, bool single, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    bm_ssd3_fwd_args f = forward_args3(a);
    const int64_t rows = (int64_t)a->seqlen * a->mimo_rank;
    const BwdLayout l = bwd_layout(a->batch, rows, a->nheads, ssd3_workspace_bytes(&f));
    if (workspace == nullptr || workspace_bytes < l.total)
        return fail(BM_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", workspace_bytes, l.total);
    char* w = static_cast<char*>(workspace);
    f.y = w + l.off_y;
    f.h_final = reinterpret_cast<float*>(w + l.off_hf);
    float* cs = reinterpret_cast<float*>(w + l.off_cs);
    if (int32_t e = ssd3_run(&f, single, w + l.off_fwd, l.off_cs - l.off_fwd, stream, cs)) return e;

    BwdParams prm{};
    prm.sc = single ? a->scale : nullptr, prm.gamma = single ? a->gamma : nullptr, prm.da = a->da;
    prm.chunk_states = cs, prm.dh_final = a->dh_final;
    prm.dx = a->dv, prm.dda = a->dda, prm.dgamma = single ? a->dgamma : nullptr, prm.dscale = single ? a->dscale : nullptr;
    prm.db = a->db, prm.dc = a->dc, prm.dh0 = a->dh0;
    prm.St = a->seqlen, prm.log2m = log2_of(a->mimo_rank);
    return launch<1>(prm, a->v, a->dy, a->b, a->c, a->batch, rows, a->nheads, a->nheads, w, l, stream);
}

}  // namespace tc
}  // namespace bm
