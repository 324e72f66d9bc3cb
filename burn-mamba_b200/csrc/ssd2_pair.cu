// Mamba-2 chunked SSD forward on the Blackwell tensor cores, two heads of one B/C group per CTA.
//
// All heads of a group share B and C (src/modules/misc/gqa.rs:30-56), so a CTA that walks two heads of a
// group in lock-step loads the C and B tiles once, forms CB = C B^T once, and runs the readout and state
// contractions 128 columns wide (both heads side by side) instead of twice 64.  That halves the shared-memory
// traffic of the TMA loads and of the tensor-core operand reads, which is what paces a one-head-per-CTA
// kernel.  Formulas: src/mamba2/ssd/serial.rs:138-506 with a 128-token tile as the chunk (the chunk
// length is a no-op for y and the final state).  Per tile, with cum the log2-domain cumulative decay
// inside the tile, cend its last value and a reference point cref = cend / 2:
//     CB   = C B^T                                       tcgen05 SS, once for both heads          (K2)
//     P_h  = bf16(causal(CB)) + diag(D_h / dt)           TMEM -> TMEM, per head (only the diagonal differs)
//     Xw_h = X_h * w_h,  w_t = dt_t 2^(cref - cum_t)     registers -> shared memory
//     Y    = C [H'_A | H'_B]^T  (+)=  P_h Xw_h           tcgen05 SS (N = 128) then TS (N = 64 each), one accumulator
//     y_t  = 2^(cum_t - cref) Y_t                        epilogue, straight to global memory
//     S    = B^T [Xw_A | Xw_B]                           tcgen05 SS (N = 128)                     (K3)
//     h   <- 2^cend h + 2^(cend - cref) S ;  H' = bf16(2^cref_next h)                             (K4)
// All exponents stay within 2^+-90: a tile whose decay is stronger than 2^-180 is walked as 2, 4, ... 128
// sub-ranges (the decay-scan warp decides per tile), each sub-range one pass of the same pipeline with the
// rows outside it weighted zero.
//
// Work items are (batch row, head pair, sequence segment).  Segments of one pair are chained through a
// float32 state in the workspace; items are handed out segment-major, so that the segment an item waits for
// was started a whole round of the machine earlier.  This turns the wave quantisation of (batch x head)
// units into a tail of one short segment.
//
// Warp roles (640 threads): warp 0 TMA loads of C and B; warp 1 issues CB; warp 2 owns TMEM and issues the
// readout and state MMAs; warp 3 scans dt and publishes one descriptor per pass into a ring that every other
// role follows; warps 4-7 mask pass; warps 8-11 / 12-15 X scaling, state update
// and state publishing of head A / head B (state in registers, X rows prefetched from global memory into
// registers one pass ahead); warps 16-19 epilogue.  Every wait is bounded.
#include "ssd2_tc.cuh"
#include "tc_common.cuh"

namespace bm {
namespace tc {

namespace {

constexpr int T = 128;        // tokens per tile
constexpr int P = 64;         // head dim
constexpr int R = 128;        // state rank
constexpr int kThreads = 640;
constexpr int kRing = 4;      // descriptor ring depth (power of two)
constexpr float kMaxRangeLog2Decay = 180.f;       // a pass covers at most this much decay: every factor within 2^+-90
// The skip term D x_t rides through the tensor cores as (D / dt_t) on the diagonal of P times the scaled row
// dt_t 2^(cref - cum_t) x_t, which needs a step that is not vanishingly small: live rows are processed with
// max(dt_t, 2^-20).  The difference is at most 1e-6 |B x_t| in the state and in y, far inside bf16 rounding.
constexpr float kMinStep = 9.5367432e-7f;

// shared-memory map (bytes from a 1024-aligned base)
constexpr uint32_t kPanel = 16384;               // [128 rows x 128 B]
constexpr uint32_t kOffC = 0;                    // 2 stages x 2 panels
constexpr uint32_t kOffB = 65536;                // 2 stages x 2 panels
constexpr uint32_t kOffXw = 131072;              // head A, head B: 1 panel each
constexpr uint32_t kOffH = 163840;               // head A, head B: 1 panel each
constexpr uint32_t kOffRing = 196608;
constexpr uint32_t kRingEntryBytes = 4 * T * 4 + 64;   // cum A, w A, cum B, w B, descriptor
// y staging: per epilogue warp two tiles of [32 rows x 64 B] (64-byte swizzle), filled and TMA-stored in turn
constexpr uint32_t kOffStage = (kOffRing + kRing * kRingEntryBytes + 1023u) & ~1023u;
constexpr uint32_t kStageTileBytes = 2048;
constexpr uint32_t kOffScan = kOffStage + 4 * 2 * kStageTileBytes;   // scan scratch: per head cum[128], dt[128]
constexpr uint32_t kOffBar = kOffScan + 2 * 2 * T * 4;
constexpr uint32_t kSmemBytes = kOffBar + 512 + 1024;  // barriers + alignment slack
static_assert(kSmemBytes <= 232448, "over the 227 KB shared-memory limit of a CTA");
constexpr uint32_t kLoadBytesCB = 4 * kPanel;

// TMEM columns
// A pass uses accumulator `it & 1`: first C B^T lands there, the mask pass turns it into P, then the same
// columns take the y accumulator of the pass; the epilogue hands them back two passes later.
constexpr uint32_t kColYC = 0;     // 2 x 128: C B^T (float32), then y accumulator (head A | head B)
constexpr uint32_t kColP = 256;    // 2 x 64: P of head A, head B (packed bf16 pairs)
constexpr uint32_t kColS = 384;    // 128: state contribution, head A | head B

enum : int { kFirst = 1, kLast = 2, kStop = 4, kTileStart = 8 };

struct Desc {          // one pass of the pipeline; 64 bytes at the end of a ring entry
    int b, ha, g, s0;  // batch row, first head of the pair, B/C group, first token of the tile
    int lo, hi;        // rows of the tile this pass covers
    int flags;         // kFirst: first pass of an item (load the state), kLast: last pass (store it), kStop
    int pair, seg;
    float cend[2], cref[2];
    int pad[3];
};
static_assert(sizeof(Desc) == 64, "descriptor layout");

struct Barriers {
    uint64_t cbld_full[2], cbld_empty[2];
    uint64_t ring_full[kRing], ring_empty[kRing];
    uint64_t cb_full[2], cb_free, p_ready, p_free, y_full[2], y_free[2];
    uint64_t h_ready, h_free, xw_ready, xw_free, s_full, s_free;
    uint64_t drain[3];
    uint32_t tmem_base;
    uint32_t abort_flag;
    int cb_issued;
};
static_assert(sizeof(Barriers) <= 512, "barrier block");

struct alignas(64) Params {
    CUtensorMap tm_b, tm_c, tm_y;
    const __nv_bfloat16* x;
    __nv_bfloat16* y;
    const float* dt;
    const float* a;
    const float* d;
    const float* h0;
    const float* dt_bias;
    float dt_min, dt_max;
    float* h_final;
    float* chunk_states;
    int* status;
    long long* trace;
    int* seg_flags;      // [npairs]: warps of the state role that have stored their part of a segment's state
    float* seg_state;    // [npairs][2][P][R]
    int B, S, H, G, Q, NC, tiles, tps, nseg, npairs, nitems;
    int stall_loads;
};

#define BM_WAIT(bar, par)                                          \
    do {                                                           \
        uint32_t n_ = 0;                                           \
        _Pragma("unroll 1")                                        \
        while (!mbar_try_wait((bar), (par)))                       \
            if (++n_ >= kWaitBudget) goto timed_out;               \
    } while (0)
// The same for a whole warp; the leave/stay decision is made warp-uniform so that no lane is left behind
// at a later __syncwarp or .aligned tcgen05 instruction.
#define BM_WAIT_WARP(bar, par)                                     \
    do {                                                           \
        uint32_t n_ = 0;                                           \
        bool ok_ = true;                                           \
        _Pragma("unroll 1")                                        \
        while (!mbar_try_wait((bar), (par)))                       \
            if (++n_ >= kWaitBudget) {                             \
                ok_ = false;                                       \
                break;                                             \
            }                                                      \
        if (!__all_sync(0xffffffffu, ok_)) goto timed_out;         \
    } while (0)

// Optional timeline instrumentation (development builds only, -DBM_SSD2_TRACE): CTA 0 records clock64() at
// role milestones of its first passes into prm.trace[role][pass][event].
#ifdef BM_SSD2_TRACE
#define BM_TRACE(role, it, ev)                                                                     \
    do {                                                                                           \
        if (blockIdx.x == 0 && (it) < 64 && lane == 0 && ((role) < 4 || (warp & 3) == 3))           \
            prm.trace[((role) * 64 + (it)) * 4 + (ev)] = clock64();                                \
    } while (0)
#else
#define BM_TRACE(role, it, ev) do { } while (0)
#endif

__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void stg_v4(void* p, const uint4& v) {
    asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// clamp(softplus(x)) of the fused dt path (src/mamba2/mamba2.rs:692-697); out of line: rarely used
__device__ __noinline__ float dt_activation(float x, float lo, float hi) { return fminf(fmaxf(softplus_f32(x), lo), hi); }

__device__ __forceinline__ float* ring_entry(unsigned char* smem, int it) {
    return reinterpret_cast<float*>(smem + kOffRing + (uint32_t)(it & (kRing - 1)) * kRingEntryBytes);
}
__device__ __forceinline__ const Desc* ring_desc(const float* entry) { return reinterpret_cast<const Desc*>(entry + 4 * T); }

// Timeout path only.  Every role has left its loop; the threads that issued asynchronous work wait, bounded
// again, for what they may still have in flight before TMEM is released.
__device__ __noinline__ void drain_after_timeout(Barriers* bars, int warp, int lane) {
    if (lane == 0 && (warp == 1 || warp == 2)) {
        uint64_t* db = &bars->drain[warp - 1];
        umma_commit(db);
        for (uint32_t n = 0; n < kWaitBudget && !mbar_try_wait(db, 0); ++n) {}
    }
    if (warp == 0 && lane == 0) {
        const int issued = bars->cb_issued;
        for (int k = issued - 1; k >= 0 && k >= issued - 2; --k)
            for (uint32_t n = 0; n < kWaitBudget && !mbar_try_wait(&bars->cbld_full[k & 1], (k >> 1) & 1); ++n) {}
    }
}

__global__ void __launch_bounds__(kThreads, 1) ssd2_pair_kernel(const __grid_constant__ Params prm) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    Barriers* bars = reinterpret_cast<Barriers*>(smem + kOffBar);
    volatile uint32_t* abort_flag = &bars->abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->cbld_full[i], 1);
            mbar_init(&bars->cbld_empty[i], 2);   // commits of both MMA issuers
        }
        for (int i = 0; i < kRing; ++i) {
            mbar_init(&bars->ring_full[i], 1);
            mbar_init(&bars->ring_empty[i], 19);  // producer, 2 issuers, 4 mask, 8 state, 4 epilogue warps
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->cb_full[i], 1);
            mbar_init(&bars->y_full[i], 1);
            mbar_init(&bars->y_free[i], 4);
        }
        mbar_init(&bars->cb_free, 4);
        mbar_init(&bars->p_ready, 4);
        mbar_init(&bars->p_free, 1);
        mbar_init(&bars->h_ready, 8);
        mbar_init(&bars->h_free, 1);
        mbar_init(&bars->xw_ready, 8);
        mbar_init(&bars->xw_free, 1);             // one commit after the last MMA that reads the scaled tiles
        mbar_init(&bars->s_full, 1);
        mbar_init(&bars->s_free, 8);
        for (int i = 0; i < 3; ++i) mbar_init(&bars->drain[i], 1);
        bars->abort_flag = 0;
        bars->cb_issued = 0;
        fence_mbar_init();
    }
    if (warp == 2) {
        tmem_alloc(&bars->tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    const int hpg = prm.H / prm.G;
    const uint32_t c_base = smem_u32(smem + kOffC), b_base = smem_u32(smem + kOffB);
    const uint32_t xw_base = smem_u32(smem + kOffXw), h_base = smem_u32(smem + kOffH);

    // Register budget per warpgroup (the CTA is launched with 640 x 96 registers; the four numbers plus twice
    // the state warpgroups' sum to 5 x 96): single-thread roles and the scan 64, mask pass 96, the two state
    // warpgroups 128 each (64 of state, 32 of prefetched X per thread), epilogue 64.
    if (warp < 4) {
        setmaxnreg_dec<64>();
        if (warp == 0) {
            // ------------------------------------------------------------------ TMA producer: C and B tiles
            if (lane == 0) {
                tma_prefetch_desc(&prm.tm_b);
                tma_prefetch_desc(&prm.tm_c);
                for (int it = 0;; ++it) {
                    const float* e = ring_entry(smem, it);
                    BM_WAIT(&bars->ring_full[it & (kRing - 1)], (it / kRing) & 1);
                    const Desc* ds = ring_desc(e);
                    const int flags = ds->flags, b = ds->b, g = ds->g, s0 = ds->s0;
                    mbar_arrive(&bars->ring_empty[it & (kRing - 1)]);
                    if (flags & kStop) break;
                    if (prm.stall_loads) continue;
                    const int st = it & 1;
                    BM_WAIT(&bars->cbld_empty[st], ((it >> 1) & 1) ^ 1);
                    mbar_expect_tx(&bars->cbld_full[st], kLoadBytesCB);
                    unsigned char* cs = smem + kOffC + st * 2 * kPanel;
                    unsigned char* bs = smem + kOffB + st * 2 * kPanel;
                    tma_load_4d(cs, &prm.tm_c, &bars->cbld_full[st], 0, g, s0, b);
                    tma_load_4d(cs + kPanel, &prm.tm_c, &bars->cbld_full[st], 64, g, s0, b);
                    tma_load_4d(bs, &prm.tm_b, &bars->cbld_full[st], 0, g, s0, b);
                    tma_load_4d(bs + kPanel, &prm.tm_b, &bars->cbld_full[st], 64, g, s0, b);
                    bars->cb_issued = it + 1;
                    BM_TRACE(0, it, 0);
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------------ MMA issuer: CB = C B^T
            if (lane == 0) {
                const uint32_t id_cb = umma_idesc_bf16(128, 128, false, false);
                for (int it = 0;; ++it) {
                    BM_WAIT(&bars->ring_full[it & (kRing - 1)], (it / kRing) & 1);
                    const int flags = ring_desc(ring_entry(smem, it))->flags;
                    mbar_arrive(&bars->ring_empty[it & (kRing - 1)]);
                    if (flags & kStop) break;
                    const int st = it & 1;
                    BM_WAIT(&bars->cbld_full[st], (it >> 1) & 1);
                    BM_WAIT(&bars->y_free[it & 1], ((it >> 1) & 1) ^ 1);   // the epilogue two passes back has drained these columns
                    BM_TRACE(1, it, 0);
                    tc_fence_after();
                    const uint64_t da = umma_desc_kmajor(c_base + st * 2 * kPanel), db = umma_desc_kmajor(b_base + st * 2 * kPanel);
#pragma unroll 1
                    for (int k = 0; k < 8; ++k) {
                        const uint32_t off = (k >> 2) * kPanel + (k & 3) * 32;
                        umma_ss(tmem + kColYC + (it & 1) * 128, desc_advance(da, off), desc_advance(db, off), id_cb, k > 0);
                    }
                    umma_commit(&bars->cb_full[it & 1]);
                    umma_commit(&bars->cbld_empty[st]);
                }
            }
        } else if (warp == 2) {
            // ------------------------------------------------------------------ MMA issuer: readout and state, both heads
            if (lane == 0) {
                const uint32_t id_y2 = umma_idesc_bf16(128, 128, false, true);
                const uint32_t id_s = umma_idesc_bf16(128, 128, true, true);
                const uint32_t id_y1 = umma_idesc_bf16(128, 64, false, true);
                const uint64_t dh = umma_desc_mnmajor(h_base, kPanel);      // [H'_A | H'_B], 64-column blocks one panel apart
                const uint64_t dxw = umma_desc_mnmajor(xw_base, kPanel);    // [Xw_A | Xw_B]
                for (int it = 0;; ++it) {
                    BM_WAIT(&bars->ring_full[it & (kRing - 1)], (it / kRing) & 1);
                    const int flags = ring_desc(ring_entry(smem, it))->flags;
                    mbar_arrive(&bars->ring_empty[it & (kRing - 1)]);
                    if (flags & kStop) break;
                    const int st = it & 1, ph = it & 1;
                    // Y = C [H'_A | H'_B]^T once both heads have published the state entering the pass and the mask
                    // pass has taken C B^T out of the accumulator
                    BM_WAIT(&bars->cbld_full[st], (it >> 1) & 1);
                    BM_WAIT(&bars->h_ready, ph);
                    BM_WAIT(&bars->cb_free, ph);
                    BM_TRACE(2, it, 0);
                    tc_fence_after();
                    const uint32_t ycol = tmem + kColYC + (it & 1) * 128;
                    const uint64_t dc = umma_desc_kmajor(c_base + st * 2 * kPanel);
#pragma unroll 1
                    for (int k = 0; k < 8; ++k) {
                        const uint32_t off = (k >> 2) * kPanel + (k & 3) * 32;
                        umma_ss(ycol, desc_advance(dc, off), desc_advance(dh, k * 2048), id_y2, k > 0);
                    }
                    umma_commit(&bars->h_free);
                    // S = B^T [Xw_A | Xw_B]
                    BM_WAIT(&bars->xw_ready, ph);
                    BM_WAIT(&bars->s_free, ph ^ 1);
                    BM_TRACE(2, it, 1);
                    tc_fence_after();
                    const uint64_t dbm = umma_desc_mnmajor(b_base + st * 2 * kPanel, kPanel);
#pragma unroll 1
                    for (int k = 0; k < 8; ++k)
                        umma_ss(tmem + kColS, desc_advance(dbm, k * 2048), desc_advance(dxw, k * 2048), id_s, k > 0);
                    umma_commit(&bars->s_full);
                    umma_commit(&bars->cbld_empty[st]);
                    // Y += P_h Xw_h for both heads, on top of the readout
                    BM_WAIT(&bars->p_ready, ph);
                    BM_TRACE(2, it, 2);
                    tc_fence_after();
#pragma unroll 1
                    for (int hh = 0; hh < 2; ++hh)
#pragma unroll 1
                        for (int k = 0; k < 8; ++k)
                            umma_ts(ycol + hh * 64, tmem + kColP + hh * 64 + k * 8, desc_advance(dxw, hh * kPanel + k * 2048), id_y1, true);
                    umma_commit(&bars->y_full[it & 1]);
                    umma_commit(&bars->p_free);
                    umma_commit(&bars->xw_free);
                }
            }
        } else {
            // ------------------------------------------------------------------ decay scan and pass scheduler
            // A lane owns four consecutive tokens of the tile for both heads.  Per tile: the log2-domain
            // cumulative decay of each head, the number of sub-ranges the tile has to be walked in, and one
            // ring entry per sub-range (cum relative to the sub-range start, row weights, descriptor).
            // The per-head work is written as rolled loops over the head with the per-token values parked in a
            // small shared-memory scratch: this role runs once per tile, so its code size is what it costs.
            const float log2e = 1.4426950408889634f;
            float* scratch = reinterpret_cast<float*>(smem + kOffScan);   // [head][cum 128 | dt 128]
            int it = 0;
            // dt of a tile for both heads (four tokens per lane), fetched one tile ahead inside an item
            float nv0[4], nv1[4];
            auto fetch_dt = [&](int b, int ha, int tile) {
                const int s0 = tile * T, left = prm.S - s0;
                const float* row = prm.dt + ((int64_t)b * prm.S + s0 + lane * 4) * prm.H + ha;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const bool live = lane * 4 + k < left;
                    nv0[k] = live ? __ldg(row + (int64_t)k * prm.H) : 0.f;
                    nv1[k] = live ? __ldg(row + (int64_t)k * prm.H + 1) : 0.f;
                }
            };
            for (int item = blockIdx.x; item < prm.nitems; item += gridDim.x) {
                const int seg = item / prm.npairs, pair = item - seg * prm.npairs;
                const int b = pair / (prm.H / 2), ha = 2 * (pair - b * (prm.H / 2)), g = ha / hpg;
                const int tile_lo = seg * prm.tps, tile_hi = min(prm.tiles, tile_lo + prm.tps);
                fetch_dt(b, ha, tile_lo);
                for (int tile = tile_lo; tile < tile_hi; ++tile) {
                    const int s0 = tile * T, left = prm.S - s0;
                    __syncwarp();
#pragma unroll 1
                    for (int hh = 0; hh < 2; ++hh) {
                        const float ah = prm.a[ha + hh] * log2e;
                        float4 dv, cv;
                        float* d4 = &dv.x;
                        float* c4 = &cv.x;
                        float run = 0.f;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            float x = hh ? nv1[k] : nv0[k];
                            if (prm.dt_bias && lane * 4 + k < left) x = dt_activation(x + prm.dt_bias[ha + hh], prm.dt_min, prm.dt_max);
                            d4[k] = x;
                            run = fmaf(x, ah, run);
                            c4[k] = run;
                        }
                        float inc = run;
#pragma unroll
                        for (int o = 1; o < 32; o <<= 1) {
                            const float up = __shfl_up_sync(0xffffffffu, inc, o);
                            if (lane >= o) inc += up;
                        }
                        const float ex = inc - run;
#pragma unroll
                        for (int k = 0; k < 4; ++k) c4[k] += ex;
                        reinterpret_cast<float4*>(scratch + hh * 2 * T)[lane] = cv;
                        reinterpret_cast<float4*>(scratch + hh * 2 * T + T)[lane] = dv;
                    }
                    __syncwarp();
                    if (tile + 1 < tile_hi) fetch_dt(b, ha, tile + 1);
                    // sub-ranges: halve until every sub-range of both heads decays by at most 2^-180
                    int len = T;
#pragma unroll 1
                    for (;;) {
                        // the sub-range this lane's first token lies in, for both heads
                        const int r0 = (lane * 4) & ~(len - 1), r1 = r0 + len - 1;
                        bool bad = false;
#pragma unroll 1
                        for (int hh = 0; hh < 2; ++hh) {
                            const float* cum = scratch + hh * 2 * T;
                            const float dec = cum[r1] - (r0 ? cum[r0 - 1] : 0.f);
                            bad |= !(fabsf(dec) <= kMaxRangeLog2Decay);
                        }
                        if (!__any_sync(0xffffffffu, bad)) break;
                        if (len == 4) {   // below a lane's four tokens: single tokens, always representable
                            len = 1;
                            break;
                        }
                        len >>= 1;
                    }
                    const int live_rows = left < T ? left : T;
#pragma unroll 1
                    for (int lo = 0; lo < live_rows; lo += len) {
                        const int hi = lo + len;
                        float* e = ring_entry(smem, it);
                        BM_TRACE(3, it, 1);
                        BM_WAIT_WARP(&bars->ring_empty[it & (kRing - 1)], ((it / kRing) & 1) ^ 1);
                        BM_TRACE(3, it, 2);
                        Desc* ds = reinterpret_cast<Desc*>(e + 4 * T);
#pragma unroll 1
                        for (int hh = 0; hh < 2; ++hh) {
                            const float* cum = scratch + hh * 2 * T;
                            const float base = lo ? cum[lo - 1] : 0.f;
                            const float cend = cum[hi - 1] - base;
                            const float cref = len == 1 ? cend : 0.5f * cend;
                            const float4 cv = reinterpret_cast<const float4*>(cum)[lane];
                            const float4 dv = reinterpret_cast<const float4*>(cum + T)[lane];
                            const float* c4 = &cv.x;
                            const float* d4 = &dv.x;
                            float4 co, wo;
                            float* cop = &co.x;
                            float* wop = &wo.x;
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const int t = lane * 4 + k;
                                const bool inr = t >= lo && t < hi;
                                const float c = c4[k] - base;
                                cop[k] = inr ? c : 0.f;
                                wop[k] = (inr && t < left) ? fmaxf(d4[k], kMinStep) * ex2(cref - c) : 0.f;
                            }
                            reinterpret_cast<float4*>(e + hh * 2 * T)[lane] = co;
                            reinterpret_cast<float4*>(e + hh * 2 * T + T)[lane] = wo;
                            if (lane == 0) ds->cend[hh] = cend, ds->cref[hh] = cref;
                        }
                        if (lane == 0) {
                            ds->b = b, ds->ha = ha, ds->g = g, ds->s0 = s0, ds->lo = lo, ds->hi = hi;
                            ds->pair = pair, ds->seg = seg;
                            ds->flags = ((tile == tile_lo && lo == 0) ? kFirst : 0) |
                                        ((tile == tile_hi - 1 && hi >= live_rows) ? kLast : 0) | (lo == 0 ? kTileStart : 0);
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bars->ring_full[it & (kRing - 1)]);
                        BM_TRACE(3, it, 0);
                        ++it;
                    }
                }
            }
            // end marker
            BM_WAIT_WARP(&bars->ring_empty[it & (kRing - 1)], ((it / kRing) & 1) ^ 1);
            if (lane == 0) {
                reinterpret_cast<Desc*>(ring_entry(smem, it) + 4 * T)->flags = kStop;
                mbar_arrive(&bars->ring_full[it & (kRing - 1)]);
            }
        }
    } else if (warp < 8) {
        // ------------------------------------------------------------------ mask pass: CB -> P_A, P_B
        const int q = warp & 3, t = q * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
        // bf16-pair masks of the diagonal block: column 32q + j is kept for row 32q + lane when j <= lane
        uint32_t causal[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            causal[j] = (2 * j <= lane ? 0x0000ffffu : 0u) | (2 * j + 1 <= lane ? 0xffff0000u : 0u);
            asm volatile("" : "+r"(causal[j]));
        }
        {   // the blocks above the diagonal stay zero for the whole launch
            uint32_t z[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) z[j] = 0u;
            for (int c = q + 1; c < 4; ++c) {
                tmem_st16(lane_addr + kColP + c * 16, z);
                tmem_st16(lane_addr + kColP + 64 + c * 16, z);
            }
            tmem_wait_st();
        }
        for (int it = 0;; ++it) {
            const float* e = ring_entry(smem, it);
            BM_WAIT_WARP(&bars->ring_full[it & (kRing - 1)], (it / kRing) & 1);
            const Desc* ds = ring_desc(e);
            if (ds->flags & kStop) break;
            const int ph = it & 1;
            // skip term: y_t = E'_t (P Xw)_t with E'_t = 2^(cum_t - cref), so D x_t = E'_t (D / (w_t E'_t)) Xw_t; the
            // factor D / (w_t E'_t) = D / dt_t is added to the diagonal of P as a packed bf16 pair
            uint32_t patch[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const float w = e[hh * 2 * T + T + t];
                const float dsk = prm.d ? prm.d[ds->ha + hh] : 0.f;
                const float dw = w > 0.f ? (dsk / w) * ex2(ds->cref[hh] - e[hh * 2 * T + t]) : 0.f;
                patch[hh] = (lane & 1) ? pack_bf16x2(0.f, dw) : pack_bf16x2(dw, 0.f);
            }
            BM_WAIT_WARP(&bars->cb_full[it & 1], (it >> 1) & 1);
            BM_WAIT_WARP(&bars->p_free, ph ^ 1);      // P Xw of the previous pass has read P
            BM_TRACE(4, it, 0);
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c <= q; ++c) {
                uint32_t r[32], out[16];
                tmem_ld32(lane_addr + kColYC + (it & 1) * 128 + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j) out[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                if (c < q) {
                    tmem_st16(lane_addr + kColP + c * 16, out);
                    tmem_st16(lane_addr + kColP + 64 + c * 16, out);
                } else {
                    // all of CB is in registers or already converted: CB may be overwritten by the next tile
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->cb_free);
                    uint32_t oa[16], ob[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const uint32_t m = out[j] & causal[j];
                        uint32_t pa = m, pb = m;
                        if (j == (lane >> 1)) {
                            asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(pa) : "r"(m), "r"(patch[0]));
                            asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(pb) : "r"(m), "r"(patch[1]));
                        }
                        oa[j] = pa;
                        ob[j] = pb;
                    }
                    tmem_st16(lane_addr + kColP + c * 16, oa);
                    tmem_st16(lane_addr + kColP + 64 + c * 16, ob);
                }
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            BM_TRACE(4, it, 1);
            if (lane == 0) {
                mbar_arrive(&bars->p_ready);
                mbar_arrive(&bars->ring_empty[it & (kRing - 1)]);
            }
        }
    } else if (warp < 16) {
        // ------------------------------------------------------------------ X scaling, state update, state publishing
        setmaxnreg_inc<128>();
        const int hh = (warp - 8) >> 2;              // head of the pair this warpgroup owns
        const int q = warp & 3, t = q * 32 + lane;   // token row for the X pass, state row r for the state
        const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
        unsigned char* xw = smem + kOffXw + hh * kPanel;
        unsigned char* hs = smem + kOffH + hh * kPanel;
        float hst[P];
        uint4 xr[8];
        // X rows of a pass, fetched into registers one pass ahead.  Eight lanes share a row (16 bytes each), so one
        // load instruction of the warp covers four whole 128-byte rows: piece i of this thread is chunk
        // (lane & 7) of row 32 q + 4 i + (lane >> 3).
        auto fetch_x = [&](const Desc* ds) {
            const __nv_bfloat16* src = prm.x + (((int64_t)ds->b * prm.S + ds->s0) * prm.H + ds->ha + hh) * P + (lane & 7) * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = q * 32 + i * 4 + (lane >> 3);
                xr[i] = ds->s0 + r < prm.S ? ldg_nc_v4(src + (int64_t)r * prm.H * P) : make_uint4(0u, 0u, 0u, 0u);
            }
        };
        auto publish_state = [&](float factor) {
            // bf16 copy of factor * h as the MN-major B operand of the readout MMA
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                uint4 v;
                v.x = pack_bf16x2(hst[8 * k] * factor, hst[8 * k + 1] * factor);
                v.y = pack_bf16x2(hst[8 * k + 2] * factor, hst[8 * k + 3] * factor);
                v.z = pack_bf16x2(hst[8 * k + 4] * factor, hst[8 * k + 5] * factor);
                v.w = pack_bf16x2(hst[8 * k + 6] * factor, hst[8 * k + 7] * factor);
                *reinterpret_cast<uint4*>(hs + sw128_offset(t, k)) = v;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->h_ready);
        };
        BM_WAIT_WARP(&bars->ring_full[0], 0);
        if (!(ring_desc(ring_entry(smem, 0))->flags & kStop)) fetch_x(ring_desc(ring_entry(smem, 0)));
        for (int it = 0;; ++it) {
            const float* e = ring_entry(smem, it);
            BM_WAIT_WARP(&bars->ring_full[it & (kRing - 1)], (it / kRing) & 1);
            const Desc* ds = ring_desc(e);
            const int flags = ds->flags;
            if (flags & kStop) break;
            const int ph = it & 1;
            const int h = ds->ha + hh;
            const int64_t state_base = ((int64_t)ds->b * prm.H + h) * P * R;
            if (flags & kFirst) {
                // item start: the state entering the segment -> registers
                const float* src = nullptr;
                if (ds->seg > 0) {
                    // the previous segment of this pair: its 8 state warps bump the counter after storing
                    const int want = 8 * ds->seg;
                    bool ok = true;
                    if (lane == 0) {
                        uint32_t n = 0;
                        while (ld_acquire(prm.seg_flags + ds->pair) < want)
                            if (++n >= kWaitBudget) {
                                ok = false;
                                break;
                            }
                    }
                    if (!__all_sync(0xffffffffu, ok)) goto timed_out;
                    src = prm.seg_state + ((int64_t)ds->pair * 2 + hh) * P * R;
                } else if (prm.h0) {
                    src = prm.h0 + state_base;
                }
#pragma unroll
                for (int p = 0; p < P; ++p) hst[p] = src ? __ldcg(src + (int64_t)p * R + t) : 0.f;
            }
            // the state entering this pass, scaled to the pass's reference point, is its readout operand; the
            // operand tile is free once the previous pass's readout MMA has completed
            if (it > 0) BM_WAIT_WARP(&bars->h_free, (it - 1) & 1);
            publish_state(ex2(ds->cref[hh]));
            if (__builtin_expect(prm.chunk_states != nullptr, 0) && (flags & kTileStart) && ds->s0 % prm.Q == 0) {
                float* cs = prm.chunk_states + (((int64_t)ds->b * prm.NC + ds->s0 / prm.Q) * prm.H + h) * P * R;
#pragma unroll
                for (int p = 0; p < P; ++p) cs[(int64_t)p * R + t] = hst[p];
            }
            // scaled tile Xw = X * w (rows keep their swizzled positions); both MMAs of the previous pass that
            // read the tile have completed
            {
                const float* wv = e + hh * 2 * T + T;
                BM_WAIT_WARP(&bars->xw_free, ph ^ 1);
                BM_TRACE(5 + 2 * hh, it, 0);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = q * 32 + i * 4 + (lane >> 3);
                    const float w = wv[r];
                    const float2 f0 = unpack_bf16x2(xr[i].x), f1 = unpack_bf16x2(xr[i].y), f2 = unpack_bf16x2(xr[i].z),
                                 f3 = unpack_bf16x2(xr[i].w);
                    uint4 o;
                    o.x = pack_bf16x2(f0.x * w, f0.y * w);
                    o.y = pack_bf16x2(f1.x * w, f1.y * w);
                    o.z = pack_bf16x2(f2.x * w, f2.y * w);
                    o.w = pack_bf16x2(f3.x * w, f3.y * w);
                    *reinterpret_cast<uint4*>(xw + sw128_offset(r, lane & 7)) = o;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->xw_ready);
            }
            // X rows of the next pass, one pass ahead (the scan runs further ahead than that)
            const float* en = ring_entry(smem, it + 1);
            BM_WAIT_WARP(&bars->ring_full[(it + 1) & (kRing - 1)], ((it + 1) / kRing) & 1);
            const Desc* dn = ring_desc(en);
            const bool more = !(dn->flags & kStop);
            BM_TRACE(5 + 2 * hh, it, 1);
            if (more) fetch_x(dn);
            // state update h <- 2^cend h + 2^(cend - cref) S
            {
                const float cend = ds->cend[hh], cref = ds->cref[hh];
                const float decay = ex2(cend), gain = ex2(cend - cref);
                BM_WAIT_WARP(&bars->s_full, ph);
                BM_TRACE(5 + 2 * hh, it, 2);
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t sv[16];
                    tmem_ld16(lane_addr + kColS + hh * 64 + c * 16, sv);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) hst[c * 16 + j] = fmaf(decay, hst[c * 16 + j], gain * __uint_as_float(sv[j]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->s_free);
            }
            if (flags & kLast) {
                // item end: the state leaves through the segment buffer, or is the final state
                const bool final_seg = ds->seg == prm.nseg - 1;
                float* dst = final_seg ? prm.h_final + state_base : prm.seg_state + ((int64_t)ds->pair * 2 + hh) * P * R;
#pragma unroll
                for (int p = 0; p < P; ++p) __stcg(dst + (int64_t)p * R + t, hst[p]);
                if (!final_seg) {
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) atomicAdd(prm.seg_flags + ds->pair, 1);
                }
            }
            __syncwarp();
            BM_TRACE(5 + 2 * hh, it, 3);
            if (lane == 0) mbar_arrive(&bars->ring_empty[it & (kRing - 1)]);
        }
    } else {
        // ------------------------------------------------------------------ epilogue: y = 2^(cum - cref) Y, to global memory
        setmaxnreg_dec<64>();
        const int q = warp & 3, t = q * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
        unsigned char* stage = smem + kOffStage + q * 2 * kStageTileBytes;
        const uint32_t srow = lane * 64, sxor = (lane >> 1) & 3;   // 64-byte swizzle: chunk ^ ((row >> 1) & 3)
        for (int it = 0;; ++it) {
            const float* e = ring_entry(smem, it);
            BM_WAIT_WARP(&bars->ring_full[it & (kRing - 1)], (it / kRing) & 1);
            const Desc* ds = ring_desc(e);
            if (ds->flags & kStop) break;
            const int ph = it & 1;
            const int row = ds->s0 + t;
            const bool store = t >= ds->lo && t < ds->hi && row < prm.S;
            float ef[2];
            ef[0] = ex2(e[t] - ds->cref[0]);
            ef[1] = ex2(e[2 * T + t] - ds->cref[1]);
            __nv_bfloat16* dst = prm.y + (((int64_t)ds->b * prm.S + row) * prm.H + ds->ha) * P;
            // a pass over the whole tile leaves through the staging tiles and TMA stores (rows past the end of
            // the sequence are clipped by the tensor map); a sub-range pass writes its rows directly
            const bool whole = ds->lo == 0 && ds->hi == T;
            const int b = ds->b, ha = ds->ha, row0 = ds->s0 + q * 32;
            BM_TRACE(6, it, 0);
            BM_WAIT_WARP(&bars->y_full[it & 1], (it >> 1) & 1);
            BM_TRACE(6, it, 1);
            tc_fence_after();
#pragma unroll 1
            for (int part = 0; part < 4; ++part) {      // head A columns 0-31, 32-63, head B columns 0-31, 32-63
                uint32_t yv[32];
                tmem_ld32(lane_addr + kColYC + (it & 1) * 128 + part * 32, yv);
                tmem_wait_ld();
                if (part == 3) {
                    // the accumulator is in registers: the next pass's readout MMA may overwrite it
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->y_free[it & 1]);
                }
                const float f = part < 2 ? ef[0] : ef[1];
                uint4 o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    o[k].x = pack_bf16x2(__uint_as_float(yv[8 * k]) * f, __uint_as_float(yv[8 * k + 1]) * f);
                    o[k].y = pack_bf16x2(__uint_as_float(yv[8 * k + 2]) * f, __uint_as_float(yv[8 * k + 3]) * f);
                    o[k].z = pack_bf16x2(__uint_as_float(yv[8 * k + 4]) * f, __uint_as_float(yv[8 * k + 5]) * f);
                    o[k].w = pack_bf16x2(__uint_as_float(yv[8 * k + 6]) * f, __uint_as_float(yv[8 * k + 7]) * f);
                }
                if (whole) {
                    unsigned char* tile = stage + (part & 1) * kStageTileBytes;
                    // the store issued from this tile two parts ago must have finished reading it
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
#pragma unroll
                    for (int k = 0; k < 4; ++k) *reinterpret_cast<uint4*>(tile + srow + ((k ^ sxor) << 4)) = o[k];
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_4d(&prm.tm_y, tile, (part & 1) * 32, ha + (part >> 1), row0, b);
                        tma_store_commit();
                    }
                } else if (store) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) stg_v4(dst + (part >> 1) * P + (part & 1) * 32 + k * 8, o[k]);
                }
            }
            __syncwarp();
            BM_TRACE(6, it, 2);
            if (lane == 0) mbar_arrive(&bars->ring_empty[it & (kRing - 1)]);
        }
    }
    goto done;
timed_out:
    atomicExch(prm.status, (int)BM_ERR_TIMEOUT);
    *abort_flag = 1;
done:
    if (warp >= 16 && lane == 0) tma_store_wait_all<0>();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag != 0u) {
        drain_after_timeout(bars, warp, lane);
        tc_fence_before();
        __syncthreads();
    }
    if (warp == 2) tmem_dealloc(tmem, 512);
}

int num_sms_pair() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

// Number of sequence segments per head pair: the count (up to 8) that minimises the longest CTA's work,
// rounds of items x tiles per item, with a small charge per segment for the state hand-off.
int choose_segments(int npairs, int tiles, int grid) {
    int best = 1;
    double best_cost = 1e30;
    for (int n = 1; n <= 8 && n <= tiles; ++n) {
        const int tps = (tiles + n - 1) / n;
        const int nseg = (tiles + tps - 1) / tps;
        if (nseg != n) continue;
        const int64_t rounds = ((int64_t)npairs * nseg + grid - 1) / grid;
        const double cost = (double)rounds * tps + 0.15 * nseg;
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = n;
        }
    }
    return best;
}

struct Plan {
    int npairs, tiles, nseg, tps, grid;
    size_t off_flags, off_state, off_trace, bytes;
};

Plan make_plan(const bm_ssd2_fwd_args* a) {
    Plan p{};
    p.npairs = a->batch * (a->nheads / 2);
    p.tiles = (int)cdiv(a->seqlen, T);
    p.grid = num_sms_pair();
    p.nseg = choose_segments(p.npairs, p.tiles, p.grid);
    p.tps = (p.tiles + p.nseg - 1) / p.nseg;
    const int nitems = p.npairs * p.nseg;
    if (nitems < p.grid) p.grid = nitems;
    p.off_flags = 256;
    p.off_state = align_up(p.off_flags + (size_t)p.npairs * sizeof(int), 256);
    p.off_trace = p.off_state + (p.nseg > 1 ? (size_t)p.npairs * 2 * P * R * sizeof(float) : 0);
    p.bytes = p.off_trace + 8 * 64 * 4 * 8;   // timeline area of development builds
    return p;
}

}  // namespace

const char* ssd2_pair_why_not(const bm_ssd2_fwd_args* a) {
    if (const char* w = ssd2_why_not(a)) return w;
    if (a->nheads % 2 != 0 || (a->nheads / a->ngroups) % 2 != 0) return "heads per group must be even to pair heads";
    return nullptr;
}

bool ssd2_pair_supported(const bm_ssd2_fwd_args* a) { return ssd2_pair_why_not(a) == nullptr; }

// Which of the two tensor-core kernels BM_PATH_AUTO / BM_PATH_TENSOR take.  Measured on the 2.7B prefill shape the
// paired kernel moves less data on chip but, with every operand single-buffered, overlaps less: it runs level
// with the one-head kernel, so it stays opt-in (BM_PATH_TENSOR_PAIR) for now.
bool ssd2_pair_preferred(const bm_ssd2_fwd_args*) { return false; }

size_t ssd2_pair_workspace_bytes(const bm_ssd2_fwd_args* a) { return make_plan(a).bytes; }

int32_t ssd2_pair_run(const bm_ssd2_fwd_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    const Plan pl = make_plan(a);
    if (workspace == nullptr || workspace_bytes < pl.bytes)
        return fail(BM_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", workspace_bytes, pl.bytes);
    Params prm{};
    const char* err = nullptr;
    const uint64_t S = a->seqlen, G = a->ngroups, B = a->batch;
    const uint32_t box[4] = {64, 1, (uint32_t)T, 1};
    {
        const uint64_t dims[4] = {(uint64_t)R, G, S, B};
        const uint64_t strides[3] = {(uint64_t)R * 2, G * R * 2, S * G * R * 2};
        if (!make_tensor_map_bf16(&prm.tm_b, a->b, 4, dims, strides, box, 128, &err) ||
            !make_tensor_map_bf16(&prm.tm_c, a->c, 4, dims, strides, box, 128, &err))
            return fail(BM_ERR_CUDA, "tensor map (b/c): %s", err);
    }
    {
        const uint64_t H = a->nheads;
        const uint64_t dims[4] = {(uint64_t)P, H, S, B};
        const uint64_t strides[3] = {(uint64_t)P * 2, H * P * 2, S * H * P * 2};
        const uint32_t box_y[4] = {32, 1, 32, 1};  // one column half of one epilogue warp's rows per store
        if (!make_tensor_map_bf16(&prm.tm_y, a->y, 4, dims, strides, box_y, 64, &err))
            return fail(BM_ERR_CUDA, "tensor map (y): %s", err);
    }
    char* ws = static_cast<char*>(workspace);
    prm.x = static_cast<const __nv_bfloat16*>(a->x), prm.y = static_cast<__nv_bfloat16*>(a->y);
    prm.dt = a->dt, prm.a = a->a, prm.d = a->d, prm.h0 = a->h0, prm.dt_bias = a->dt_bias;
    prm.dt_min = a->dt_min, prm.dt_max = a->dt_max;
    prm.h_final = a->h_final, prm.chunk_states = a->chunk_states;
    prm.status = reinterpret_cast<int*>(ws);
    prm.seg_flags = reinterpret_cast<int*>(ws + pl.off_flags);
    prm.seg_state = reinterpret_cast<float*>(ws + pl.off_state);
    prm.trace = reinterpret_cast<long long*>(ws + pl.off_trace);
    prm.B = a->batch, prm.S = a->seqlen, prm.H = a->nheads, prm.G = a->ngroups, prm.Q = a->chunk_len;
    prm.NC = (int)cdiv(a->seqlen, a->chunk_len);
    prm.tiles = pl.tiles, prm.tps = pl.tps, prm.nseg = pl.nseg, prm.npairs = pl.npairs, prm.nitems = pl.npairs * pl.nseg;
    prm.stall_loads = (a->reserved == BM_DEBUG_STALL_LOADS) ? 1 : 0;
    {
        cudaError_t e = cudaFuncSetAttribute(ssd2_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(ssd2_pair_kernel)");
    }
    // status word and segment counters start at zero
    if (int32_t e = check_cuda(cudaMemsetAsync(workspace, 0, pl.off_state, stream), "cudaMemsetAsync(status)")) return e;
    ssd2_pair_kernel<<<pl.grid, kThreads, kSmemBytes, stream>>>(prm);
    return check_launch("ssd2_pair_kernel");
}

}  // namespace tc
}  // namespace bm
