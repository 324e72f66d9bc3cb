// Mamba-2 chunked SSD forward on the Blackwell tensor cores (tcgen05 / TMEM / TMA), bf16 operands
// with float32 accumulation and float32 recurrent state.
//
// One persistent CTA per SM walks (batch, head) units; inside a unit it walks the sequence in tiles of
// T = 128 tokens, keeping the head's state [r = 128, p = 64] in registers (float32) for the whole
// sequence, so no per-chunk state ever goes to HBM.  The tiles of all units, laid end to end, are cut
// into one contiguous range per CTA, so every CTA gets the same number of tiles (+-1) whatever the
// number of units; a unit that straddles two ranges is walked by two CTAs, the first handing the state
// it reached to the second through the workspace (a CTA walks its range's last piece first and its
// first piece last, so the piece it depends on has long been finished).  Per tile (reference formulas:
// src/mamba2/ssd/serial.rs:138-506, restated with the tile as the chunk):
//     CB   = C B^T                                          tcgen05 SS   (K1/K2)
//     P    = bf16(CB * exp(cum_t - cum_s)[s<=t] dt_s + D [s==t])  in TMEM (mask + skip of K5)
//     Y1   = P X            Y2 = C h^T                      tcgen05 TS / SS (K5)
//     y    = Y1 + exp(cum_t) Y2                             epilogue, TMA store
//     S    = B^T (X * dt exp(cum_end - cum))                tcgen05 SS   (K3)
//     h   <- exp(cum_end) h + S                             registers    (K4)
// Two dependency chains run concurrently and are software-pipelined across tiles:
//     scan chain   CB(i+1) | mask(i) -> Y1(i) -> epilogue(i)
//     state chain  Xw(i+1) | S(i) -> h(i+1) -> Y2(i+1)
// Warp roles (512 threads): warp 0 TMA loads, warp 1 MMA issue for the scan chain, warp 2 TMEM
// allocation + MMA issue for the state chain, warp 3 decay scan of dt, warps 4-7 mask pass (CB -> P),
// warps 8-11 X scaling and state update, warps 12-15 epilogue.
// Every wait is bounded; a wait that gives up stores BM_ERR_TIMEOUT in the status word of the
// workspace and raises the CTA's abort flag; the other roles leave as their own budgets run out.  Once
// all have left, the MMA issuers and the TMA producer wait (bounded again) for what they still have in
// flight before TMEM is released.
#include "ssd2_tc.cuh"
#include "tc_common.cuh"

namespace bm {
namespace tc {

namespace {

constexpr int T = 128;        // tokens per tile
constexpr int P = 64;         // head dim
constexpr int R = 128;        // state rank
constexpr int kThreads = 512;
constexpr int kCumStages = 4;
// Tiles whose total log2 decay |cend| stays below this use the factored mask: every factor
// exp2(+-cend) then stays far inside the float32 / bfloat16 exponent range.
constexpr float kFactoredMaxLog2Decay = 100.f;
// ... and whose per-row weight dt_t * 2^(cend - cum_t) of every live row stays above this floor: the
// factored form recovers the skip term D x by dividing the scaled tile by that weight.
// Together with |cend| <= 100 this only excludes rows whose step dt is itself below ~2^-12 of a tile's
// weakest weight: D / w stays below 2^112 (inside bf16) and x * w stays a normal number.
constexpr float kFactoredMinRowWeight = 1.9259299e-34f;   // 2^-112

// shared-memory map (bytes from a 1024-aligned base)
constexpr uint32_t kPanel = 16384;               // [128 rows x 128 B]
constexpr uint32_t kOffC = 0;                    // 2 stages x 2 panels
constexpr uint32_t kOffB = 65536;                // 2 stages x 2 panels
constexpr uint32_t kOffX = 131072;               // 2 stages x 1 panel
constexpr uint32_t kOffXw = 163840;              // 2 buffers x 1 panel
constexpr uint32_t kOffH = 196608;
constexpr uint32_t kOffCum = 212992;             // kCumStages x (4 arrays x 128 floats + flag)
constexpr uint32_t kCumStageBytes = 4 * T * 4 + 16;  // cum, dt, state weight, column factor + the tile's flag
constexpr int kCumDt = T, kCumW = 2 * T, kCumColf = 3 * T, kCumFlag = 4 * T;   // float offsets inside a stage
constexpr uint32_t kOffStage = 222208;           // y staging: 4 warps x [32 rows x 64 B], 64-byte swizzle (1024-aligned)
constexpr uint32_t kStageWarpBytes = 2048;
constexpr uint32_t kOffBar = kOffStage + 4 * kStageWarpBytes;
constexpr uint32_t kSmemBytes = kOffBar + 512 + 1024;  // barriers + alignment slack
static_assert(sizeof(uint64_t) * 43 + 64 <= 512, "barrier block outgrew its reserve");
static_assert(kOffCum + kCumStages * kCumStageBytes <= kOffStage, "decay ring overlaps the staging tile");
static_assert(kSmemBytes <= 232448, "over the 227 KB shared-memory limit of a CTA");
constexpr uint32_t kLoadBytesCB = 4 * kPanel;
constexpr uint32_t kLoadBytesX = kPanel;

// TMEM columns
constexpr uint32_t kColCB = 0;     // 2 buffers x 128 columns; P (bf16 pairs) aliases the first 64 of each
constexpr uint32_t kColY1 = 256;
constexpr uint32_t kColY2 = 320;
constexpr uint32_t kColS = 384;    // 2 buffers x 64 columns

struct Barriers {
    uint64_t cbld_full[2], cbld_empty[2];   // C + B tiles
    uint64_t xld_full[2], xld_empty[2];     // X tile (later the y staging tile)
    uint64_t cum_full[kCumStages], cum_empty[kCumStages];
    uint64_t cb_full[2], p_ready[2], p_free[2];
    uint64_t y1_full, y1_empty, y2_full, y2_empty;
    uint64_t h_ready, h_free, xw_ready[2], xw_free[2], xsrc_read[2], s_full[2], s_empty[2];
    uint64_t drain[3];                      // timeout path only: one per MMA-issuing thread
    uint64_t rot_done[2];                   // Mamba-3 with angles: the C + B stage has been rotated in place
    uint32_t tmem_base;
    uint32_t abort_flag;
    int x_issued, cb_issued;                // TMA producer: tiles whose X / C+B loads have been issued
    int w_total, w_items, w_unit0, w_first, w_last_end;   // this CTA's tile range, as items (see item_of)
};

struct alignas(64) Params {
    CUtensorMap tm_x, tm_b, tm_c, tm_y;
    const float* dt;
    const float* a;
    const float* d;
    const float* h0;
    const float* dt_bias;
    float dt_min, dt_max;
    float* h_final;
    float* chunk_states;
    int* status;
    int* handoff_flags;   // [grid] warps of CTA c that have stored the state their last piece ends with
    float* handoff;       // [grid][P][R] that state
    long long* trace;
    int B, S, H, G, Q, NC, tiles_per_unit, num_units;
    int share_q, share_r;   // (num_units * tiles_per_unit) / grid and the remainder
    int stall_loads;
    // Mamba-3 cores (kMode 1): S counts fused (time x rank) rows, St time steps, rows per step = 1 << log2m;
    // `dt` holds the column scale (NULL = 1, the generic core), `da` the per-step log decay, `gamma` the same-step
    // weight (NULL = 1)
    const float* da;
    const float* gamma;
    int St, log2m;
    // optional rotation of the B / C tiles inside the kernel: cumulative angles [b, St, H, rope_pairs]; pairs are
    // (2j, 2j+1) when `pairwise`, else (j, j + R/2)
    const float* angles;
    int rope_pairs, pairwise;
};

// Optional timeline instrumentation (development builds only, -DBM_SSD2_TRACE): CTA 0 records
// clock64() at role milestones of its first tiles into prm.trace[role][tile][event].
#ifdef BM_SSD2_TRACE
#define BM_TRACE(role, it, ev)                                                                     \
    do {                                                                                           \
        if (blockIdx.x == 0 && (it) < 64 && lane == 0 && ((role) < 4 || (warp & 3) == 3))           \
            prm.trace[((role) * 64 + (it)) * 4 + (ev)] = clock64();                                \
    } while (0)
#else
#define BM_TRACE(role, it, ev) do { } while (0)
#endif

// Bounded waits, inline: a short try_wait loop with an iteration budget (each try_wait itself blocks for a
// short hardware-defined time).  A wait that runs out of budget leaves through the `timed_out` label at the
// end of the kernel, which records BM_ERR_TIMEOUT and raises the CTA's abort flag.  The loops are kept to
// the bare minimum of instructions (there are dozens of them and the roles' hot code has to fit the
// instruction cache): they do not look at the abort flag, so after one role has given up the others leave
// when their own budgets run out, all of which count down concurrently.
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

// Several barriers at once: the phases are first tested without blocking, back to back, so that the usual
// case (all of them already complete) costs one shared-memory round trip instead of one per barrier.
#define BM_WAIT_WARP2(b1, p1, b2, p2)                                              \
    do {                                                                           \
        const bool f_ = mbar_test((b1), (p1)) & mbar_test((b2), (p2));             \
        if (!__all_sync(0xffffffffu, f_)) {                                        \
            BM_WAIT_WARP((b1), (p1));                                              \
            BM_WAIT_WARP((b2), (p2));                                              \
        }                                                                          \
    } while (0)
#define BM_WAIT_WARP3(b1, p1, b2, p2, b3, p3)                                      \
    do {                                                                           \
        const bool f_ = mbar_test((b1), (p1)) & mbar_test((b2), (p2)) & mbar_test((b3), (p3)); \
        if (!__all_sync(0xffffffffu, f_)) {                                        \
            BM_WAIT_WARP((b1), (p1));                                              \
            BM_WAIT_WARP((b2), (p2));                                              \
            BM_WAIT_WARP((b3), (p3));                                              \
        }                                                                          \
    } while (0)

// One 32-column block of the decay mask: out = bf16 pairs of P for columns [32c, 32c + 32).
// Exact form (any decay): the kernel exp(cum_t - cum_s) dt_s is applied here.
//   below the diagonal block:  rowfac * colf[s]   (both factors <= 1, reference = end of column block)
//   diagonal block:            exp2(cum_t - cum_s) dt_s, then the causal bit mask (the reference's -inf fill)
// Factored form (tiles whose total decay stays far inside the float32 exponent range): the whole
// kernel factors as exp2(cum_t - cend) * [dt_s exp2(cend - cum_s)]; the column factor is already in
// the scaled tile Xw and the row factor is applied in the epilogue, so P is just the causally masked CB.
// causal[j] keeps the halves of pair j at or below the diagonal (it depends on the lane only).
// The skip term D x is added by the epilogue in both forms.
__device__ __forceinline__ void mask_block(const uint32_t (&r)[32], uint32_t (&out)[16], bool factored, bool diagonal, int c,
                                           float ct, const float* cum2, const float* dtv, const float* colf,
                                           const uint32_t (&causal)[16]) {
    if (factored) {
        if (!diagonal) {
#pragma unroll
            for (int j = 0; j < 16; ++j) out[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                out[j] = pack_bf16x2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])) & causal[j];
        }
    } else if (!diagonal) {
        const float rf = ex2(ct - cum2[c * 32 + 31]);
        const uint64_t rf2 = pair_f32(rf, rf);
        const uint64_t* cf = reinterpret_cast<const uint64_t*>(colf + c * 32);
#pragma unroll
        for (int j = 0; j < 16; ++j) out[j] = pack_bf16x2_pair(mul2(pair_u32(r[2 * j], r[2 * j + 1]), mul2(rf2, cf[j])));
    } else {
        const uint64_t ct2 = pair_f32(ct, ct), neg1 = pair_f32(-1.f, -1.f);
        const uint64_t* cs = reinterpret_cast<const uint64_t*>(cum2 + c * 32);
        const uint64_t* ds = reinterpret_cast<const uint64_t*>(dtv + c * 32);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            // above the diagonal the exponent is positive and may overflow; the bit mask clears whatever
            // comes out of it
            float a0, a1;
            asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(fma2(cs[j], neg1, ct2)));
            const uint64_t w = mul2(pair_f32(ex2(a0), ex2(a1)), ds[j]);
            out[j] = pack_bf16x2_pair(mul2(pair_u32(r[2 * j], r[2 * j + 1]), w)) & causal[j];
        }
    }
}

// Diagonal block of the Mamba-3 cores (src/mamba3/single_ssd/ssd/serial.rs:216-258): rows and columns are fused
// (time, rank) indices, 1 << log2m per time step.  A column of an earlier step takes the decay kernel times
// its column scale, a column of the same step (any rank, also above the diagonal) takes the same-step weight,
// later steps are cut.  Factored form: the column scale and the decay are in Xw and in the epilogue's row
// factor, so the same-step entries carry rho = gamma / scale instead.
__device__ __forceinline__ void mask_block_m3(const uint32_t (&r)[32], uint32_t (&out)[16], bool factored, int c, int lane,
                                              int log2m, float ct, float same, const float* cum2, const float* dtv,
                                              uint32_t same_cols, uint32_t lower_cols) {
    if (factored) {
        // the usual case, kept short (this code is fetched on every tile): bit `col` of same_cols / lower_cols says
        // whether column `col` of the block lies in the row's own step / in an earlier step
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float f0 = (same_cols >> (2 * j)) & 1u ? same : ((lower_cols >> (2 * j)) & 1u ? 1.f : 0.f);
            const float f1 = (same_cols >> (2 * j + 1)) & 1u ? same : ((lower_cols >> (2 * j + 1)) & 1u ? 1.f : 0.f);
            out[j] = pack_bf16x2(__uint_as_float(r[2 * j]) * f0, __uint_as_float(r[2 * j + 1]) * f1);
        }
        return;
    }
    const int tr = lane >> log2m;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        float f[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = 2 * j + e, tc_ = col >> log2m;
            float w = 0.f;
            if (tc_ == tr) w = same;
            else if (tc_ < tr) w = ex2(ct - cum2[c * 32 + col]) * dtv[c * 32 + col];
            f[e] = w;
        }
        out[j] = pack_bf16x2(__uint_as_float(r[2 * j]) * f[0], __uint_as_float(r[2 * j + 1]) * f[1]);
    }
}

// Rotation of 8 pairs held in two 16-byte chunks (src/modules/misc/rope.rs:50-170).
__device__ __forceinline__ void rotate8(uint4& lo, uint4& hi, const float (&cs)[8], const float (&sn)[8], bool pairwise) {
    uint32_t* l = &lo.x;
    uint32_t* h = &hi.x;
    if (pairwise) {   // lo, hi hold 16 consecutive elements: pair j is the two halves of word j
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t& w = j < 4 ? l[j] : h[j - 4];
            const float2 f = unpack_bf16x2(w);
            w = pack_bf16x2(cs[j] * f.x - sn[j] * f.y, sn[j] * f.x + cs[j] * f.y);
        }
    } else {          // lo holds elements j0 .. j0+7 of the first half, hi the same positions of the second half
#pragma unroll
        for (int j2 = 0; j2 < 4; ++j2) {
            const float2 a = unpack_bf16x2(l[j2]), b = unpack_bf16x2(h[j2]);
            l[j2] = pack_bf16x2(cs[2 * j2] * a.x - sn[2 * j2] * b.x, cs[2 * j2 + 1] * a.y - sn[2 * j2 + 1] * b.y);
            h[j2] = pack_bf16x2(sn[2 * j2] * a.x + cs[2 * j2] * b.x, sn[2 * j2 + 1] * a.y + cs[2 * j2 + 1] * b.y);
        }
    }
}


// In-place rotation of one C + B stage (two 128-row x 128-column bf16 tiles, two 64-column panels each, 128-byte
// swizzle) by the cumulative angles of its time steps: thread t of 128 takes (step, group of 8 pairs) items, forms
// cos / sin of its 8 angles once and rotates that step's rows of both tensors.  Two warpgroups share a stage: thread
// vt of 256 (warpgroup `part`, thread t) starts at item vt.  The angles of the thread's first item (its only one at
// MIMO rank 4) arrive in `first`: the caller requests them a whole tile earlier (rotation_angles), so their latency
// hides behind that tile's work.  Out of line: one copy of the code.  Returns false when the wait for the stage's
// copy ran out of its budget.
struct Ang8 {
    float v[8];
};
__device__ __forceinline__ Ang8 rotation_angles(const float* angles, int b, int i, int h, int St, int H, int na, int log2m, int vt) {
    const int nsteps = T >> log2m, sl = vt >> 3, gq = vt & 7, step = i * nsteps + sl;
    Ang8 a;
#pragma unroll
    for (int j = 0; j < 8; ++j)
        a.v[j] = (sl < nsteps && step < St && gq * 8 + j < na) ? angles[(((int64_t)b * St + step) * H + h) * na + gq * 8 + j] : 0.f;
    return a;
}
__device__ __noinline__ bool rotate_tile(unsigned char* cstage, unsigned char* bstage, const float* angles, int b, int i, int h,
                                         int St, int H, int na, int log2m, bool pairwise, int vt, uint64_t* full_bar,
                                         uint32_t parity, Ang8 first) {
    const int m = 1 << log2m, nsteps = T >> log2m;
    auto angle_of = [&](int item, int j) {
        const int sl = item >> 3, gq = item & 7, step = i * nsteps + sl;
        return (step < St && gq * 8 + j < na) ? angles[(((int64_t)b * St + step) * H + h) * na + gq * 8 + j] : 0.f;
    };
    {
        uint32_t n = 0;
        bool ok = true;
#pragma unroll 1
        while (!mbar_try_wait(full_bar, parity))
            if (++n >= kWaitBudget) {
                ok = false;
                break;
            }
        if (!__all_sync(0xffffffffu, ok)) return false;
    }
    for (int item = vt; item < nsteps * 8; item += 256) {
        const int sl = item >> 3, gq = item & 7;
        float cs[8], sn[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // MIMO ranks below 4 have more items than threads: the angles of the later ones are fetched here
            const float a = item == vt ? first.v[j] : angle_of(item, j);
            __sincosf(wrap_angle(a), &sn[j], &cs[j]);   // angle 0 (pairs past rope_dim, rows past the end) rotates nothing
        }
        // the two 16-byte chunks of a row that hold the 8 pairs: panel byte offset and chunk index inside the panel
        const uint32_t pan_lo = pairwise ? (gq >> 2) * kPanel : 0u, pan_hi = pairwise ? pan_lo : kPanel;
        const uint32_t ch_lo = pairwise ? (2 * gq) & 7 : gq, ch_hi = pairwise ? ch_lo + 1 : gq;
        for (int r = 0; r < m; ++r) {
            const uint32_t row = sl * m + r;
            const uint32_t alo = pan_lo + sw128_offset(row, ch_lo), ahi = pan_hi + sw128_offset(row, ch_hi);
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                unsigned char* base = which ? bstage : cstage;
                uint4 lo = *reinterpret_cast<uint4*>(base + alo), hi = *reinterpret_cast<uint4*>(base + ahi);
                rotate8(lo, hi, cs, sn, pairwise);
                *reinterpret_cast<uint4*>(base + alo) = lo;
                *reinterpret_cast<uint4*>(base + ahi) = hi;
            }
        }
    }
    return true;
}

// clamp(softplus(x)) of the fused dt path (src/mamba2/mamba2.rs:692-697); out of line: rarely used
__device__ __noinline__ float dt_activation(float x, float lo, float hi) { return fminf(fmaxf(softplus_f32(x), lo), hi); }

// This CTA's tile range [lo, hi) of the global (unit-major) tile sequence, as items: an item is the part of
// one unit inside the range, tiles [i0, iend) of that unit.  Natural item j covers unit w_unit0 + j; the first
// may start inside its unit (it continues what the CTA before this one began), the last may end inside its
// unit (the next CTA continues it).  Walk order: the last item first, the first item last, the rest in
// between -- so the piece another CTA waits for is produced at once, and the piece that waits comes last.
// -> {i0, iend, batch row, head}
__device__ __noinline__ int4 item_of(const Barriers* bars, int tpu, int H, int pos) {
    const int n = bars->w_items;
    const int j = pos == 0 ? n - 1 : (pos == n - 1 ? 0 : pos);
    const int unit = bars->w_unit0 + j;
    int4 v;
    v.x = j == 0 ? bars->w_first : 0;
    v.y = j == n - 1 ? bars->w_last_end : tpu;
    v.z = unit / H;
    v.w = unit - v.z * H;
    return v;
}

struct TileWalk {
    int i, iend, b, h, pos, i0;
};

// Timeout path only (kept out of line, away from the hot code).  A wait gave up somewhere in this CTA and
// every role has left its loop.  Before TMEM goes back, each thread that issued asynchronous work waits --
// bounded again -- for what it may still have in flight: the MMA issuers through a commit onto a barrier of
// their own, the producer through the full barriers of the (at most two) stages it loaded last.
__device__ __noinline__ void drain_after_timeout(Barriers* bars, int warp, int lane, uint32_t budget) {
    const int x_issued = bars->x_issued, cb_issued = bars->cb_issued;
    if (lane == 0 && (warp == 1 || warp == 2 || warp == 4)) {
        uint64_t* db = &bars->drain[warp == 4 ? 2 : warp - 1];
        umma_commit(db);
        for (uint32_t n = 0; n < budget && !mbar_try_wait(db, 0); ++n) {}
    }
    if (warp == 0 && lane == 0) {
        for (int k = x_issued - 1; k >= 0 && k >= x_issued - 2; --k)
            for (uint32_t n = 0; n < budget && !mbar_try_wait(&bars->xld_full[k & 1], (k >> 1) & 1); ++n) {}
        for (int k = cb_issued - 1; k >= 0 && k >= cb_issued - 2; --k)
            for (uint32_t n = 0; n < budget && !mbar_try_wait(&bars->cbld_full[k & 1], (k >> 1) & 1); ++n) {}
    }
}

// kMode 0: Mamba-2.  kMode 1: the Mamba-3 cores on the fused (time x rank) axis (single-pass core with column
// scale and same-step weight, or the generic core with both equal to one).
template <int kMode>
__global__ void __launch_bounds__(kThreads, 1) ssd2_tc_kernel(const __grid_constant__ Params prm) {
    extern __shared__ unsigned char smem_raw[];
    // 1024-byte aligned base, formed as an offset on the __shared__ array so that the compiler keeps the
    // shared address space (32-bit LDS / STS) for everything derived from it
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    Barriers* bars = reinterpret_cast<Barriers*>(smem + kOffBar);
    volatile uint32_t* abort_flag = &bars->abort_flag;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->cbld_full[i], 1);
            mbar_init(&bars->cbld_empty[i], 2);   // commits of both MMA issuers
            mbar_init(&bars->xld_full[i], 1);
            mbar_init(&bars->xld_empty[i], 8);    // 4 scaling warps + 4 epilogue warps (exact tiles) or the scaling warps again
            mbar_init(&bars->xw_free[i], 1);      // S commit: the scaled tile may be overwritten by y
            mbar_init(&bars->xsrc_read[i], 4);    // epilogue warps: their rows of the skip-term source are in registers
            mbar_init(&bars->cb_full[i], 1);
            mbar_init(&bars->p_ready[i], 4);
            mbar_init(&bars->p_free[i], 1);       // Y1 commit: the P / CB accumulator may be overwritten
            mbar_init(&bars->s_full[i], 1);
            mbar_init(&bars->s_empty[i], 4);
            mbar_init(&bars->xw_ready[i], 4);
        }
        for (int i = 0; i < kCumStages; ++i) {
            mbar_init(&bars->cum_full[i], 1);
            mbar_init(&bars->cum_empty[i], 12);   // mask, state and epilogue warps
        }
        mbar_init(&bars->y1_full, 1);
        mbar_init(&bars->y1_empty, 4);
        mbar_init(&bars->h_ready, 4);
        mbar_init(&bars->h_free, 1);
        mbar_init(&bars->y2_full, 1);
        mbar_init(&bars->y2_empty, 4);
        for (int i = 0; i < 3; ++i) mbar_init(&bars->drain[i], 1);
        for (int i = 0; i < 2; ++i) mbar_init(&bars->rot_done[i], 8);   // four warps each of the mask and the epilogue warpgroup
        bars->abort_flag = 0;
        bars->x_issued = bars->cb_issued = 0;
        {
            // tiles [lo, hi) of the global tile sequence: share_q tiles per CTA, one more for the first share_r
            const int c = blockIdx.x, extra = c < prm.share_r ? c : prm.share_r;
            const int lo = c * prm.share_q + extra, hi = lo + prm.share_q + (c < prm.share_r ? 1 : 0);
            const int u0 = lo / prm.tiles_per_unit, u1 = (hi - 1) / prm.tiles_per_unit;
            bars->w_total = hi - lo;
            bars->w_items = u1 - u0 + 1;
            bars->w_unit0 = u0;
            bars->w_first = lo - u0 * prm.tiles_per_unit;
            bars->w_last_end = hi - u1 * prm.tiles_per_unit;
        }
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

    const int tpu = prm.tiles_per_unit;
    const int total = bars->w_total;
    // Mamba-3 with angles: the mask and the epilogue warpgroups rotate every C + B stage in place once it has landed
    // (half of its time steps each), and the MMA issuers wait for that instead of for the copy
    const bool rotating = kMode == 1 && prm.angles != nullptr;
    // a walker starts before its first tile: the first walk_next() loads item 0
    auto walk_next = [&](TileWalk& w) {
        if (++w.i == w.iend) {
            const int4 v = item_of(bars, tpu, prm.H, ++w.pos);
            w.i = w.i0 = v.x, w.iend = v.y, w.b = v.z, w.h = v.w;
        }
    };
#define BM_WALK(w) TileWalk w; w.pos = -1, w.i = 0, w.iend = 1, w.b = w.h = w.i0 = 0
    const int hpg = prm.H / prm.G;
    const uint32_t c_base = smem_u32(smem + kOffC), b_base = smem_u32(smem + kOffB);
    const uint32_t x_base = smem_u32(smem + kOffX), xw_base = smem_u32(smem + kOffXw), h_base = smem_u32(smem + kOffH);

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&prm.tm_x);
            tma_prefetch_desc(&prm.tm_b);
            tma_prefetch_desc(&prm.tm_c);
            tma_prefetch_desc(&prm.tm_y);
            BM_WALK(tw);
            for (int it = 0; it < (prm.stall_loads ? 0 : total); ++it) {
                walk_next(tw);
                const int b = tw.b, h = tw.h, g = h / hpg;
                const int st = it & 1, s0 = tw.i * T;
                // X stage first: it is released early (by the scaling pass of the tile two back; on exact
                // tiles by Y1 as well) and must not queue behind the wait for the C + B stage
                BM_WAIT(&bars->xld_empty[st], ((it >> 1) & 1) ^ 1);
                BM_TRACE(0, it, 1);
                mbar_expect_tx(&bars->xld_full[st], kLoadBytesX);
                tma_load_4d(smem + kOffX + st * kPanel, &prm.tm_x, &bars->xld_full[st], 0, h, s0, b);
                bars->x_issued = it + 1;
                // C + B stage: released once CB, Y2 and S of the tile two back have completed
                BM_WAIT(&bars->cbld_empty[st], ((it >> 1) & 1) ^ 1);
                BM_TRACE(0, it, 0);
                mbar_expect_tx(&bars->cbld_full[st], kLoadBytesCB);
                unsigned char* cs = smem + kOffC + st * 2 * kPanel;
                unsigned char* bs = smem + kOffB + st * 2 * kPanel;
                tma_load_4d(cs, &prm.tm_c, &bars->cbld_full[st], 0, g, s0, b);
                tma_load_4d(cs + kPanel, &prm.tm_c, &bars->cbld_full[st], 64, g, s0, b);
                tma_load_4d(bs, &prm.tm_b, &bars->cbld_full[st], 0, g, s0, b);
                tma_load_4d(bs + kPanel, &prm.tm_b, &bars->cbld_full[st], 64, g, s0, b);
                bars->cb_issued = it + 1;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer, scan chain
        // CB(it) = C B^T as soon as the C + B stage of tile it has landed and Y1(it-2) has finished reading
        // P from the accumulator CB(it) overwrites.  (Y1 itself is issued by the mask warpgroup, right
        // where P becomes complete, so that it never queues behind a wait for a TMA stage.)
        if (lane == 0) {
            const uint32_t id_cb = umma_idesc_bf16(128, 128, false, false);
            for (int it = 0; it < total; ++it) {
                const int st = it & 1;
                BM_WAIT(rotating ? &bars->rot_done[st] : &bars->cbld_full[st], (it >> 1) & 1);
                BM_WAIT(&bars->p_free[st], ((it >> 1) & 1) ^ 1);
                BM_TRACE(1, it, 0);
                tc_fence_after();
                const uint32_t cs = c_base + st * 2 * kPanel, bs = b_base + st * 2 * kPanel;
                const uint64_t da = umma_desc_kmajor(cs), db = umma_desc_kmajor(bs);
#pragma unroll 1
                for (int k = 0; k < 8; ++k) {
                    const uint32_t off = (k >> 2) * kPanel + (k & 3) * 32;
                    umma_ss(tmem + kColCB + st * 128, desc_advance(da, off), desc_advance(db, off), id_cb, k > 0);
                }
                umma_commit(&bars->cb_full[st]);
                umma_commit(&bars->cbld_empty[st]);
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------------ MMA issuer, state chain
        // Per step: Y2(it) = C h^T, then S(it+1) = B^T Xw (one tile ahead, double-buffered accumulator): the
        // order in which their inputs are produced.
        if (lane == 0) {
            const uint32_t id_kmn = umma_idesc_bf16(128, 64, false, true);
            const uint32_t id_mnmn = umma_idesc_bf16(128, 64, true, true);
            const uint64_t dh = umma_desc_mnmajor(h_base, kPanel);
            for (int it = -1; it < total; ++it) {
                if (it >= 0) {
                    // Y2(it) = C h^T once the state entering the tile is published; last reader of the C + B
                    // stage (S(it) was issued in the previous step)
                    const int st = it & 1;
                    const uint32_t cs = c_base + st * 2 * kPanel;
                    BM_WAIT(&bars->h_ready, it & 1);
                    BM_WAIT(&bars->y2_empty, (it & 1) ^ 1);
                    BM_TRACE(2, it, 0);
                    tc_fence_after();
                    const uint64_t dc = umma_desc_kmajor(cs);
#pragma unroll 1
                    for (int k = 0; k < 8; ++k) {
                        const uint32_t off = (k >> 2) * kPanel + (k & 3) * 32;
                        umma_ss(tmem + kColY2, desc_advance(dc, off), desc_advance(dh, k * 2048), id_kmn, k > 0);
                    }
                    umma_commit(&bars->y2_full);
                    umma_commit(&bars->h_free);
                    umma_commit(&bars->cbld_empty[st]);
                }
                if (it + 1 < total) {
                    // S(it+1) = B^T Xw: independent of the state, so it runs one tile ahead into the other
                    // of its two accumulators while the state update of tile it is still reading its own
                    const int nx = it + 1, st = nx & 1;
                    const uint32_t bs = b_base + st * 2 * kPanel, xw = xw_base + st * kPanel;
                    BM_WAIT(rotating ? &bars->rot_done[st] : &bars->cbld_full[st], (nx >> 1) & 1);
                    BM_WAIT(&bars->xw_ready[st], (nx >> 1) & 1);
                    BM_WAIT(&bars->s_empty[st], ((nx >> 1) & 1) ^ 1);
                    BM_TRACE(2, nx, 1);
                    tc_fence_after();
                    const uint64_t dbm = umma_desc_mnmajor(bs, kPanel), dxw = umma_desc_mnmajor(xw, kPanel);
#pragma unroll 1
                    for (int k = 0; k < 8; ++k)
                        umma_ss(tmem + kColS + st * 64, desc_advance(dbm, k * 2048), desc_advance(dxw, k * 2048), id_mnmn, k > 0);
                    umma_commit(&bars->s_full[st]);
                    umma_commit(&bars->xw_free[st]);
                }
            }
        }
    } else if (warp == 3) {
        // ------------------------------------------------------------------ decay scan of dt
        // log2-domain cumulative sum of dt*A over the tile, plus the derived per-token factors.
        const float log2e = 1.4426950408889634f;
        // A lane owns four consecutive tokens: a serial sum over its four steps, one warp scan over the lane
        // totals, and the per-token factors follow.  The dt values of a tile are fetched one tile ahead
        // (four loads per lane, issued together), so the global-memory latency is hidden behind the tile before.
        BM_WALK(twn);
        TileWalk tw;
        float nv[4], nda[4];
        auto fetch = [&](const TileWalk& w) {
            const int left = prm.S - w.i * T;
            if (kMode == 0) {
                const float* row = prm.dt + ((int64_t)w.b * prm.S + w.i * T) * prm.H + w.h;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int t = lane * 4 + k;
                    nv[k] = t < left ? row[(int64_t)t * prm.H] : 0.f;
                }
            } else {
                // fused row -> time step; the step's decay enters at its first rank, so that every rank of a
                // step sees the cumulative decay including that step
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int rrow = w.i * T + lane * 4 + k;
                    const int64_t o = ((int64_t)w.b * prm.St + (rrow >> prm.log2m)) * prm.H + w.h;
                    const bool live = lane * 4 + k < left;
                    nv[k] = live ? (prm.dt ? prm.dt[o] : 1.f) : 0.f;
                    nda[k] = (live && (rrow & ((1 << prm.log2m) - 1)) == 0) ? prm.da[o] : 0.f;
                }
            }
        };
        for (int it = -1; it < total; ++it) {
            // the pass before the first tile (it = -1) only fetches that tile's steps
            tw = twn;
            const int cst = (it & (kCumStages - 1));
            float* cum2 = reinterpret_cast<float*>(smem + kOffCum + cst * kCumStageBytes);
            float *dtv = cum2 + kCumDt, *wv = cum2 + kCumW, *colf = cum2 + kCumColf;
            const int left = prm.S - tw.i * T;      // tokens of the sequence from the start of this tile on
            float d4[4], c4[4];
            float run = 0.f;
            bool zero = false;
            if (it >= 0) {
                const float ah = kMode == 0 ? prm.a[tw.h] * log2e : log2e;
                const float bias = (kMode == 0 && prm.dt_bias) ? prm.dt_bias[tw.h] : 0.f;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float v = nv[k];
                    const bool live = lane * 4 + k < left;
                    if (kMode == 0) {
                        if (prm.dt_bias && live) v = dt_activation(v + bias, prm.dt_min, prm.dt_max);
                        zero |= live && !(v > 0.f);
                        run = fmaf(v, ah, run);
                    } else {
                        run = fmaf(nda[k], ah, run);
                    }
                    d4[k] = v;
                    c4[k] = run;
                }
            }
            if (it + 1 < total) {
                walk_next(twn);
                fetch(twn);
            }
            if (it < 0) continue;
            float incl = run;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            const float excl = incl - run;
            const float cend_tile = __shfl_sync(0xffffffffu, incl, 31);
            // end-of-32-block cumulative value: lane 8*blk+7 holds it as its inclusive total
            const float cend_blk = __shfl_sync(0xffffffffu, incl, (lane & ~7) | 7);
            const bool any_zero = __any_sync(0xffffffffu, zero);
            BM_WAIT_WARP(&bars->cum_empty[cst], ((it >> 2) & 1) ^ 1);
            bool weak = false;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int t = lane * 4 + k;
                const float c = excl + c4[k];
                const float w = d4[k] * ex2(cend_tile - c);
                cum2[t] = c;
                dtv[t] = d4[k];
                wv[t] = w;
                colf[t] = d4[k] * ex2(cend_blk - c);
                if (kMode == 0) weak |= (t < left) && !(w >= kFactoredMinRowWeight);
            }
            // the factored form divides by the row weight w_t (the D x term): a tile with a live row whose
            // weight is zero, denormal or merely tiny takes the exact form
            const bool any_weak = __any_sync(0xffffffffu, weak) || any_zero;
            if (lane == 0) cum2[kCumFlag] = (fabsf(cend_tile) <= kFactoredMaxLog2Decay && !any_weak) ? 1.f : 0.f;
            __syncwarp();
            BM_TRACE(3, it, 0);
            if (lane == 0) mbar_arrive(&bars->cum_full[cst]);
        }
    } else if (warp < 8) {
        // ------------------------------------------------------------------ mask pass: CB -> P
        const int q = warp & 3, t = q * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
        // bf16-pair masks of the diagonal block: column 32q + j is kept for row 32q + lane when j <= lane
        uint32_t causal[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            causal[j] = (2 * j <= lane ? 0x0000ffffu : 0u) | (2 * j + 1 <= lane ? 0xffff0000u : 0u);
            asm volatile("" : "+r"(causal[j]));   // keep the masks in registers instead of recomputing them per tile
        }
        BM_WALK(tw);
        // Mamba-3, diagonal block: columns of the row's own step and of earlier steps, as bit masks (lane-constant)
        uint32_t same_cols = 0u, lower_cols = 0u;
        if (kMode == 1) {
            const int m_ = 1 << prm.log2m, first = (lane >> prm.log2m) << prm.log2m;   // first column of the row's step
            same_cols = (m_ >= 32 ? 0xffffffffu : ((1u << m_) - 1u)) << first;
            lower_cols = first == 0 ? 0u : (0xffffffffu >> (32 - first));
        }
        // Mamba-3: the row's same-step weight gamma is fetched one tile ahead (at the end of the pass before), so
        // that its global-memory latency is hidden behind the wait for the next C B^T
        float gam_next = 0.f;
        // moves the walker to the next tile, requests its gamma and (rotating) does this warpgroup's half of the
        // rotation of its C + B stage
        Ang8 ang_next;
        auto prefetch_tile = [&]() {   // the walker moves to the next tile; its gamma and rotation angles are requested
            walk_next(tw);
            if (prm.gamma != nullptr) {
                const int rrow = tw.i * T + t;
                gam_next = rrow < prm.S ? prm.gamma[((int64_t)tw.b * prm.St + (rrow >> prm.log2m)) * prm.H + tw.h] : 0.f;
            }
            if (rotating) ang_next = rotation_angles(prm.angles, tw.b, tw.i, tw.h, prm.St, prm.H, prm.rope_pairs, prm.log2m, t);
        };
        auto rotate_next = [&](int n) {   // this warpgroup's half of the rotation of tile n's stage (the walker is on it)
            if (!rotating) return true;
            const int rst = n & 1;
            const bool ok = rotate_tile(smem + kOffC + rst * 2 * kPanel, smem + kOffB + rst * 2 * kPanel, prm.angles, tw.b, tw.i, tw.h,
                                        prm.St, prm.H, prm.rope_pairs, prm.log2m, prm.pairwise != 0, t, &bars->cbld_full[rst],
                                        (n >> 1) & 1, ang_next);
            fence_proxy_async_smem();
            __syncwarp();
            if (ok && lane == 0) mbar_arrive(&bars->rot_done[rst]);
            return ok;
        };
        if (kMode == 1 && total > 0) {
            prefetch_tile();
            if (!rotate_next(0)) goto timed_out;
        }
        for (int it = 0; it < total; ++it) {
            const float gam = gam_next;
            // Mamba-3: what the next tile needs from global memory is requested now, a whole tile ahead of its use
            if (kMode == 1 && it + 1 < total) prefetch_tile();
            const int st = it & 1, cst = (it & (kCumStages - 1));
            const float* cum2 = reinterpret_cast<const float*>(smem + kOffCum + cst * kCumStageBytes);
            const float *dtv = cum2 + kCumDt, *colf = cum2 + kCumColf;
            BM_TRACE(4, it, 0);
            BM_WAIT_WARP2(&bars->cum_full[cst], (it >> 2) & 1, &bars->cb_full[st], (it >> 1) & 1);
            BM_TRACE(4, it, 1);
            tc_fence_after();
            const float ct = cum2[t];
            const bool factored = cum2[kCumFlag] != 0.f;
            const uint32_t cb = lane_addr + kColCB + st * 128;
            float same = 1.f;   // Mamba-3: weight of the same-step block for this row
            if (kMode == 1 && prm.gamma != nullptr) {
                const float sc = dtv[t];
                same = factored ? (sc > 0.f ? gam / sc : 0.f) : gam;
            }
            // blocks 0..q carry data (block q holds the diagonal), blocks above are zero
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t out[16];
                if (c <= q) {
                    uint32_t r[32];
                    tmem_ld32(cb + c * 32, r);
                    tmem_wait_ld();
                    if (kMode == 1 && c == q) mask_block_m3(r, out, factored, c, lane, prm.log2m, ct, same, cum2, dtv, same_cols, lower_cols);
                    else mask_block(r, out, factored, kMode == 0 && c == q, c, ct, cum2, dtv, colf, causal);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) out[j] = 0u;
                }
                tmem_st16(cb + c * 16, out);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            BM_TRACE(4, it, 3);
            if (lane == 0) {
                mbar_arrive(&bars->p_ready[st]);
                mbar_arrive(&bars->cum_empty[cst]);
            }
            if (q == 0) {
                // The warp with the least mask work (one block) also issues Y1(it) = P X: it waits, as a
                // whole, for the other three warps' parts of P, for the B operand and for the epilogue to
                // have drained Y1(it-1); then one lane issues.  Factored tiles multiply by the scaled tile
                // Xw, exact tiles by X itself.
                BM_WAIT_WARP3(&bars->p_ready[st], (it >> 1) & 1, &bars->xw_ready[st], (it >> 1) & 1,
                              &bars->y1_empty, (it & 1) ^ 1);
                BM_TRACE(1, it, 1);
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t xs = factored ? xw_base + st * kPanel : x_base + st * kPanel;
                    const uint64_t dx = umma_desc_mnmajor(xs, kPanel);
                    const uint32_t pa = tmem + kColCB + st * 128;
                    const uint32_t id_kmn = umma_idesc_bf16(128, 64, false, true);
#pragma unroll 1
                    for (int k = 0; k < 8; ++k)
                        umma_ts(tmem + kColY1, pa + k * 8, desc_advance(dx, k * 2048), id_kmn, k > 0);
                    umma_commit(&bars->y1_full);
                    umma_commit(&bars->p_free[st]);
                }
                __syncwarp();
            }
            // Mamba-3: on to the next tile (its gamma, this warpgroup's half of its rotation) after Y1 has been issued
            if (kMode == 1 && it + 1 < total && !rotate_next(it + 1)) goto timed_out;
        }
    } else if (warp < 12) {
        // ------------------------------------------------------------------ X scaling and state update
        const int q = warp & 3, t = q * 32 + lane;  // t doubles as the state row r
        const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
        unsigned char* hs = smem + kOffH;
        float hst[P];
        auto scale_x = [&](int it) {
            // Xw = X * dt * exp(cum_end - cum) for tile `it` (rows keep their swizzled positions)
            const int st = it & 1, cst = (it & (kCumStages - 1));
            const float* wv = reinterpret_cast<const float*>(smem + kOffCum + cst * kCumStageBytes) + kCumW;
            const unsigned char* xs = smem + kOffX + st * kPanel;
            unsigned char* xw = smem + kOffXw + st * kPanel;
            const float w = wv[t];
            // two batches of four 16-byte chunks: the four loads of a batch are in flight together
#pragma unroll 1
            for (int kb = 0; kb < 8; kb += 4) {
                uint4 v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = *reinterpret_cast<const uint4*>(xs + sw128_offset(t, kb + j));
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f0 = unpack_bf16x2(v[j].x), f1 = unpack_bf16x2(v[j].y), f2 = unpack_bf16x2(v[j].z),
                                 f3 = unpack_bf16x2(v[j].w);
                    uint4 o;
                    o.x = pack_bf16x2(f0.x * w, f0.y * w);
                    o.y = pack_bf16x2(f1.x * w, f1.y * w);
                    o.z = pack_bf16x2(f2.x * w, f2.y * w);
                    o.w = pack_bf16x2(f3.x * w, f3.y * w);
                    *reinterpret_cast<uint4*>(xw + sw128_offset(t, kb + j)) = o;
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bars->xw_ready[st]);
                mbar_arrive(&bars->xld_empty[st]);
                // factored tiles: nothing reads X after this pass, so each warp also makes the arrival that
                // the epilogue warp of the same rows makes on exact tiles (where Y1 and D x still read X)
                if (wv[kCumFlag - kCumW] != 0.f) mbar_arrive(&bars->xld_empty[st]);
            }
        };
        auto publish_state = [&]() {
            // bf16 copy of the state as the MN-major B operand of the readout GEMM
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                uint4 v;
                v.x = pack_bf16x2(hst[8 * k], hst[8 * k + 1]);
                v.y = pack_bf16x2(hst[8 * k + 2], hst[8 * k + 3]);
                v.z = pack_bf16x2(hst[8 * k + 4], hst[8 * k + 5]);
                v.w = pack_bf16x2(hst[8 * k + 6], hst[8 * k + 7]);
                *reinterpret_cast<uint4*>(hs + sw128_offset(t, k)) = v;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->h_ready);
        };
        // Iteration `it` scales the X tile of tile it+1 (so that S(it+1) can run while this warpgroup is
        // still busy with tile it), folds S(it) into the state and publishes the result as the readout
        // operand of tile it+1.
        // At the first tile of a unit the initial state is loaded and published instead.
        BM_WALK(tw);
        for (int it = -1; it < total; ++it) {
            if (it != 0) walk_next(tw);
            const int itc = it < 0 ? 0 : it;
            const int i = tw.i, b = tw.b, h = tw.h;
            const int cst = (itc & (kCumStages - 1));
            const float* cumv = reinterpret_cast<const float*>(smem + kOffCum + cst * kCumStageBytes);
            const int64_t state_base = ((int64_t)b * prm.H + h) * P * R;
            if (it >= 0) {
                if (__builtin_expect(i == tw.i0, 0)) {
                    // item start: the state entering it -> registers, published as the operand of this tile's
                    // readout (the operand tile is free once Y2(it-1) has completed).  At the start of a unit
                    // that is the caller's initial state; inside a unit, what the CTA before this one stored
                    // when its piece of the unit ended.
                    const float* src = prm.h0 ? prm.h0 + state_base : nullptr;
                    if (i != 0) {
                        const int* flag = prm.handoff_flags + (blockIdx.x - 1);
                        uint32_t n_ = 0;
                        bool ok_ = true;
#pragma unroll 1
                        while (ld_acquire_gpu(flag) < 4)
                            if (++n_ >= kWaitBudget) {
                                ok_ = false;
                                break;
                            }
                        if (!__all_sync(0xffffffffu, ok_)) goto timed_out;
                        src = prm.handoff + (int64_t)(blockIdx.x - 1) * P * R;
                    }
#pragma unroll
                    for (int p = 0; p < P; ++p) hst[p] = src ? src[(int64_t)p * R + t] : 0.f;
                    if (it > 0) BM_WAIT_WARP(&bars->h_free, (it - 1) & 1);
                    publish_state();
                    BM_TRACE(5, it, 3);
                }
                if (__builtin_expect(prm.chunk_states != nullptr, 0) && (i * T) % prm.Q == 0) {
                    const int n = (i * T) / prm.Q;
                    float* cs = prm.chunk_states + (((int64_t)b * prm.NC + n) * prm.H + h) * P * R;
#pragma unroll
                    for (int p = 0; p < P; ++p) cs[(int64_t)p * R + t] = hst[p];
                }
            }
            if (it + 1 < total) {
                BM_WAIT_WARP2(&bars->xld_full[(it + 1) & 1], ((it + 1) >> 1) & 1,
                              &bars->cum_full[((it + 1) & (kCumStages - 1))], ((it + 1) >> 2) & 1);
                // the scaled tile of this parity still serves tile it-1: S(it-1) (seen complete through s_full
                // in the previous iteration), Y1(it-1) on factored tiles, and the epilogue's skip-term rows
                BM_WAIT_WARP2(&bars->p_free[(it + 1) & 1], (((it + 1) >> 1) & 1) ^ 1,
                              &bars->xsrc_read[(it + 1) & 1], (((it + 1) >> 1) & 1) ^ 1);
                BM_TRACE(5, itc, 0);
                scale_x(it + 1);
                BM_TRACE(3, itc, 1);
            }
            if (it >= 0) {
                // state update h <- exp(cum_end) h + S(it)
                BM_WAIT_WARP(&bars->s_full[it & 1], (it >> 1) & 1);
                BM_TRACE(5, it, 1);
                tc_fence_after();
                const float decay = ex2(cumv[T - 1]);
                const uint64_t decay2 = pair_f32(decay, decay);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t sv[16];
                    tmem_ld16(lane_addr + kColS + (it & 1) * 64 + c * 16, sv);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; j += 2) {
                        const uint64_t r = fma2(decay2, pair_f32(hst[c * 16 + j], hst[c * 16 + j + 1]), pair_u32(sv[j], sv[j + 1]));
                        asm("mov.b64 {%0, %1}, %2;" : "=f"(hst[c * 16 + j]), "=f"(hst[c * 16 + j + 1]) : "l"(r));
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&bars->s_empty[it & 1]);
                    mbar_arrive(&bars->cum_empty[cst]);
                }
                // unless the item ends here, the updated state is the readout operand of the next tile;
                // the operand tile is free once Y2(it) has completed
                if (__builtin_expect(i + 1 < tw.iend, 1)) {
                    BM_WAIT_WARP(&bars->h_free, it & 1);
                    publish_state();
                }
                BM_TRACE(5, it, 2);
                if (__builtin_expect(i + 1 == tw.iend, 0)) {
                    // end of the unit: the final state; end of this CTA's piece of it: the hand-over
                    const bool whole = tw.iend == tpu;
                    float* dst = whole ? prm.h_final + state_base : prm.handoff + (int64_t)blockIdx.x * P * R;
#pragma unroll
                    for (int p = 0; p < P; ++p) dst[(int64_t)p * R + t] = hst[p];
                    if (!whole) {
                        __threadfence();
                        __syncwarp();
                        if (lane == 0) atomicAdd(prm.handoff_flags + blockIdx.x, 1);
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        // y = E' Y1 + exp(cum_t) Y2 + D x, written in two column halves through a small staging tile of
        // the warp's own (32 rows x 64 bytes, 64-byte swizzle) with one TMA store each; the store of one
        // half drains while the next half is computed.
        const int q = warp & 3, t = q * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
        unsigned char* stage = smem + kOffStage + q * kStageWarpBytes;
        const uint32_t srow = lane * 64, sxor = (lane >> 1) & 3;   // 64-byte swizzle: chunk ^ ((row >> 1) & 3)
        BM_WALK(tw);
        TileWalk twn = tw;   // rotating: one tile ahead of tw
        // waits for the copy of tile n's C + B stage, rotates it in place and releases it to the MMA issuers
        Ang8 ang_next;
        auto rotate_stage = [&](int n, const TileWalk& w) {
            const int rst = n & 1;
            const bool ok = rotate_tile(smem + kOffC + rst * 2 * kPanel, smem + kOffB + rst * 2 * kPanel, prm.angles, w.b, w.i, w.h,
                                        prm.St, prm.H, prm.rope_pairs, prm.log2m, prm.pairwise != 0, 128 + t, &bars->cbld_full[rst],
                                        (n >> 1) & 1, ang_next);
            fence_proxy_async_smem();
            __syncwarp();
            if (ok && lane == 0) mbar_arrive(&bars->rot_done[rst]);
            return ok;
        };
        if (rotating && total > 0) {
            walk_next(twn);
            ang_next = rotation_angles(prm.angles, twn.b, twn.i, twn.h, prm.St, prm.H, prm.rope_pairs, prm.log2m, 128 + t);
            if (!rotate_stage(0, twn)) goto timed_out;
        }
        for (int it = 0; it < total; ++it) {
            if (rotating) {
                tw = twn;
                if (it + 1 < total) {   // the next tile's angles, a whole tile ahead of their use
                    walk_next(twn);
                    ang_next = rotation_angles(prm.angles, twn.b, twn.i, twn.h, prm.St, prm.H, prm.rope_pairs, prm.log2m, 128 + t);
                }
            } else {
                walk_next(tw);
            }
            const int i = tw.i, b = tw.b, h = tw.h;
            const int st = it & 1, cst = (it & (kCumStages - 1));
            const float* cum2 = reinterpret_cast<const float*>(smem + kOffCum + cst * kCumStageBytes);
            BM_WAIT_WARP(&bars->cum_full[cst], (it >> 2) & 1);
            const float e = ex2(cum2[t]);
            // row factor of the factored mask: exp2(cum_t - cend); 1 for exact tiles
            const bool factored = cum2[kCumFlag] != 0.f;
            const float e1 = factored ? ex2(cum2[t] - cum2[T - 1]) : 1.f;
            // skip term D x: factored tiles recover x from the scaled tile (x w = Xw, w > 0 on these tiles),
            // exact tiles read the X tile, which they hold until Y1 has completed and this row is read
            const float wt = cum2[kCumW + t];
            const float dsk = prm.d ? prm.d[h] : 0.f;
            const float dxw = factored ? (wt > 0.f ? dsk / wt : 0.f) : dsk;   // wt = 0 only on padding rows
            const unsigned char* xsrc = smem + (factored ? kOffXw : kOffX) + st * kPanel;
            const uint64_t ee = pair_f32(e, e), ee1 = pair_f32(e1, e1);
            const uint32_t dd = pack_bf16x2(dxw, dxw);
            // the source row is fetched before the accumulators are waited for (the tile has been in place
            // since the scaling pass), so the scaled tile can be handed back for tile it+2 early
            BM_WAIT_WARP(&bars->xw_ready[st], (it >> 1) & 1);
            uint4 xrow[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                xrow[k] = *reinterpret_cast<const uint4*>(xsrc + sw128_offset(t, k));
                asm volatile("" ::"r"(xrow[k].x), "r"(xrow[k].y), "r"(xrow[k].z), "r"(xrow[k].w));   // loads have landed
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->xsrc_read[st]);
            if (rotating && it + 1 < total) {   // the next tile's stage, while this tile's MMAs are still running
                if (!rotate_stage(it + 1, twn)) goto timed_out;
            }
            BM_WAIT_WARP2(&bars->y2_full, it & 1, &bars->y1_full, it & 1);
            if (!factored && lane == 0) mbar_arrive(&bars->xld_empty[st]);   // exact tiles: Y1 and this warp are done with X
            BM_TRACE(6, it, 0);
            tc_fence_after();
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t y1[32], y2[32];
                tmem_ld32(lane_addr + kColY1 + half * 32, y1);
                tmem_ld32(lane_addr + kColY2 + half * 32, y2);
                tmem_wait_ld();
                if (half == 1) {
                    // both accumulators are in registers: release them to the MMA issuers
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&bars->y1_empty);
                        mbar_arrive(&bars->y2_empty);
                    }
                }
                uint4 o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int j = k * 8;
                    const uint4 xv = xrow[half * 4 + k];
                    const uint32_t xw4[4] = {xv.x, xv.y, xv.z, xv.w};
                    uint32_t o4[4];
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        uint64_t acc = mul2(ee1, pair_u32(y1[j + 2 * m], y1[j + 2 * m + 1]));
                        acc = fma2(ee, pair_u32(y2[j + 2 * m], y2[j + 2 * m + 1]), acc);
                        // + (D / w_t) * Xw as one packed bf16 fma on the rounded result
                        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(o4[m]) : "r"(xw4[m]), "r"(dd), "r"(pack_bf16x2_pair(acc)));
                    }
                    o[k] = make_uint4(o4[0], o4[1], o4[2], o4[3]);
                }
                // the previous store of this warp must have drained the staging tile
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
#pragma unroll
                for (int k = 0; k < 4; ++k) *reinterpret_cast<uint4*>(stage + srow + ((k ^ sxor) << 4)) = o[k];
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_4d(&prm.tm_y, stage, half * 32, h, i * T + q * 32, b);
                    tma_store_commit();
                }
            }
            BM_TRACE(6, it, 1);
            if (lane == 0) mbar_arrive(&bars->cum_empty[cst]);
            __syncwarp();
            BM_TRACE(6, it, 2);
        }
    }
    goto done;
timed_out:
    atomicExch(prm.status, (int)BM_ERR_TIMEOUT);
    *abort_flag = 1;
done:
    if (warp >= 12 && lane == 0) tma_store_wait_all<0>();
    tc_fence_before();
    __syncthreads();
    if (*abort_flag != 0u) {
        drain_after_timeout(bars, warp, lane, kWaitBudget);
        tc_fence_before();
        __syncthreads();
    }
    if (warp == 2) tmem_dealloc(tmem, 512);
}

int num_sms() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

}  // namespace

const char* ssd2_why_not(const bm_ssd2_fwd_args* a) {
    if (a->dtype != BM_DTYPE_BF16) return "activations must be bf16";
    if (a->headdim != P) return "headdim must be 64";
    if (a->state_rank != R) return "state_rank must be 128";
    if (a->z != nullptr) return "fused z gate is only on the exact path";
    if (a->chunk_states != nullptr && a->chunk_len % T != 0) return "chunk_states needs chunk_len % 128 == 0";
    return nullptr;
}

bool ssd2_supported(const bm_ssd2_fwd_args* a) { return ssd2_why_not(a) == nullptr; }

// Workspace head shared by both launchers: status word and the CTAs' hand-over flags in the first kWsFlagBytes
// (reset before every launch), the trace area of development builds, then one state per CTA for hand-overs.
constexpr size_t kWsFlagBytes = 2048, kWsTraceBytes = 7 * 64 * 4 * 8;
static size_t ws_head_bytes() { return align_up(kWsFlagBytes + kWsTraceBytes, 256) + (size_t)num_sms() * P * R * sizeof(float); }
static void ws_head_pointers(void* workspace, Params& prm) {
    char* w = static_cast<char*>(workspace);
    prm.status = reinterpret_cast<int*>(w);
    prm.handoff_flags = reinterpret_cast<int*>(w + 64);
    prm.trace = reinterpret_cast<long long*>(w + kWsFlagBytes);
    prm.handoff = reinterpret_cast<float*>(w + align_up(kWsFlagBytes + kWsTraceBytes, 256));
}

size_t ssd2_workspace_bytes(const bm_ssd2_fwd_args*) { return ws_head_bytes(); }

int32_t ssd2_run(const bm_ssd2_fwd_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (workspace == nullptr || workspace_bytes < ssd2_workspace_bytes(a))
        return fail(BM_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", workspace_bytes,
                    ssd2_workspace_bytes(a));
    Params prm{};
    const char* err = nullptr;
    const uint64_t S = a->seqlen, H = a->nheads, G = a->ngroups, B = a->batch;
    const uint32_t box[4] = {64, 1, (uint32_t)T, 1};
    {
        const uint64_t dims[4] = {(uint64_t)P, H, S, B};
        const uint64_t strides[3] = {(uint64_t)P * 2, H * P * 2, S * H * P * 2};
        const uint32_t box_y[4] = {32, 1, 32, 1};  // one column half of one epilogue warp's rows per store
        if (!make_tensor_map_bf16(&prm.tm_x, a->x, 4, dims, strides, box, 128, &err) ||
            !make_tensor_map_bf16(&prm.tm_y, a->y, 4, dims, strides, box_y, 64, &err))
            return fail(BM_ERR_CUDA, "tensor map (x/y): %s", err);
    }
    {
        const uint64_t dims[4] = {(uint64_t)R, G, S, B};
        const uint64_t strides[3] = {(uint64_t)R * 2, G * R * 2, S * G * R * 2};
        if (!make_tensor_map_bf16(&prm.tm_b, a->b, 4, dims, strides, box, 128, &err) ||
            !make_tensor_map_bf16(&prm.tm_c, a->c, 4, dims, strides, box, 128, &err))
            return fail(BM_ERR_CUDA, "tensor map (b/c): %s", err);
    }
    prm.dt = a->dt, prm.a = a->a, prm.d = a->d, prm.h0 = a->h0, prm.dt_bias = a->dt_bias;
    prm.dt_min = a->dt_min, prm.dt_max = a->dt_max;
    prm.h_final = a->h_final, prm.chunk_states = a->chunk_states;
    ws_head_pointers(workspace, prm);
    prm.B = a->batch, prm.S = a->seqlen, prm.H = a->nheads, prm.G = a->ngroups, prm.Q = a->chunk_len;
    prm.NC = (int)cdiv(a->seqlen, a->chunk_len);
    prm.tiles_per_unit = (int)cdiv(a->seqlen, T);
    prm.num_units = a->batch * a->nheads;
    // `reserved` carries one test-only request: BM_DEBUG_STALL_LOADS makes the producer issue nothing, so
    // that a bounded wait runs out and the error path can be exercised
    prm.stall_loads = (a->reserved == BM_DEBUG_STALL_LOADS) ? 1 : 0;
    {
        cudaError_t e = cudaFuncSetAttribute(ssd2_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(ssd2_tc_kernel)");
    }
    if (int32_t e = check_cuda(cudaMemsetAsync(workspace, 0, kWsFlagBytes, stream), "cudaMemsetAsync(status)")) return e;
    const int grid = prm.num_units < num_sms() ? prm.num_units : num_sms();
    if ((int64_t)prm.num_units * prm.tiles_per_unit > INT32_MAX) return fail(BM_ERR_UNSUPPORTED, "more than 2^31 tiles");
    prm.share_q = (int)((int64_t)prm.num_units * prm.tiles_per_unit / grid);
    prm.share_r = (int)((int64_t)prm.num_units * prm.tiles_per_unit % grid);
    ssd2_tc_kernel<0><<<grid, kThreads, kSmemBytes, stream>>>(prm);
    return check_launch("ssd2_tc_kernel");
}

// ---------------------------------------------------------------------------------------------
// Mamba-3 cores on the same kernel
// ---------------------------------------------------------------------------------------------
namespace {

int log2_exact(int v) {
    int l = 0;
    while ((1 << l) < v) ++l;
    return (1 << l) == v ? l : -1;
}

}  // namespace

const char* ssd3_why_not(const bm_ssd3_fwd_args* a) {
    if (a->dtype != BM_DTYPE_BF16) return "activations must be bf16";
    if (a->headdim != P) return "headdim must be 64";
    if (a->state_rank != R) return "state_rank must be 128";
    if (log2_exact(a->mimo_rank) < 0 || a->mimo_rank > 4) return "mimo_rank must be 1, 2 or 4";
    return nullptr;
}

bool ssd3_supported(const bm_ssd3_fwd_args* a) { return ssd3_why_not(a) == nullptr; }

size_t ssd3_workspace_bytes(const bm_ssd3_fwd_args* a) {
    (void)a;
    return ws_head_bytes();
}

int32_t ssd3_run(const bm_ssd3_fwd_args* a, bool single, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                 float* chunk_states) {
    if (workspace == nullptr || workspace_bytes < ssd3_workspace_bytes(a))
        return fail(BM_ERR_WORKSPACE_TOO_SMALL, "workspace of %zu bytes given, %zu needed", workspace_bytes,
                    ssd3_workspace_bytes(a));
    const void* bsrc = a->b;
    const void* csrc = a->c;
    Params prm{};
    const char* err = nullptr;
    const uint64_t S = (uint64_t)a->seqlen * a->mimo_rank, H = a->nheads, B = a->batch;
    const uint32_t box[4] = {64, 1, (uint32_t)T, 1};
    {
        const uint64_t dims[4] = {(uint64_t)P, H, S, B};
        const uint64_t strides[3] = {(uint64_t)P * 2, H * P * 2, S * H * P * 2};
        const uint32_t box_y[4] = {32, 1, 32, 1};
        if (!make_tensor_map_bf16(&prm.tm_x, a->v, 4, dims, strides, box, 128, &err) ||
            !make_tensor_map_bf16(&prm.tm_y, a->y, 4, dims, strides, box_y, 64, &err))
            return fail(BM_ERR_CUDA, "tensor map (v/y): %s", err);
    }
    {
        const uint64_t dims[4] = {(uint64_t)R, H, S, B};   // B / C are per head: one group per head
        const uint64_t strides[3] = {(uint64_t)R * 2, H * R * 2, S * H * R * 2};
        if (!make_tensor_map_bf16(&prm.tm_b, bsrc, 4, dims, strides, box, 128, &err) ||
            !make_tensor_map_bf16(&prm.tm_c, csrc, 4, dims, strides, box, 128, &err))
            return fail(BM_ERR_CUDA, "tensor map (b/c): %s", err);
    }
    prm.dt = single ? a->scale : nullptr, prm.da = a->da, prm.gamma = single ? a->gamma : nullptr;
    prm.a = nullptr, prm.d = nullptr, prm.h0 = a->h0, prm.dt_bias = nullptr;
    prm.h_final = a->h_final, prm.chunk_states = chunk_states;
    ws_head_pointers(workspace, prm);
    prm.B = a->batch, prm.S = (int)S, prm.St = a->seqlen, prm.log2m = log2_exact(a->mimo_rank);
    // the rotation of B / C (angles given) happens inside the kernel, on the tiles in shared memory
    prm.angles = (a->angles != nullptr && a->rope_dim > 0) ? a->angles : nullptr;
    prm.rope_pairs = a->rope_dim / 2, prm.pairwise = a->mimo_rank == 1 ? 1 : 0;
    prm.H = a->nheads, prm.G = a->nheads, prm.Q = T, prm.NC = (int)cdiv((int64_t)S, T);
    prm.tiles_per_unit = (int)cdiv((int64_t)S, T);
    prm.num_units = a->batch * a->nheads;
    prm.stall_loads = 0;
    {
        cudaError_t e = cudaFuncSetAttribute(ssd2_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(ssd3 tensor kernel)");
    }
    if (int32_t e = check_cuda(cudaMemsetAsync(workspace, 0, kWsFlagBytes, stream), "cudaMemsetAsync(status)")) return e;
    const int grid = prm.num_units < num_sms() ? prm.num_units : num_sms();
    if ((int64_t)prm.num_units * prm.tiles_per_unit > INT32_MAX) return fail(BM_ERR_UNSUPPORTED, "more than 2^31 tiles");
    prm.share_q = (int)((int64_t)prm.num_units * prm.tiles_per_unit / grid);
    prm.share_r = (int)((int64_t)prm.num_units * prm.tiles_per_unit % grid);
    ssd2_tc_kernel<1><<<grid, kThreads, kSmemBytes, stream>>>(prm);
    return check_launch("ssd3 tensor kernel");
}

}  // namespace tc
}  // namespace bm
