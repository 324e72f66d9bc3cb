// Cumulative data-dependent rotation angles of Mamba-3's Complex2D rotation
// (src/mamba3/rotation/mod.rs:559-567, :653-679):
//   theta[b, s, h, j] = prev[b, h, j] + sum_{t <= s} dt[b, t, h] * range * pi * tanh(rot[b, t, j]).
// HBM-bound on the theta write.  One thread per (b, h, j) lane walks the sequence; consecutive
// threads are consecutive j, so every load of rot and store of theta is coalesced, and the loop is
// unrolled so several independent loads are in flight per thread.
#include "common.cuh"

using namespace bm;

namespace {

__global__ void angle_cumsum_kernel(bm_angle_cumsum_args a) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int A = a.nangles, H = a.nheads, S = a.seqlen;
    if (idx >= (int64_t)a.batch * H * A) return;
    const int j = idx % A, h = (idx / A) % H, b = idx / ((int64_t)A * H);
    const float scale = a.range * 3.14159265358979323846f;
    float run = a.prev ? a.prev[idx] : 0.f;
    const float* rot = a.rot + (int64_t)b * S * A + j;
    const float* dt = a.dt + (int64_t)b * S * H + h;
    float* th = a.theta + ((int64_t)b * S * H + h) * A + j;
    constexpr int U = 8;
    int s = 0;
    for (; s + U <= S; s += U) {
        float r[U], d[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            r[k] = rot[(int64_t)(s + k) * A];
            d[k] = dt[(int64_t)(s + k) * H];
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            run += d[k] * (tanhf(r[k]) * scale);
            th[(int64_t)(s + k) * H * A] = run;
        }
    }
    for (; s < S; ++s) {
        run += dt[(int64_t)s * H] * (tanhf(rot[(int64_t)s * A]) * scale);
        th[(int64_t)s * H * A] = run;
    }
    if (a.last) a.last[idx] = wrap_angle(run);
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
    int64_t total = (int64_t)a->batch * a->nheads * a->nangles;
    angle_cumsum_kernel<<<(unsigned)cdiv(total, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(*a);
    return check_launch("angle_cumsum");
}
