// Shared host/device helpers for libbm_b200: status + error text, dtype-generic loads/stores,
// the reference's elementwise numerics (softplus thresholds, SiLU, angle wrapping).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/bm_b200.h"

namespace bm {

// ---- host side ------------------------------------------------------------------------------
// Records `msg` as the calling thread's last error and returns `code`.
int32_t fail(int32_t code, const char* fmt, ...);
void clear_error();
// Converts a CUDA runtime error into BM_ERR_CUDA (recording the error string); BM_OK if none.
int32_t check_cuda(cudaError_t e, const char* what);
// Launch check: cudaGetLastError after a kernel launch.
int32_t check_launch(const char* kernel);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

#define BM_REQUIRE_PTR(p)                                                              \
    do {                                                                               \
        if ((p) == nullptr) return ::bm::fail(BM_ERR_NULL_POINTER, "%s is NULL", #p);  \
        if (!::bm::aligned16(p)) return ::bm::fail(BM_ERR_BAD_ALIGNMENT, "%s is not 16-byte aligned", #p); \
    } while (0)
#define BM_OPTIONAL_PTR(p)                                                             \
    do {                                                                               \
        if ((p) != nullptr && !::bm::aligned16(p))                                     \
            return ::bm::fail(BM_ERR_BAD_ALIGNMENT, "%s is not 16-byte aligned", #p);  \
    } while (0)
#define BM_REQUIRE(cond, code, ...)                                                    \
    do {                                                                               \
        if (!(cond)) return ::bm::fail(code, __VA_ARGS__);                             \
    } while (0)

// ---- device side ----------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// softplus with the reference's float32 threshold: identity above 18, log1p(exp(x)) below
// (src/modules/activation/softplus.rs:17-48).  dt and its bias are float32 at this boundary.
__device__ __forceinline__ float softplus_f32(float x) { return x > 18.f ? x : log1pf(expf(x)); }
// Burn's stock softplus(x, beta = 1) used by Mamba-1 (src/mamba1/mamba1.rs:394): log(1 + exp(x)),
// evaluated as max(x, 0) + log1p(exp(-|x|)) so large x does not overflow.
__device__ __forceinline__ float softplus_stock(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
// x / (1 + exp(-x)) (src/modules/activation/silu.rs:24-27)
__device__ __forceinline__ float silu_f32(float x) { return x / (1.f + expf(-x)); }
// 2^x and 1/x on the special-function unit, denormals flushed: one instruction each (the plain approximate forms
// carry range fix-ups around them, a few instructions per call, which a streaming loop pays per element).
__device__ __forceinline__ float ex2_ftz(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_ftz(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// The same gate with the hardware exponential and reciprocal (about 1e-6 relative): for the streaming kernels
// that evaluate it once per element of a large activation tensor, where the exact division is most of the work.
// The denominator is at least 1, so the reciprocal needs no range handling; far out on the negative side the
// result is flushed to zero where the exact value is below 1e-36.
__device__ __forceinline__ float silu_fast(float x) { return x * rcp_ftz(1.f + ex2_ftz(x * -1.4426950408889634f)); }
// theta - round(theta / 2pi) * 2pi (src/modules/misc/rope.rs:23-27)
__device__ __forceinline__ float wrap_angle(float t) {
    const float two_pi = 6.28318530717958647692f;
    return t - rintf(t * (1.0f / two_pi)) * two_pi;
}

}  // namespace bm
