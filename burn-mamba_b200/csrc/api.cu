// Version, build string and the per-thread error message of libbm_b200.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace bm {

static thread_local char g_err[512] = {0};

int32_t fail(int32_t code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

void clear_error() { g_err[0] = 0; }

int32_t check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return BM_OK;
    return fail(BM_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

int32_t check_launch(const char* kernel) { return check_cuda(cudaGetLastError(), kernel); }

}  // namespace bm

extern "C" {

int32_t bm_version(void) { return (0 << 16) | 1; }

const char* bm_build_info(void) { return "libbm_b200 sm_100a (" __DATE__ ")"; }

const char* bm_last_error_string(void) { return bm::g_err; }

}  // extern "C"
