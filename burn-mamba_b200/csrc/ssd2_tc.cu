// Tensor-core path of the Mamba-2 SSD forward (placeholder until the tcgen05 kernel lands).
#include "ssd2_tc.cuh"

namespace bm {
namespace tc {

bool ssd2_supported(const bm_ssd2_fwd_args*) { return false; }
const char* ssd2_why_not(const bm_ssd2_fwd_args*) { return "tensor-core kernel not built"; }
size_t ssd2_workspace_bytes(const bm_ssd2_fwd_args*) { return 0; }
int32_t ssd2_run(const bm_ssd2_fwd_args*, void*, size_t, cudaStream_t) {
    return fail(BM_ERR_UNSUPPORTED, "tensor-core kernel not built");
}

}  // namespace tc
}  // namespace bm
