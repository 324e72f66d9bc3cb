// Host helpers of the tensor-core path: tensor-map encoding through the driver entry point (the
// library does not link libcuda; the symbol is resolved at run time from the loaded driver).
#include "tc_common.cuh"

#include <mutex>

namespace bm {
namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

static bool make_tensor_map(CUtensorMap* out, CUtensorMapDataType dtype, const void* base, int rank, const uint64_t* dims,
                            const uint64_t* strides, const uint32_t* box, int swizzle_bytes, const char** err);

bool make_tensor_map_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                          const uint32_t* box, int swizzle_bytes, const char** err) {
    return make_tensor_map(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, rank, dims, strides, box, swizzle_bytes, err);
}

bool make_tensor_map_f32(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                         const uint32_t* box, int swizzle_bytes, const char** err) {
    return make_tensor_map(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, rank, dims, strides, box, swizzle_bytes, err);
}

static bool make_tensor_map(CUtensorMap* out, CUtensorMapDataType dtype, const void* base, int rank, const uint64_t* dims,
                            const uint64_t* strides, const uint32_t* box, int swizzle_bytes, const char** err) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) {
        *err = "cuTensorMapEncodeTiled not available from the driver";
        return false;
    }
    cuuint64_t d[5], s[5];
    cuuint32_t b[5], e[5];
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        e[i] = 1;
        if (i + 1 < rank) s[i] = strides[i];
    }
    CUresult r = fn(out, dtype, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, e,
                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                    : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                          : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        *err = "cuTensorMapEncodeTiled failed";
        return false;
    }
    return true;
}

}  // namespace tc
}  // namespace bm
