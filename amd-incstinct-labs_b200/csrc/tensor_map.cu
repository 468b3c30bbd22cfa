#include "tensor_map.cuh"
#include <mutex>

namespace b200p {
namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::once_flag g_once;

void resolve() {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
        g_encode = reinterpret_cast<EncodeFn>(fn);
    else
        cudaGetLastError();
}
} // namespace

cudaError_t make_tensor_map(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base,
                            const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                            Swizzle swizzle, bool l2_promote_256) {
    std::call_once(g_once, resolve);
    if (!g_encode) return cudaErrorNotSupported;
    cuuint64_t d[5]; cuuint64_t s[4]; cuuint32_t b[5]; cuuint32_t es[5];
    for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; es[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
    CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
    switch (swizzle) {
        case Swizzle::B32:  sw = CU_TENSOR_MAP_SWIZZLE_32B; break;
        case Swizzle::B64:  sw = CU_TENSOR_MAP_SWIZZLE_64B; break;
        case Swizzle::B128: sw = CU_TENSOR_MAP_SWIZZLE_128B; break;
        default: break;
    }
    const CUresult r = g_encode(out, dtype, cuuint32_t(rank), const_cast<void*>(base), d, s, b, es,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                l2_promote_256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

} // namespace b200p
