// Small helpers shared by the attention kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace b200p {

template <typename T> __device__ __forceinline__ T from_float(float f);
template <> __device__ __forceinline__ float         from_float<float>(float f)         { return f; }
template <> __device__ __forceinline__ __half        from_float<__half>(float f)        { return __float2half_rn(f); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float f) { return __float2bfloat16_rn(f); }

__device__ __forceinline__ float to_float(float f)         { return f; }
__device__ __forceinline__ float to_float(__half f)        { return __half2float(f); }
__device__ __forceinline__ float to_float(__nv_bfloat16 f) { return __bfloat162float(f); }

// 2^x on the SFU; -inf gives +0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

} // namespace b200p
