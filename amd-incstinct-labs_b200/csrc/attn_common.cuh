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

// max of three (one FMNMX3 on sm_100a)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// (2^(a*scale + bias), 2^(b*scale + bias)): the scaling is ONE packed fp32x2 FMA, the exponentials are SFU ops.
__device__ __forceinline__ float2 exp2_pair(float a, float b, float scale, float bias) {
    unsigned long long x, sc, bi, r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(a), "f"(b));
    asm("mov.b64 %0, {%1, %1};" : "=l"(sc) : "f"(scale));
    asm("mov.b64 %0, {%1, %1};" : "=l"(bi) : "f"(bias));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(x), "l"(sc), "l"(bi));
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(r));
    return make_float2(fast_exp2(lo), fast_exp2(hi));
}

} // namespace b200p
