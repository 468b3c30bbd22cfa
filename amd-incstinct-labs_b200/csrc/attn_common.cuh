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

// The same pair WITHOUT the SFU: Cody-Waite range reduction and a cubic on the FMA pipes.
//   x = max(a*scale + bias, -126);  t = x + 1.5*2^23 (rounds x to an integer n in the low mantissa bits);
//   f = x - n in [-0.5, 0.5];  2^f ~ c0 + f(c1 + f(c2 + f c3)) (max relative error 7.5e-5, below the
//   rounding of the 16-bit P it feeds);  2^x = bits(2^f) + (n << 23).
// Used for a fraction of the softmax exponentials so that the 16-per-clock SFU is not the bottleneck.
__device__ __forceinline__ float2 exp2_pair_poly(float a, float b, float scale, float bias) {
    unsigned long long x, sc, bi, t, nf, f, pz, magic, nmagic, c0, c1, c2, c3, m1;
    asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(a), "f"(b));
    asm("mov.b64 %0, {%1, %1};" : "=l"(sc) : "f"(scale));
    asm("mov.b64 %0, {%1, %1};" : "=l"(bi) : "f"(bias));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(x) : "l"(x), "l"(sc), "l"(bi));
    float xl, xh;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(xl), "=f"(xh) : "l"(x));
    xl = fmaxf(xl, -126.f); xh = fmaxf(xh, -126.f);
    asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(xl), "f"(xh));
    asm("mov.b64 %0, {%1, %1};" : "=l"(magic) : "f"(12582912.f));
    asm("mov.b64 %0, {%1, %1};" : "=l"(nmagic) : "f"(-12582912.f));
    asm("mov.b64 %0, {%1, %1};" : "=l"(m1) : "f"(-1.f));
    asm("mov.b64 %0, {%1, %1};" : "=l"(c0) : "f"(0.99992806f));
    asm("mov.b64 %0, {%1, %1};" : "=l"(c1) : "f"(0.69326097f));
    asm("mov.b64 %0, {%1, %1};" : "=l"(c2) : "f"(0.24261113f));
    asm("mov.b64 %0, {%1, %1};" : "=l"(c3) : "f"(0.05517167f));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(t) : "l"(x), "l"(magic));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(nf) : "l"(t), "l"(nmagic));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(f) : "l"(nf), "l"(m1), "l"(x));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(pz) : "l"(f), "l"(c3), "l"(c2));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(pz) : "l"(pz), "l"(f), "l"(c1));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(pz) : "l"(pz), "l"(f), "l"(c0));
    unsigned pl, ph, tl, th;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(pl), "=r"(ph) : "l"(pz));
    asm("mov.b64 {%0, %1}, %2;" : "=r"(tl), "=r"(th) : "l"(t));
    return make_float2(__uint_as_float(pl + (tl << 23)), __uint_as_float(ph + (th << 23)));
}

} // namespace b200p
