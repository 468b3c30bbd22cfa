// ---------------------------------------------------------------------------
// skinny_gemm.cuh -- Y[M,N] = X[M,K] . W[N,K]^T for the decode step (M <= 8 rows).
//
// At decode time the reference runs every projection as a rocBLAS GEMM with
// M = batch (cdna3-prims/include/cdna3/runtime/rocblas_gemm.hpp:112-209) between
// separate RMSNorm / SiLU kernels (forward.hpp:34-56, 154-160).  With a handful of
// rows these products are streams over the weight matrix: HBM-bound, and short
// enough that launch and dependency latency count.  This kernel treats them so:
//
//  * W is [N, K] with K contiguous, so one warp owns two output columns (two rows
//    of W) and streams them with 32-byte loads, 4 x 2 vectors in flight per lane,
//    issued BEFORE the prologue so that weights travel while activations are
//    prepared; nothing of W is ever staged in shared memory;
//  * X (16-bit, at most 8 rows) sits in shared memory, read as 32-byte rows;
//    accumulation is fp32, the lanes' partial sums meet in the warp butterfly of
//    wave64.cuh (wave::dpp::reduce_sum, 32-lane form);
//  * prologue PRO_RMSNORM computes the RMSNorm of the fp32 residual stream (one
//    warp per row) straight into shared memory: the norm kernel and its 16-bit
//    round trip through HBM are gone;
//  * epilogues: 16-bit store (Q/K/V), fp32 store (logits), fp32 accumulate into
//    the residual stream (O and down projections: the GEMM's beta = 1), and
//    SiLU(gate) * up over row pairs (n, n + F) of the concatenated gate/up matrix.
//
// Same arithmetic contract as the GEMM path: 16-bit operands, fp32 products and
// sums, outputs rounded once.
// ---------------------------------------------------------------------------
#pragma once
#include "common.cuh"
#include "attn_common.cuh"
#include "vec_io.cuh"
#include "wave_primitives/wave64.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b200p {

enum SkinnyPrologue { PRO_PLAIN = 0, PRO_RMSNORM = 1 };
enum SkinnyEpilogue { EPI_STORE16 = 0, EPI_ACC32 = 1, EPI_STORE32 = 2, EPI_SILU16 = 3 };

struct SkinnyArgs {
    const void*  W;        // [N][K] 16-bit (EPI_SILU16: [2N][K], gate rows then up rows)
    const void*  X16;      // PRO_PLAIN:   [M][ldx] 16-bit activations
    const float* X32;      // PRO_RMSNORM: [M][K] fp32 residual stream
    const void*  norm_w;   // PRO_RMSNORM: [K] 16-bit norm weights
    void*        out;      // [M][ldo] 16-bit or fp32
    int M, N, K, ldx, ldo;
    float eps;
};

constexpr int kSkinnyThreads = 256;
constexpr int kSkinnyMaxM = 8;
constexpr int kSkinnyChunks = 4;      // 32-byte vectors per lane per row in flight

template <typename T> __device__ __forceinline__ void unpack_pair(uint32_t w, float& a, float& b);
template <> __device__ __forceinline__ void unpack_pair<__nv_bfloat16>(uint32_t w, float& a, float& b) {
    a = __uint_as_float(w << 16); b = __uint_as_float(w & 0xffff0000u);
}
template <> __device__ __forceinline__ void unpack_pair<__half>(uint32_t w, float& a, float& b) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    a = f.x; b = f.y;
}

template <typename T, int MT, int PRO, int EPI>
__global__ void __launch_bounds__(kSkinnyThreads, 2)
skinny_gemm_kernel(const SkinnyArgs a) {
    extern __shared__ __align__(32) unsigned char skinny_smem[];
    T* xs = reinterpret_cast<T*>(skinny_smem);                 // [MT][K]
    constexpr int CH = kSkinnyChunks;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int K = a.K;
    const int nchunk = (K + 511) / 512;                        // 512 elements = 32 lanes x 16
    const int npairs = EPI == EPI_SILU16 ? a.N : (a.N + 1) / 2;
    const int nwarps = gridDim.x * (kSkinnyThreads / 32);
    const char* Wb = static_cast<const char*>(a.W);

    uint32_t wreg[2][CH][8];
    // rows of W for pair p, and whether the second exists
    auto rows_of = [&](int p, size_t& r0, size_t& r1, bool& has1) {
        if (EPI == EPI_SILU16) { r0 = size_t(p); r1 = size_t(p) + size_t(a.N); has1 = true; }
        else                   { r0 = 2 * size_t(p); r1 = r0 + 1; has1 = int(r1) < a.N; }
    };
    auto load_group = [&](int p, int c0) {
        size_t r0, r1; bool has1;
        rows_of(p, r0, r1, has1);
        #pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int k0 = ((c0 + c) * 32 + lane) * 16;
            if (c0 + c < nchunk && k0 < K) {
                VecIO<32>::load(Wb + (r0 * K + k0) * 2, wreg[0][c]);
                if (has1) VecIO<32>::load(Wb + (r1 * K + k0) * 2, wreg[1][c]);
            }
        }
    };

    int p = blockIdx.x * (kSkinnyThreads / 32) + warp;
    if (p < npairs) load_group(p, 0);                          // weights travel during the prologue

    // ---- prologue: X into shared memory as 16-bit ------------------------------------------------
    if (PRO == PRO_RMSNORM) {
        // forward.hpp:34-56: y = x * rsqrt(mean(x^2) + eps) * w; one warp per row
        for (int m = warp; m < MT; m += kSkinnyThreads / 32) {
            T* dst = xs + size_t(m) * K;
            if (m < a.M) {
                const float* x = a.X32 + size_t(m) * K;
                float ss = 0.f;
                for (int i = lane * 4; i < K; i += 128) {
                    const float4 v = *reinterpret_cast<const float4*>(x + i);
                    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                }
                ss = wave::dpp::reduce_sum(ss);
                const float inv = rsqrtf(ss / K + a.eps);
                const T* nw = static_cast<const T*>(a.norm_w);
                for (int i = lane * 4; i < K; i += 128) {
                    const float4 v = *reinterpret_cast<const float4*>(x + i);
                    dst[i]     = from_float<T>(v.x * inv * to_float(nw[i]));
                    dst[i + 1] = from_float<T>(v.y * inv * to_float(nw[i + 1]));
                    dst[i + 2] = from_float<T>(v.z * inv * to_float(nw[i + 2]));
                    dst[i + 3] = from_float<T>(v.w * inv * to_float(nw[i + 3]));
                }
            } else {
                for (int i = lane; i < K; i += 32) dst[i] = from_float<T>(0.f);
            }
        }
    } else {
        const int vec_per_row = K / 8;                          // 16-byte vectors
        for (int i = threadIdx.x; i < MT * vec_per_row; i += kSkinnyThreads) {
            const int m = i / vec_per_row, v = i % vec_per_row;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (m < a.M) val = *reinterpret_cast<const uint4*>(static_cast<const T*>(a.X16) + size_t(m) * a.ldx + size_t(v) * 8);
            *reinterpret_cast<uint4*>(xs + size_t(m) * K + size_t(v) * 8) = val;
        }
    }
    __syncthreads();

    // ---- stream the rows of W ---------------------------------------------------------------------
    for (; p < npairs; p += nwarps) {
        size_t r0, r1; bool has1;
        rows_of(p, r0, r1, has1);
        float acc[2][MT];
        #pragma unroll
        for (int m = 0; m < MT; ++m) { acc[0][m] = 0.f; acc[1][m] = 0.f; }
        for (int c0 = 0; c0 < nchunk; c0 += CH) {
            if (c0 > 0) load_group(p, c0);
            #pragma unroll
            for (int c = 0; c < CH; ++c) {
                const int k0 = ((c0 + c) * 32 + lane) * 16;
                if (c0 + c < nchunk && k0 < K) {
                    float w0[16], w1[16];
                    #pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        unpack_pair<T>(wreg[0][c][i], w0[2 * i], w0[2 * i + 1]);
                        if (has1) unpack_pair<T>(wreg[1][c][i], w1[2 * i], w1[2 * i + 1]);
                        else      { w1[2 * i] = 0.f; w1[2 * i + 1] = 0.f; }
                    }
                    #pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        const uint4* xp = reinterpret_cast<const uint4*>(xs + size_t(m) * K + k0);
                        const uint4 xa = xp[0], xb = xp[1];
                        const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                        #pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float x0, x1;
                            unpack_pair<T>(xw[i], x0, x1);
                            acc[0][m] = fmaf(w0[2 * i], x0, acc[0][m]); acc[0][m] = fmaf(w0[2 * i + 1], x1, acc[0][m]);
                            acc[1][m] = fmaf(w1[2 * i], x0, acc[1][m]); acc[1][m] = fmaf(w1[2 * i + 1], x1, acc[1][m]);
                        }
                    }
                }
            }
        }
        // issue the next pair's first loads before the reduction
        const int pn = p + nwarps;
        #pragma unroll
        for (int m = 0; m < MT; ++m) {
            acc[0][m] = wave::dpp::reduce_sum(acc[0][m]);
            acc[1][m] = wave::dpp::reduce_sum(acc[1][m]);
        }
        if (pn < npairs) load_group(pn, 0);
        if (lane == 0) {
            #pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m >= a.M) break;
                if (EPI == EPI_SILU16) {
                    const float g = acc[0][m], u = acc[1][m];
                    static_cast<T*>(a.out)[size_t(m) * a.ldo + p] = from_float<T>((g / (1.f + expf(-g))) * u);
                } else {
                    #pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        if (r == 1 && !has1) break;
                        const size_t idx = size_t(m) * a.ldo + (r ? r1 : r0);
                        if (EPI == EPI_STORE16)      static_cast<T*>(a.out)[idx] = from_float<T>(acc[r][m]);
                        else if (EPI == EPI_STORE32) static_cast<float*>(a.out)[idx] = acc[r][m];
                        else                         static_cast<float*>(a.out)[idx] += acc[r][m];
                    }
                }
            }
        }
    }
}

// Launch: returns B200P_E_RANGE when the shape is outside the kernel's domain (the caller then
// takes the library GEMM).  K must be a multiple of 16 (32-byte rows of W and X), ldx of 8.
template <typename T, int PRO, int EPI>
int launch_skinny(const SkinnyArgs& a, cudaStream_t st) {
    if (a.M < 1 || a.M > kSkinnyMaxM || a.K % 16 != 0 || a.N < 1) return B200P_E_RANGE;
    if (PRO == PRO_PLAIN && (a.ldx % 8 != 0 || !aligned(a.X16, 16))) return B200P_E_RANGE;
    if (!aligned(a.W, 32)) return B200P_E_RANGE;
    const int MT = a.M <= 1 ? 1 : a.M <= 2 ? 2 : a.M <= 4 ? 4 : 8;
    const size_t smem = size_t(MT) * a.K * 2;
    if (smem > 200 * 1024) return B200P_E_RANGE;
    const int npairs = EPI == EPI_SILU16 ? a.N : (a.N + 1) / 2;
    const int sms = sm_count() > 0 ? sm_count() : 148;
    int grid = (npairs + 7) / 8;
    if (grid > 2 * sms) grid = 2 * sms;
    auto go = [&](auto kern) -> int {
        if (smem > 48 * 1024) {
            const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
            if (e != cudaSuccess) return int(e);
        }
        kern<<<grid, kSkinnyThreads, smem, st>>>(a);
        return launched();
    };
    switch (MT) {
        case 1: return go(skinny_gemm_kernel<T, 1, PRO, EPI>);
        case 2: return go(skinny_gemm_kernel<T, 2, PRO, EPI>);
        case 4: return go(skinny_gemm_kernel<T, 4, PRO, EPI>);
        default: return go(skinny_gemm_kernel<T, 8, PRO, EPI>);
    }
}

} // namespace b200p
