// ---------------------------------------------------------------------------
// skinny_gemm.cuh -- Y[M,N] = X[M,K] . W[N,K]^T for the decode step (M <= 16 rows).
//
// At decode time the reference runs every projection as a rocBLAS GEMM with
// M = batch (cdna3-prims/include/cdna3/runtime/rocblas_gemm.hpp:112-209) between
// separate RMSNorm / SiLU kernels (forward.hpp:34-56, 154-160).  With a handful of
// rows these products are streams over the weight matrix: HBM-bound, and short
// enough that launch and dependency latency count.  This kernel treats them so.
//
//  * One CTA owns 16 rows of W (16 output columns); its 8 warps split K.  Every
//    lane loads 32 contiguous bytes of one row per step, four steps for each of
//    its two rows in flight (the whole share of a warp when K = 2048), issued
//    BEFORE the prologue so that the weights travel while the activations are
//    prepared.  W never touches shared memory.
//  * The product runs on the tensor cores as mma.sync m16n8k16 with W as the A
//    operand (16 rows) and X^T as B (8 columns = up to 8 rows of X).  A dot
//    product does not care about the order of k, so the 16 values a lane loaded
//    ARE its A fragments: within a 64-wide block, lane t4 of a row's four lanes
//    supplies columns 16*t4 + 4s .. +3 to k-step s, and reads the same columns
//    of X for the B fragment.  No unpacking, no shuffles: 4 MMAs per 2 KB of W.
//  * X (16-bit, M rounded up to 1, 2, 4, 8 or 16 rows) sits in shared memory with rows 16 bytes
//    longer than K, which makes the 16-byte fragment reads bank-conflict free.  Up to 8 rows of X
//    are the 8 columns of ONE B fragment; rows 8..15 are a second B fragment and a second MMA
//    per A fragment (template parameter MH = 2), so the weights are still read once.
//  * Prologue PRO_RMSNORM computes the RMSNorm of the fp32 residual stream
//    straight into shared memory (all 8 warps, values held in registers between
//    the sum of squares and the scaling): the norm kernel and its 16-bit round
//    trip through HBM are gone.
//  * The kernel is launched as a programmatic dependent of its predecessor: its
//    CTAs start while that kernel drains, put their weight loads in flight, and
//    only then wait (griddepcontrol.wait) for the activations.
//  * The 8 partial accumulators meet in shared memory; epilogues: 16-bit store
//    (Q/K/V), fp32 store (logits), fp32 accumulate into the residual stream (O
//    and down projections: the GEMM's beta = 1), and SiLU(gate) * up, for which a
//    CTA takes 8 gate rows and the 8 matching up rows of the concatenated matrix.
//
// Same arithmetic contract as the GEMM path: 16-bit operands, fp32 products and
// sums, outputs rounded once.
//
// Two kernels share the fragment scheme, the prologue and the epilogues:
// skinny_gemm_kernel as described above (W goes from global memory to registers to
// the MMA), and skinny_stream_kernel further down, the default, in which a producer
// thread stages W through a shared-memory ring so that loads run ahead across row
// groups and the bytes in flight are not bounded by registers.
// ---------------------------------------------------------------------------
#pragma once
#include "common.cuh"
#include "attn_common.cuh"
#include "dme/dme_tma.cuh"
#include "mma_sync.cuh"
#include "vec_io.cuh"
#include "wave_primitives/wave64.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace b200p {

enum SkinnyPrologue { PRO_PLAIN = 0, PRO_RMSNORM = 1 };
enum SkinnyEpilogue { EPI_STORE16 = 0, EPI_ACC32 = 1, EPI_STORE32 = 2, EPI_SILU16 = 3, EPI_ROPE = 4,
                      EPI_STORE32_BEST = 5 };   // fp32 store + running argmax key per row (decode_mega.cuh only)

// EPI_ROPE: W is the concatenated Q/K/V projection; the epilogue is the reference's bias add,
// rotate-half RoPE and KV-cache scatter (forward.hpp:135-148, 211-224; rocblas_gemm.hpp:56-63)
// for ONE new token per sequence (row m of X is sequence m).  A CTA takes 8 rows d and the 8
// rows d + D/2 of one head, so each rotation pair meets in one thread.
struct SkinnyRope {
    const void*  bias;      // [N] 16-bit or null
    const float* cos_t;     // [max_seq][D/2]
    const float* sin_t;
    void* kcache;           // [batch][nKVH][max_seq][D] 16-bit
    void* vcache;
    const int* pos_dev;     // position of the new token, read on the device (null: pos0)
    int pos0, nQH, nKVH, D, max_seq;
};

struct SkinnyArgs {
    const void*  W;        // [N][K] 16-bit (EPI_SILU16: [2N][K], gate rows then up rows)
    const void*  X16;      // PRO_PLAIN:   [M][ldx] 16-bit activations
    const float* X32;      // PRO_RMSNORM: [M][K] fp32 residual stream
    const void*  norm_w;   // PRO_RMSNORM: [K] 16-bit norm weights
    const void*  Xemb;     // skinny_prologue<T, PRO_RMSNORM, true>: row m of X is float(Xemb[Xids[m]][:]) (16-bit table [*][K]) instead of X32
    const int*   Xids;
    void*        out;      // [M][ldo] 16-bit or fp32
    int M, N, K, ldx, ldo;
    float eps;
    SkinnyRope rope;       // EPI_ROPE only
    int* abort_word;       // streaming kernel: the abort word its bounded waits poll and raise.  A caller that
                           // launches many of these on one stream (the runtime's decode step) owns one word,
                           // clears it before the step and reads it after; null: a per-launch slot is taken.
};

constexpr int kSkinnyThreads = 256;
constexpr int kSkinnyWarps = kSkinnyThreads / 32;
constexpr int kSkinnyMaxM = 16;
constexpr int kSkinnyDepth = 4;       // 64-column blocks in flight per warp
constexpr int kSkinnyXPad = 8;        // elements: X rows are 16 bytes longer than K

// Barrier over the 256 threads that compute (the whole CTA of skinny_gemm_kernel; the eight
// consumer warps of skinny_stream_kernel, whose producer warp is streaming meanwhile).
__device__ __forceinline__ void skinny_barrier() { asm volatile("bar.sync 1, %0;" :: "r"(kSkinnyThreads) : "memory"); }

// X into shared memory as 16-bit rows of K + kSkinnyXPad elements, rows in [M, Mp) zero; ends with a barrier.
template <typename T, int PRO, bool EMB = false>
__device__ __forceinline__ void skinny_prologue(const SkinnyArgs& a, T* xs, float* part_ss, int Mp, int warp, int lane) {
    const int K = a.K, xstride = K + kSkinnyXPad;
    // ---- prologue: X into shared memory as 16-bit, rows in [M, Mp) zero --------------------------------
    if (PRO == PRO_RMSNORM && Mp > kSkinnyWarps) {
        // more rows than warps (Mp = 16): a warp normalises rows warp and warp + 8, one after the other
        const T* nw = static_cast<const T*>(a.norm_w);
        for (int m = warp; m < Mp; m += kSkinnyWarps) {
            T* dst = xs + size_t(m) * xstride;
            if (m < a.M) {
                const float* x = a.X32 + size_t(m) * K;
                float ss = 0.f;
                for (int q = lane; q < K / 4; q += 32) {
                    const float4 v = *reinterpret_cast<const float4*>(x + 4 * q);
                    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                }
                ss = wave::dpp::reduce_sum(ss);
                const float inv = rsqrtf(ss / K + a.eps);
                for (int q = lane; q < K / 4; q += 32) {
                    const float4 v = *reinterpret_cast<const float4*>(x + 4 * q);
                    const uint2 wv = *reinterpret_cast<const uint2*>(nw + 4 * q);
                    const T* w4 = reinterpret_cast<const T*>(&wv);
                    uint2 o;
                    o.x = pack2<T>(v.x * inv * to_float(w4[0]), v.y * inv * to_float(w4[1]));
                    o.y = pack2<T>(v.z * inv * to_float(w4[2]), v.w * inv * to_float(w4[3]));
                    *reinterpret_cast<uint2*>(dst + 4 * q) = o;
                }
            } else {
                for (int q = lane; q < K / 4; q += 32) *reinterpret_cast<uint2*>(dst + 4 * q) = make_uint2(0u, 0u);
            }
        }
    } else if (PRO == PRO_RMSNORM) {
        // forward.hpp:34-56: y = x * rsqrt(mean(x^2) + eps) * w.  8 / Mp warps share a row; each keeps
        // up to 4 quads per lane in registers between the sum of squares and the scaling.
        constexpr int CACHE = 4;
        const int wpr = kSkinnyWarps / Mp;                      // warps per row
        const int m = warp / wpr, part = warp % wpr;
        const int quads = K / 4, qper = (quads + wpr - 1) / wpr;
        const int q0 = part * qper, q1 = min(q0 + qper, quads);
        const float* x = a.X32 + size_t(m) * K;
        const T* xe = EMB && m < a.M ? static_cast<const T*>(a.Xemb) + size_t(a.Xids[m]) * K : nullptr;
        auto ldx = [&](int q) -> float4 {                       // four elements of row m as fp32
            if (!EMB) return *reinterpret_cast<const float4*>(x + 4 * q);
            const uint2 r = *reinterpret_cast<const uint2*>(xe + 4 * q);
            const T* e = reinterpret_cast<const T*>(&r);
            return make_float4(to_float(e[0]), to_float(e[1]), to_float(e[2]), to_float(e[3]));
        };
        const T* nw = static_cast<const T*>(a.norm_w);
        T* dst = xs + size_t(m) * xstride;
        float4 cx[CACHE]; float4 cw[CACHE];                    // the norm weights as fp32: converted here, so that their loads
        float ss = 0.f;                                        // have landed before the barrier and not behind it
        if (m < a.M) {
            #pragma unroll
            for (int it = 0; it < CACHE; ++it) {
                const int q = q0 + lane + 32 * it;
                if (q < q1) {
                    cx[it] = ldx(q);
                    const uint2 wv = *reinterpret_cast<const uint2*>(nw + 4 * q);
                    const T* w4 = reinterpret_cast<const T*>(&wv);
                    cw[it] = make_float4(to_float(w4[0]), to_float(w4[1]), to_float(w4[2]), to_float(w4[3]));
                    ss += cx[it].x * cx[it].x + cx[it].y * cx[it].y + cx[it].z * cx[it].z + cx[it].w * cx[it].w;
                }
            }
            for (int q = q0 + lane + 32 * CACHE; q < q1; q += 32) {
                const float4 v = ldx(q);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
        const float inv_k = 1.f / float(K);                     // off the chain: computed while the loads are in flight
        ss = wave::dpp::reduce_sum(ss);
        if (lane == 0) part_ss[warp] = ss;
        skinny_barrier();
        // all eight partial sums in two vector loads, then the row's own: a loop of dependent loads and adds, a
        // division and the root made 0.5 us of this scalar tail
        const float4 pa = *reinterpret_cast<const float4*>(&part_ss[0]), pb = *reinterpret_cast<const float4*>(&part_ss[4]);
        const float pv[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
        float tot = 0.f;
        #pragma unroll
        for (int w = 0; w < kSkinnyWarps; ++w) tot += (w >= m * wpr && w < (m + 1) * wpr) ? pv[w] : 0.f;
        const float inv = rsqrtf(tot * inv_k + a.eps);
        auto put = [&](int q, const float4& v, const float4& w) {
            uint2 o;
            o.x = pack2<T>(v.x * inv * w.x, v.y * inv * w.y);
            o.y = pack2<T>(v.z * inv * w.z, v.w * inv * w.w);
            *reinterpret_cast<uint2*>(dst + 4 * q) = o;
        };
        auto ldw = [&](int q) -> float4 {
            const uint2 wv = *reinterpret_cast<const uint2*>(nw + 4 * q);
            const T* w4 = reinterpret_cast<const T*>(&wv);
            return make_float4(to_float(w4[0]), to_float(w4[1]), to_float(w4[2]), to_float(w4[3]));
        };
        if (m < a.M) {
            #pragma unroll
            for (int it = 0; it < CACHE; ++it) {
                const int q = q0 + lane + 32 * it;
                if (q < q1) put(q, cx[it], cw[it]);
            }
            for (int q = q0 + lane + 32 * CACHE; q < q1; q += 32)
                put(q, ldx(q), ldw(q));
        } else {
            for (int q = q0 + lane; q < q1; q += 32) *reinterpret_cast<uint2*>(dst + 4 * q) = make_uint2(0u, 0u);
        }
    } else {
        // 16-byte vectors, two rows at a time and up to three vectors per row and thread: the loads of a batch are all
        // issued before its first store.  (One load and one store per trip, the stores to xs order the loads behind
        // them: two rows of 5632 columns took six dependent trips to L2.)
        constexpr int VB = 3;
        const int vec_per_row = K / 8;
        for (int m0 = 0; m0 < Mp; m0 += 2) {
            for (int base = warp * 32 + lane; base < vec_per_row; base += kSkinnyThreads * VB) {
                uint4 val[2][VB];
                #pragma unroll
                for (int r = 0; r < 2; ++r) {
                    #pragma unroll
                    for (int u = 0; u < VB; ++u) {
                        const int v = base + u * kSkinnyThreads;
                        val[r][u] = make_uint4(0u, 0u, 0u, 0u);
                        if (m0 + r < a.M && v < vec_per_row)
                            val[r][u] = *reinterpret_cast<const uint4*>(static_cast<const T*>(a.X16) + size_t(m0 + r) * a.ldx + size_t(v) * 8);
                    }
                }
                #pragma unroll
                for (int r = 0; r < 2; ++r) {
                    #pragma unroll
                    for (int u = 0; u < VB; ++u) {
                        const int v = base + u * kSkinnyThreads;
                        if (m0 + r < Mp && v < vec_per_row) *reinterpret_cast<uint4*>(xs + size_t(m0 + r) * xstride + size_t(v) * 8) = val[r][u];
                    }
                }
            }
        }
    }
    skinny_barrier();

}

// The eight warps' partial accumulators (red[warp][lane][4]: the m16n8 C fragments) meet; the first 64 * R
// threads write the group's outputs.  prev: for EPI_ACC32, the residual values fetched ahead (use_prev).
// What a thread's epilogue of row group grp reads from global memory, fetched BEFORE the group's products so
// that the latency lies under them: the residual values (EPI_ACC32), the rotation's cos / sin and the bias
// pair (EPI_ROPE).  The values must not change between the fetch and the epilogue: true after the grid
// dependency wait / the grid barrier that precedes the product, since each output element has one owner.
template <int MH>
struct EpiAhead {
    float prev[MH];
    float c, sn, b0, b1;
};
template <typename T, int EPI, int R, int MH>
__device__ __forceinline__ void skinny_epilogue_fetch(const SkinnyArgs& a, int grp, int tid, EpiAhead<MH>& e) {
    if (EPI == EPI_ACC32) {
        if (tid < 64 * R) {
            const int l = tid % 32, c = tid / 32;
            const int n = grp * 8 * R + l / 4 + 8 * (c >> 1);
            #pragma unroll
            for (int mh = 0; mh < MH; ++mh) {
                const int m = 8 * mh + 2 * (l % 4) + (c & 1);
                e.prev[mh] = (m < a.M && n < a.N) ? static_cast<const float*>(a.out)[size_t(m) * a.ldo + n] : 0.f;
            }
        }
    } else if (EPI == EPI_ROPE) {
        if (tid < 64) {
            const SkinnyRope& r = a.rope;
            const int l = tid % 32;
            const int cph = r.D / 16, half = r.D / 2;
            const int slot = grp / cph, d = (grp % cph) * 8 + l / 4;
            const int pos = r.pos_dev ? min(*r.pos_dev, r.max_seq - 1) : r.pos0;
            e.c = r.cos_t[size_t(pos) * half + d]; e.sn = r.sin_t[size_t(pos) * half + d];
            e.b0 = e.b1 = 0.f;
            if (r.bias) {
                const T* bias = static_cast<const T*>(r.bias);
                e.b0 = to_float(bias[slot * r.D + d]); e.b1 = to_float(bias[slot * r.D + d + half]);
            }
        }
    }
}

// red[warp][lane][4 * mh + c]: the m16n8 C fragment of the MMA over rows 8 mh .. 8 mh + 7 of X.
template <typename T, int EPI, int R, int MH>
__device__ __forceinline__ void skinny_epilogue(const SkinnyArgs& a, const float (*red)[32][4 * MH], int grp, int tid, bool use_prev, float prev,
                                                unsigned long long* best = nullptr, const EpiAhead<MH>* ahead = nullptr) {
    #pragma unroll
    for (int mh = 0; mh < MH; ++mh) {
        if (EPI == EPI_SILU16) {
            if (tid < 64) {
                const int l = tid % 32, sel = tid / 32;
                float gate = 0.f, up = 0.f;
                #pragma unroll
                for (int w = 0; w < kSkinnyWarps; ++w) { gate += red[w][l][4 * mh + sel]; up += red[w][l][4 * mh + 2 + sel]; }
                const int m = 8 * mh + 2 * (l % 4) + sel, p = grp * 8 + l / 4;
                if (m < a.M && p < a.N)
                    static_cast<T*>(a.out)[size_t(m) * a.ldo + p] = from_float<T>((gate / (1.f + expf(-gate))) * up);
            }
        } else if (EPI == EPI_ROPE) {
            if (tid < 64) {
                const SkinnyRope& r = a.rope;
                const int l = tid % 32, sel = tid / 32;
                float x0 = 0.f, x1 = 0.f;
                #pragma unroll
                for (int w = 0; w < kSkinnyWarps; ++w) { x0 += red[w][l][4 * mh + sel]; x1 += red[w][l][4 * mh + 2 + sel]; }
                const int m = 8 * mh + 2 * (l % 4) + sel;
                if (m < a.M) {
                    const int cph = r.D / 16, half = r.D / 2;
                    const int slot = grp / cph, d = (grp % cph) * 8 + l / 4;
                    x0 = to_float(from_float<T>(x0)); x1 = to_float(from_float<T>(x1));      // the projection's 16-bit output
                    if (r.bias) {
                        const T* bias = static_cast<const T*>(r.bias);
                        x0 = to_float(from_float<T>(x0 + (ahead ? ahead->b0 : to_float(bias[slot * r.D + d]))));
                        x1 = to_float(from_float<T>(x1 + (ahead ? ahead->b1 : to_float(bias[slot * r.D + d + half]))));
                    }
                    const int pos = r.pos_dev ? min(*r.pos_dev, r.max_seq - 1) : r.pos0;
                    if (slot < r.nQH + r.nKVH) {                  // q or k: rotate
                        const float c = ahead ? ahead->c : r.cos_t[size_t(pos) * half + d], sn = ahead ? ahead->sn : r.sin_t[size_t(pos) * half + d];
                        const float y0 = x0 * c - x1 * sn, y1 = x1 * c + x0 * sn;
                        x0 = y0; x1 = y1;
                    }
                    const T o0 = from_float<T>(x0), o1 = from_float<T>(x1);
                    if (slot < r.nQH) {                           // q stays in the token-major buffer
                        T* row = static_cast<T*>(a.out) + size_t(m) * a.ldo + size_t(slot) * r.D;
                        row[d] = o0; row[d + half] = o1;
                    } else {                                      // k or v: into cache[m][kvh][pos][:]
                        const bool is_k = slot < r.nQH + r.nKVH;
                        const int kvh = is_k ? slot - r.nQH : slot - r.nQH - r.nKVH;
                        T* dst = static_cast<T*>(is_k ? r.kcache : r.vcache) + ((size_t(m) * r.nKVH + kvh) * r.max_seq + pos) * r.D;
                        dst[d] = o0; dst[d + half] = o1;
                    }
                }
            }
        } else if (tid < 64 * R) {
            const int l = tid % 32, c = tid / 32;
            float v = 0.f;
            #pragma unroll
            for (int w = 0; w < kSkinnyWarps; ++w) v += red[w][l][4 * mh + c];
            const int m = 8 * mh + 2 * (l % 4) + (c & 1), n = grp * 8 * R + l / 4 + 8 * (c >> 1);
            if (m < a.M && n < a.N) {
                const size_t idx = size_t(m) * a.ldo + n;
                if (EPI == EPI_STORE16)      static_cast<T*>(a.out)[idx] = from_float<T>(v);
                else if (EPI == EPI_STORE32) static_cast<float*>(a.out)[idx] = v;
                else if (EPI == EPI_STORE32_BEST) {
                    // forward.hpp:244-262: argmax over the 16-bit logits, ties to the lowest index, as a 64-bit key
                    // (order-preserving value bits, then the complemented index); best[mh] belongs to row m
                    static_cast<float*>(a.out)[idx] = v;
                    unsigned u = __float_as_uint(to_float(from_float<T>(v)));
                    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
                    const unsigned long long key = (unsigned long long)u << 32 | (0xffffffffu - unsigned(n));
                    if (key > best[mh]) best[mh] = key;
                }
                else if (ahead)              static_cast<float*>(a.out)[idx] = ahead->prev[mh] + v;
                else if (use_prev && mh == 0) static_cast<float*>(a.out)[idx] = prev + v;
                else                         static_cast<float*>(a.out)[idx] += v;
            }
        }
    }
}

// R = rows of W per lane: 2 -> a CTA step covers 16 rows (accumulator rows g and g + 8), 4 column
// blocks in flight; 1 -> 8 rows (the upper half of the A operand is zero), 8 blocks in flight: twice
// the CTAs for matrices too small to fill the GPU otherwise.
template <typename T, int PRO, int EPI, int R, int MH>
__global__ void __launch_bounds__(kSkinnyThreads, 2)
skinny_gemm_kernel(const SkinnyArgs a) {
    griddep_launch_dependents();
    extern __shared__ __align__(128) unsigned char skinny_smem[];
    T* xs = reinterpret_cast<T*>(skinny_smem);                 // [Mp][K + pad]
    __shared__ float red[2][kSkinnyWarps][32][4 * MH];          // double-buffered by group
    __shared__ __align__(16) float part_ss[kSkinnyWarps];
    constexpr int DEPTH = 8 / R;
    static_assert(R == 2 || (EPI != EPI_SILU16 && EPI != EPI_ROPE), "paired epilogues need both halves");
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g = lane / 4, t4 = lane % 4;
    const int K = a.K, xstride = K + kSkinnyXPad;
    const int Mp = a.M <= 1 ? 1 : a.M <= 2 ? 2 : a.M <= 4 ? 4 : a.M <= 8 ? 8 : 16;   // rows of X kept in shared memory

    // Row groups: group `grp` is 8 * R rows of W (8 row pairs for the paired epilogues); the CTA
    // takes groups blockIdx.x, blockIdx.x + gridDim.x, ...
    const int ngroups = (EPI == EPI_SILU16) ? (a.N + 7) / 8 : (a.N + 8 * R - 1) / (8 * R);
    auto row_ptrs = [&](int grp, const char*& wA, const char*& wB) {
        size_t rowA, rowB;
        if (EPI == EPI_SILU16) {
            const int p = min(grp * 8 + g, a.N - 1);            // pair index: gate row p, up row N + p
            rowA = size_t(p); rowB = size_t(a.N) + size_t(p);
        } else if (EPI == EPI_ROPE) {
            const int cph = a.rope.D / 16;                      // groups per head
            rowA = size_t(grp / cph) * a.rope.D + size_t(grp % cph) * 8 + g;
            rowB = rowA + a.rope.D / 2;
        } else {
            rowA = size_t(min(grp * 8 * R + g, a.N - 1));
            rowB = size_t(min(grp * 8 * R + g + 8, a.N - 1));
        }
        wA = static_cast<const char*>(a.W) + rowA * size_t(K) * 2;
        wB = static_cast<const char*>(a.W) + rowB * size_t(K) * 2;
    };

    // this warp's share of K, in blocks of 64 columns
    const int nblk = (K + 63) / 64;
    const int per = (nblk + kSkinnyWarps - 1) / kSkinnyWarps;
    const int b0 = warp * per, b1 = min(b0 + per, nblk);
    const int nb = max(b1 - b0, 0);                             // blocks per group for this warp

    uint32_t wb[DEPTH][R][8];
    // A block is taken by the whole warp or not at all (mma.sync needs every lane); a lane whose 16
    // columns lie past K (K not a multiple of 64) contributes zeros instead of loading.
    auto lane_live = [&](int blk) { return blk * 64 + t4 * 16 < K; };
    auto issue = [&](int slot, int grp, int j) {               // block j of this warp's share, for group grp
        if (grp < ngroups && j < nb) {
            const int blk = b0 + j;
            if (lane_live(blk)) {
                const char *wA, *wB;
                row_ptrs(grp, wA, wB);
                const size_t off = (size_t(blk) * 64 + size_t(t4) * 16) * 2;
                VecIO<32>::load(wA + off, wb[slot][0]);
                if (R == 2) VecIO<32>::load(wB + off, wb[slot][R - 1]);
            } else {
                #pragma unroll
                for (int r = 0; r < R; ++r)
                    #pragma unroll
                    for (int i = 0; i < 8; ++i) wb[slot][r][i] = 0u;
            }
        }
    };
    #pragma unroll
    for (int d = 0; d < DEPTH; ++d) issue(d, blockIdx.x, d);    // weights (constants) travel during all that follows

    // Everything below reads what earlier kernels of the stream produced.
    griddep_wait();

    skinny_prologue<T, PRO>(a, xs, part_ss, Mp, warp, lane);

    // EPI_ACC32: fetch the first group's residual values now, so the epilogue's read-modify-write
    // does not start with a trip to L2
    float prev = 0.f;
    if (EPI == EPI_ACC32 && threadIdx.x < 64 * R) {
        const int l = threadIdx.x % 32, c = threadIdx.x / 32;
        const int m = 2 * (l % 4) + (c & 1), n = int(blockIdx.x) * 8 * R + l / 4 + 8 * (c >> 1);
        if (m < a.M && n < a.N) prev = static_cast<const float*>(a.out)[size_t(m) * a.ldo + n];
    }

    // ---- stream the CTA's row groups through the tensor cores ------------------------------------------
    const T* xrow = xs + size_t(g) * xstride + t4 * 16;        // B fragment: X row g, the lane's 16 columns
    int parity = 0;
    for (int grp = blockIdx.x; grp < ngroups; grp += gridDim.x, parity ^= 1) {
        float acc[MH][4];
        #pragma unroll
        for (int mh = 0; mh < MH; ++mh) { acc[mh][0] = acc[mh][1] = acc[mh][2] = acc[mh][3] = 0.f; }
        for (int jb = 0; jb < nb; jb += DEPTH) {
            #pragma unroll
            for (int d = 0; d < DEPTH; ++d) {
                const int j = jb + d;
                if (j < nb) {                                   // warp-uniform
                    const int blk = b0 + j;
                    #pragma unroll
                    for (int mh = 0; mh < MH; ++mh) {
                        uint4 xa = make_uint4(0u, 0u, 0u, 0u), xb = xa;
                        if (g + 8 * mh < Mp && lane_live(blk)) {    // columns of B past Mp are zero: no row to read
                            const uint4* xp = reinterpret_cast<const uint4*>(xrow + size_t(8 * mh) * xstride + size_t(blk) * 64);
                            xa = xp[0]; xb = xp[1];
                        }
                        const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                        #pragma unroll
                        for (int s = 0; s < 4; ++s) {
                            const uint32_t af[4] = {wb[d][0][2 * s], R == 2 ? wb[d][R - 1][2 * s] : 0u,
                                                    wb[d][0][2 * s + 1], R == 2 ? wb[d][R - 1][2 * s + 1] : 0u};
                            mma_16816<T>(acc[mh], af, xw[2 * s], xw[2 * s + 1]);
                        }
                    }
                    // the slot is free: next block of this group that maps to it, else the next group's
                    if (j + DEPTH < nb) issue(d, grp, j + DEPTH);
                    else                issue(d, grp + gridDim.x, d);
                }
            }
        }

        // ---- the 8 warps' partial sums meet; epilogue (the next group's loads are in flight) ---------
        #pragma unroll
        for (int mh = 0; mh < MH; ++mh)
            *reinterpret_cast<float4*>(&red[parity][warp][lane][4 * mh]) = make_float4(acc[mh][0], acc[mh][1], acc[mh][2], acc[mh][3]);
        skinny_barrier();
        skinny_epilogue<T, EPI, R, MH>(a, red[parity], grp, threadIdx.x, grp == int(blockIdx.x), prev);
    }
}

// ---------------------------------------------------------------------------
// skinny_stream_kernel: the same product with W staged through shared memory.
// In skinny_gemm_kernel the bytes in flight are the registers that hold them
// (8 KB per warp), and a group's loads are only issued once the previous group has
// been consumed.  Here a producer thread streams W with bulk copies into a ring of
// shared-memory stages (16 rows x up to 2048 columns each, ~64 KB, as many as fit
// beside X), running as far ahead of the eight consumer warps as the ring allows,
// across row groups; one persistent CTA per SM.  Rows are 16 bytes longer than the
// slab so that the 16-byte fragment reads of a quarter-warp (two rows x four column
// chunks) fall on eight different bank groups.  The consumers read their A
// fragments from the stage exactly as skinny_gemm_kernel reads them from
// registers; prologue and epilogue are shared.  Waits are bounded; a wait that
// gives up raises *status and the kernel drains.
// ---------------------------------------------------------------------------
constexpr int kSkinnySlab = 2048;                  // columns of W per stage
constexpr int kSkinnyStreamThreads = kSkinnyThreads + 32;

template <typename T, int PRO, int EPI, int MH>
__global__ void __launch_bounds__(kSkinnyStreamThreads, 1)
skinny_stream_kernel(const SkinnyArgs a, int nstages, int slab_cols, int* status, int* sticky) {
    griddep_launch_dependents();
    extern __shared__ __align__(128) unsigned char skinny_smem[];
    __shared__ float red[2][kSkinnyWarps][32][4 * MH];
    __shared__ __align__(16) float part_ss[kSkinnyWarps];
    __shared__ uint64_t bars[16];
    constexpr int kMaxStages = 8;
    uint64_t* full_bar = bars;
    uint64_t* empty_bar = bars + kMaxStages;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int K = a.K, xstride = K + kSkinnyXPad;
    const int Mp = a.M <= 1 ? 1 : a.M <= 2 ? 2 : a.M <= 4 ? 4 : a.M <= 8 ? 8 : 16;
    const int slab = K < slab_cols ? K : slab_cols;               // columns per stage
    const int nslab = (K + slab - 1) / slab;
    const int rowb = slab * 2 + 16;                               // bytes between rows of a stage
    const int stage_bytes = 16 * rowb;
    const int x_bytes = ((Mp * xstride * 2 + 127) / 128) * 128;
    T* xs = reinterpret_cast<T*>(skinny_smem);
    unsigned char* stages = skinny_smem + x_bytes;
    const int ngroups = (EPI == EPI_SILU16) ? (a.N + 7) / 8 : (a.N + 15) / 16;

    if (threadIdx.x == 0) {
        for (int s = 0; s < nstages; ++s) { dme::mbar_init(&full_bar[s], 1); dme::mbar_init(&empty_bar[s], kSkinnyWarps); }
        dme::mbar_init_fence();
    }
    __syncthreads();

    if (warp == kSkinnyWarps) {
        // ---- producer: W is constant, so it streams before and through the dependency wait of the consumers ----
        if (lane == 0) {
            const uint64_t pol = dme::policy_evict_first();
            int stage = 0, uses = 0; uint32_t phase = 0;
            bool ok = true;
            for (int grp = blockIdx.x; grp < ngroups && ok; grp += gridDim.x) {
                for (int sl = 0; sl < nslab; ++sl) {
                    if (uses >= nstages && !dme::wait(&empty_bar[stage], phase ^ 1u, status)) { ok = false; break; }
                    const int c0 = sl * slab, cols = min(slab, K - c0);
                    unsigned char* dst = stages + size_t(stage) * stage_bytes;
                    dme::mbar_arrive_expect_tx(&full_bar[stage], uint32_t(16 * cols * 2));
                    for (int r = 0; r < 16; ++r) {
                        size_t row;
                        if (EPI == EPI_SILU16)    row = r < 8 ? size_t(min(grp * 8 + r, a.N - 1)) : size_t(a.N) + size_t(min(grp * 8 + r - 8, a.N - 1));
                        else if (EPI == EPI_ROPE) { const int cph = a.rope.D / 16;
                                                    row = size_t(grp / cph) * a.rope.D + size_t(grp % cph) * 8 + (r & 7) + (r >= 8 ? a.rope.D / 2 : 0); }
                        else                      row = size_t(min(grp * 16 + r, a.N - 1));
                        dme::copy_tile_1d_stream(dst + size_t(r) * rowb, static_cast<const char*>(a.W) + (row * size_t(K) + c0) * 2,
                                                 uint32_t(cols * 2), &full_bar[stage], pol);
                    }
                    ++uses; if (++stage == nstages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) atomicExch(sticky, 1);
        }
    } else {
        // ---- consumers ------------------------------------------------------------------------------------------
        const int g = lane / 4, t4 = lane % 4;
        griddep_wait();                                           // activations come from earlier kernels of the stream
        skinny_prologue<T, PRO>(a, xs, part_ss, Mp, warp, lane);
        const T* xrow = xs + size_t(g) * xstride + t4 * 16;
        int stage = 0; uint32_t phase = 0;
        int parity = 0;
        bool ok = true;
        for (int grp = blockIdx.x; grp < ngroups; grp += gridDim.x, parity ^= 1) {
            // one accumulator per 16-column step of a 64-column block: four independent chains instead of one of
            // 4 x (blocks per warp) dependent MMAs; they meet in one balanced add per group
            float acc[MH][4][4];
            #pragma unroll
            for (int mh = 0; mh < MH; ++mh) {
                #pragma unroll
                for (int s = 0; s < 4; ++s) { acc[mh][s][0] = acc[mh][s][1] = acc[mh][s][2] = acc[mh][s][3] = 0.f; }
            }
            EpiAhead<MH> ahead;
            skinny_epilogue_fetch<T, EPI, 2, MH>(a, grp, threadIdx.x, ahead);
            for (int sl = 0; sl < nslab; ++sl) {
                if (ok && !dme::wait(&full_bar[stage], phase, status)) ok = false;
                const int c0 = sl * slab, cols = min(slab, K - c0);
                const int nblk = (cols + 63) / 64;
                const unsigned char* st = stages + size_t(stage) * stage_bytes;
                if (ok && cols % (64 * kSkinnyWarps) == 0) {
                    // whole blocks for every warp (the usual stage): nb blocks each, taken BB at a time with every
                    // shared-memory load of the batch issued before its first MMA
                    constexpr int BB = 4 / MH;
                    const int nb = cols / (64 * kSkinnyWarps);
                    const unsigned char* wrow_a = st + size_t(g) * rowb + t4 * 32;
                    const unsigned char* wrow_b = st + size_t(g + 8) * rowb + t4 * 32;
                    for (int b0 = 0; b0 < nb; b0 += BB) {                         // warp-uniform
                        uint4 wv[BB][4], xv[BB][MH][2];
                        #pragma unroll
                        for (int b = 0; b < BB; ++b) {
                            const int blk = warp + kSkinnyWarps * min(b0 + b, nb - 1);
                            const uint4* pa = reinterpret_cast<const uint4*>(wrow_a + blk * 128);
                            const uint4* pb = reinterpret_cast<const uint4*>(wrow_b + blk * 128);
                            wv[b][0] = pa[0]; wv[b][1] = pa[1]; wv[b][2] = pb[0]; wv[b][3] = pb[1];
                            #pragma unroll
                            for (int mh = 0; mh < MH; ++mh) {
                                xv[b][mh][0] = xv[b][mh][1] = make_uint4(0u, 0u, 0u, 0u);
                                if (g + 8 * mh < Mp) {
                                    const uint4* xp = reinterpret_cast<const uint4*>(xrow + size_t(8 * mh) * xstride + c0 + blk * 64);
                                    xv[b][mh][0] = xp[0]; xv[b][mh][1] = xp[1];
                                }
                            }
                        }
                        #pragma unroll
                        for (int b = 0; b < BB; ++b) {
                            if (b0 + b < nb) {
                                const uint32_t wA[8] = {wv[b][0].x, wv[b][0].y, wv[b][0].z, wv[b][0].w, wv[b][1].x, wv[b][1].y, wv[b][1].z, wv[b][1].w};
                                const uint32_t wB[8] = {wv[b][2].x, wv[b][2].y, wv[b][2].z, wv[b][2].w, wv[b][3].x, wv[b][3].y, wv[b][3].z, wv[b][3].w};
                                #pragma unroll
                                for (int mh = 0; mh < MH; ++mh) {
                                    const uint32_t xw[8] = {xv[b][mh][0].x, xv[b][mh][0].y, xv[b][mh][0].z, xv[b][mh][0].w,
                                                            xv[b][mh][1].x, xv[b][mh][1].y, xv[b][mh][1].z, xv[b][mh][1].w};
                                    #pragma unroll
                                    for (int s = 0; s < 4; ++s) {
                                        const uint32_t af[4] = {wA[2 * s], wB[2 * s], wA[2 * s + 1], wB[2 * s + 1]};
                                        mma_16816<T>(acc[mh][s], af, xw[2 * s], xw[2 * s + 1]);
                                    }
                                }
                            }
                        }
                    }
                } else if (ok) {
                    for (int blk = warp; blk < nblk; blk += kSkinnyWarps) {       // warp-uniform
                        const bool live = blk * 64 + t4 * 16 < cols;
                        uint4 wa0 = make_uint4(0u, 0u, 0u, 0u), wa1 = wa0, wb0 = wa0, wb1 = wa0;
                        if (live) {
                            const uint4* pa = reinterpret_cast<const uint4*>(st + size_t(g) * rowb + (blk * 64 + t4 * 16) * 2);
                            const uint4* pb = reinterpret_cast<const uint4*>(st + size_t(g + 8) * rowb + (blk * 64 + t4 * 16) * 2);
                            wa0 = pa[0]; wa1 = pa[1]; wb0 = pb[0]; wb1 = pb[1];
                        }
                        const uint32_t wA[8] = {wa0.x, wa0.y, wa0.z, wa0.w, wa1.x, wa1.y, wa1.z, wa1.w};
                        const uint32_t wB[8] = {wb0.x, wb0.y, wb0.z, wb0.w, wb1.x, wb1.y, wb1.z, wb1.w};
                        #pragma unroll
                        for (int mh = 0; mh < MH; ++mh) {
                            uint4 xa = make_uint4(0u, 0u, 0u, 0u), xb = xa;
                            if (live && g + 8 * mh < Mp) {
                                const uint4* xp = reinterpret_cast<const uint4*>(xrow + size_t(8 * mh) * xstride + c0 + blk * 64);
                                xa = xp[0]; xb = xp[1];
                            }
                            const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
                            #pragma unroll
                            for (int s = 0; s < 4; ++s) {
                                const uint32_t af[4] = {wA[2 * s], wB[2 * s], wA[2 * s + 1], wB[2 * s + 1]};
                                mma_16816<T>(acc[mh][s], af, xw[2 * s], xw[2 * s + 1]);
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) dme::mbar_arrive(&empty_bar[stage]);
                if (++stage == nstages) { stage = 0; phase ^= 1u; }
            }
            #pragma unroll
            for (int mh = 0; mh < MH; ++mh)
                *reinterpret_cast<float4*>(&red[parity][warp][lane][4 * mh]) =
                    make_float4((acc[mh][0][0] + acc[mh][1][0]) + (acc[mh][2][0] + acc[mh][3][0]), (acc[mh][0][1] + acc[mh][1][1]) + (acc[mh][2][1] + acc[mh][3][1]),
                                (acc[mh][0][2] + acc[mh][1][2]) + (acc[mh][2][2] + acc[mh][3][2]), (acc[mh][0][3] + acc[mh][1][3]) + (acc[mh][2][3] + acc[mh][3][3]));
            skinny_barrier();
            skinny_epilogue<T, EPI, 2, MH>(a, red[parity], grp, threadIdx.x, false, 0.f, nullptr, &ahead);
        }
        if (!ok && lane == 0) atomicExch(sticky, 1);
    }
}

// Launch: returns B200P_E_RANGE when the shape is outside the kernel's domain (the caller then
// takes the library GEMM).  K must be a multiple of 16 (32-byte steps along the rows of W and X),
// ldx of 8, W 32-byte aligned.
template <typename T, int PRO, int EPI, int MH>
int launch_skinny_mh(const SkinnyArgs& a, cudaStream_t st);

// Up to 8 rows of X: one B fragment per A fragment; 9 .. 16 rows: two.
template <typename T, int PRO, int EPI>
int launch_skinny(const SkinnyArgs& a, cudaStream_t st) {
    return a.M <= 8 ? launch_skinny_mh<T, PRO, EPI, 1>(a, st) : launch_skinny_mh<T, PRO, EPI, 2>(a, st);
}

template <typename T, int PRO, int EPI, int MH>
int launch_skinny_mh(const SkinnyArgs& a, cudaStream_t st) {
    if (a.M < 1 || a.M > kSkinnyMaxM || a.K < 16 || a.K % 16 != 0 || a.N < 1) return B200P_E_RANGE;
    if (PRO == PRO_PLAIN && (a.ldx % 8 != 0 || !aligned(a.X16, 16))) return B200P_E_RANGE;
    if (PRO == PRO_RMSNORM && (!aligned(a.X32, 16) || !aligned(a.norm_w, 8))) return B200P_E_RANGE;
    if (!aligned(a.W, 16)) return B200P_E_RANGE;               // bulk copies need 16 bytes; the register kernel's 32-byte loads are checked below
    const int Mp = a.M <= 1 ? 1 : a.M <= 2 ? 2 : a.M <= 4 ? 4 : a.M <= 8 ? 8 : 16;
    const size_t smem = size_t(Mp) * (a.K + kSkinnyXPad) * 2;
    if (smem > 190 * 1024) return B200P_E_RANGE;
    if (EPI == EPI_ROPE && (a.rope.D % 16 != 0 || a.N != (a.rope.nQH + 2 * a.rope.nKVH) * a.rope.D)) return B200P_E_RANGE;
    const int sms = sm_count() > 0 ? sm_count() : 148;
    constexpr bool paired = EPI == EPI_SILU16 || EPI == EPI_ROPE;
    const bool pdl = tuning(KNOB_RUNTIME_PDL, 1) != 0;
    if (tuning(KNOB_RUNTIME_SKINNY, 2) == 2 && aligned(a.W, 16)) {
        // W staged through shared memory by a producer thread (skinny_stream_kernel), one CTA per SM
        const int slab_cols = kSkinnySlab;                               // measured: 0.67 ms per token at 2048, 0.72 at 1024, 0.73 at 4096
        const int slab = a.K < slab_cols ? a.K : slab_cols;
        const int stage_bytes = 16 * (slab * 2 + 16);
        const int x_bytes = int((smem + 127) / 128 * 128);
        int nstages = (224000 - 8192 * (MH - 1) - x_bytes) / stage_bytes;
        if (nstages > 8) nstages = 8;
        // A few more row groups than SMs (the decode step's Q/K/V: 160 on 148), each one stage long: with one CTA per
        // SM a dozen CTAs would take two groups one after the other and the whole grid would wait for them.  One CTA
        // per group with a single stage instead: two of them fit an SM and run side by side.
        const int groups_all = EPI == EPI_SILU16 ? (a.N + 7) / 8 : (a.N + 15) / 16;
        // (the two-fragment kernel holds too many registers for two CTAs of 288 threads on an SM)
        const bool one_group_ctas = MH == 1 && groups_all > sms && groups_all <= 2 * sms && a.K <= slab_cols &&
                                    x_bytes + stage_bytes + 8704 * MH + 1024 <= 113 * 1024 && nstages >= 2;
        if (one_group_ctas) nstages = 1;
        int* sticky = device_status_ptr();
        int* status = a.abort_word;
        if ((nstages >= 2 || one_group_ctas) && sticky && !status) {               // no caller-owned abort word: this launch's own slot
            LaunchSlot slot{};
            if (int se = take_launch_slot(st, &slot)) return se;
            status = slot.abort;
        }
        if ((nstages >= 2 || one_group_ctas) && sticky) {
            const int groups = groups_all;
            const size_t dyn = size_t(x_bytes) + size_t(nstages) * stage_bytes;
            void (*sk)(SkinnyArgs, int, int, int*, int*) = skinny_stream_kernel<T, PRO, EPI, MH>;
            const cudaError_t ae = cudaFuncSetAttribute(sk, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dyn));
            if (ae != cudaSuccess) return int(ae);
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(groups < sms || one_group_ctas ? groups : sms); cfg.blockDim = dim3(kSkinnyStreamThreads); cfg.dynamicSmemBytes = dyn; cfg.stream = st;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
            const cudaError_t le = cudaLaunchKernelEx(&cfg, sk, a, nstages, slab_cols, status, sticky);
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return le == cudaSuccess ? B200P_OK : int(le);
        }
    }
    if (!aligned(a.W, 32)) return B200P_E_RANGE;               // the register kernel loads 32-byte vectors of W
    // 8-row groups when 16-row groups would leave a third of the CTA slots (2 per SM) empty
    const bool half_rows = !paired && (a.N + 15) / 16 < (4 * sms) / 3;
    const int ngroups = EPI == EPI_SILU16 ? (a.N + 7) / 8 : half_rows ? (a.N + 7) / 8 : (a.N + 15) / 16;
    const int grid = ngroups < 2 * sms ? ngroups : 2 * sms;      // CTAs loop over their groups, loads running ahead
    void (*kern)(SkinnyArgs) = skinny_gemm_kernel<T, PRO, EPI, 2, MH>;
    if constexpr (!paired) { if (half_rows) kern = skinny_gemm_kernel<T, PRO, EPI, 1, MH>; }
    if (smem > 28 * 1024) {                                     // static (8 or 16 KB) + dynamic beyond 48 KB needs the opt-in
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return int(e);
    }
    // Launched as a programmatic dependent: the CTAs may start while the previous kernel of the
    // stream is still draining, fetch their weights, and wait at griddep_wait() for its results.
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kSkinnyThreads); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, kern, a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return le == cudaSuccess ? B200P_OK : int(le);
}

} // namespace b200p
