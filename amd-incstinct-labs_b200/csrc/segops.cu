// ---------------------------------------------------------------------------
// segops.cu -- segmented wave64 reduce / scan over arrays in HBM.
//
// Array-level form of the reference's wave::dpp::reduce_* / scan_* device
// functions (research/wave-primitives/include/wave_primitives/
// wave_reduce_dpp.hpp:106-113, wave_scan_dpp.hpp:70-87) and of its
// fp32-accumulating 16-bit overloads (wave_reduce.hpp:48-119,
// wave_scan.hpp:52-74): every run of 64 consecutive elements is one wave.
//
// Both kernels are pure streaming kernels bound by HBM bandwidth:
//   reduce: reads n*sizeof(T), writes n/64 results;
//   scan  : reads n*sizeof(T), writes n*sizeof(T).
// A lane loads one 16- or 32-byte vector (VEC consecutive elements), so a
// segment occupies 64/VEC adjacent lanes and a warp holds several segments.
// All cross-lane traffic is shuffles / redux.sync; no shared memory is used.
// Each warp keeps U independent vector loads in flight before the first
// shuffle.  The kernels stride over warp tiles, so any grid works; measured on
// B200 a grid of one tile per warp (the hardware CTA scheduler balances the
// tail) is 2-5% faster than a resident grid of 148 x 8 CTAs, and is the default
// (knob seg_ctas_per_sm caps the grid at that many CTAs per SM).
// ---------------------------------------------------------------------------
#include "common.cuh"
#include "vec_io.cuh"
#include "wave_primitives/wave64.cuh"

namespace b200p {
namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerCta = kThreads / 32;

// --- word <-> element codecs -------------------------------------------------
// S: storage type in memory, A: type the arithmetic runs in.
template <typename S> struct Codec;

template <> struct Codec<float> {
    using acc_t = float;
    template <int W> static __device__ __forceinline__ void unpack(const uint32_t (&w)[W], float (&v)[W]) {
        #pragma unroll
        for (int i = 0; i < W; ++i) v[i] = __uint_as_float(w[i]);
    }
    template <int W> static __device__ __forceinline__ void pack(const float (&v)[W], uint32_t (&w)[W]) {
        #pragma unroll
        for (int i = 0; i < W; ++i) w[i] = __float_as_uint(v[i]);
    }
};
template <> struct Codec<int> {
    using acc_t = int;
    template <int W> static __device__ __forceinline__ void unpack(const uint32_t (&w)[W], int (&v)[W]) {
        #pragma unroll
        for (int i = 0; i < W; ++i) v[i] = int(w[i]);
    }
    template <int W> static __device__ __forceinline__ void pack(const int (&v)[W], uint32_t (&w)[W]) {
        #pragma unroll
        for (int i = 0; i < W; ++i) w[i] = uint32_t(v[i]);
    }
};
template <> struct Codec<double> {
    using acc_t = double;
    template <int W> static __device__ __forceinline__ void unpack(const uint32_t (&w)[W], double (&v)[W / 2]) {
        #pragma unroll
        for (int i = 0; i < W / 2; ++i) v[i] = __hiloint2double(int(w[2 * i + 1]), int(w[2 * i]));
    }
    template <int W> static __device__ __forceinline__ void pack(const double (&v)[W / 2], uint32_t (&w)[W]) {
        #pragma unroll
        for (int i = 0; i < W / 2; ++i) { w[2 * i] = uint32_t(__double2loint(v[i])); w[2 * i + 1] = uint32_t(__double2hiint(v[i])); }
    }
};
template <> struct Codec<long long> {
    using acc_t = long long;
    template <int W> static __device__ __forceinline__ void unpack(const uint32_t (&w)[W], long long (&v)[W / 2]) {
        #pragma unroll
        for (int i = 0; i < W / 2; ++i) v[i] = (long long)(((unsigned long long)w[2 * i + 1] << 32) | w[2 * i]);
    }
    template <int W> static __device__ __forceinline__ void pack(const long long (&v)[W / 2], uint32_t (&w)[W]) {
        #pragma unroll
        for (int i = 0; i < W / 2; ++i) { w[2 * i] = uint32_t((unsigned long long)v[i]); w[2 * i + 1] = uint32_t((unsigned long long)v[i] >> 32); }
    }
};
template <> struct Codec<__half> {
    using acc_t = float;
    template <int W> static __device__ __forceinline__ void unpack(const uint32_t (&w)[W], float (&v)[2 * W]) {
        #pragma unroll
        for (int i = 0; i < W; ++i) {
            __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
            float2 f = __half22float2(h);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
    template <int W> static __device__ __forceinline__ void pack(const float (&v)[2 * W], uint32_t (&w)[W]) {
        #pragma unroll
        for (int i = 0; i < W; ++i) {
            __half2 h = __halves2half2(__float2half_rn(v[2 * i]), __float2half_rn(v[2 * i + 1]));
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
    static __device__ __forceinline__ __half narrow(float f) { return __float2half_rn(f); }
};
template <> struct Codec<__nv_bfloat16> {
    using acc_t = float;
    template <int W> static __device__ __forceinline__ void unpack(const uint32_t (&w)[W], float (&v)[2 * W]) {
        #pragma unroll
        for (int i = 0; i < W; ++i) {           // bf16 -> f32 is a 16-bit shift
            v[2 * i]     = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    template <int W> static __device__ __forceinline__ void pack(const float (&v)[2 * W], uint32_t (&w)[W]) {
        #pragma unroll
        for (int i = 0; i < W; ++i) {
            __nv_bfloat162 h = __halves2bfloat162(__float2bfloat16_rn(v[2 * i]), __float2bfloat16_rn(v[2 * i + 1]));
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
    static __device__ __forceinline__ __nv_bfloat16 narrow(float f) { return __float2bfloat16_rn(f); }
};

template <typename S, int BYTES> struct Shape {
    static constexpr int VEC = BYTES / int(sizeof(S));      // elements per lane vector
    static constexpr int LPS = wave::kSegment / VEC;        // lanes per segment
    static constexpr int G   = 32 / LPS;                    // segments per warp load
};

// ---------------------------------------------------------------------------
// Reduce.  Warp tile = U loads; lane group g handles the U consecutive
// segments tile*G*U + g*U + j (j = 0..U-1), so its U results are adjacent in
// `out` and are written by the group's first U lanes.
// O is the stored result type: acc_t, or the narrow input type.
// ---------------------------------------------------------------------------
template <typename S, typename O, typename Op, int BYTES, int U>
__global__ void __launch_bounds__(kThreads)
segreduce_kernel(const S* __restrict__ in, O* __restrict__ out, size_t nseg) {
    using C = Codec<S>;
    using A = typename C::acc_t;
    using Sh = Shape<S, BYTES>;
    constexpr int VEC = Sh::VEC, LPS = Sh::LPS, G = Sh::G, W = BYTES / 4;
    static_assert(U <= LPS, "one output lane per segment of the tile");

    const unsigned lane = wave::lane_id();
    const unsigned g = lane / LPS, q = lane % LPS;
    const size_t warp  = size_t(blockIdx.x) * kWarpsPerCta + threadIdx.x / 32;
    const size_t nwarp = size_t(gridDim.x) * kWarpsPerCta;
    const size_t ntile = (nseg + size_t(G * U) - 1) / size_t(G * U);
    const char* base = reinterpret_cast<const char*>(in);
    const Op op{};
    const A ident = Op::template identity<A>();

    for (size_t tile = warp; tile < ntile; tile += nwarp) {
        const size_t seg0 = tile * size_t(G * U) + size_t(g) * U;
        uint32_t w[U][W];
        #pragma unroll
        for (int j = 0; j < U; ++j) {
            if (seg0 + j < nseg) {
                VecIO<BYTES>::load(base + ((seg0 + j) * LPS + q) * size_t(BYTES), w[j]);
            }
        }
        A mine = ident;
        #pragma unroll
        for (int j = 0; j < U; ++j) {
            A v[VEC];
            if (seg0 + j < nseg) {
                C::unpack(w[j], v);
            } else {
                #pragma unroll
                for (int i = 0; i < VEC; ++i) v[i] = ident;
            }
            const A r = wave::segment_reduce<VEC>(v, op);
            if (q == unsigned(j)) mine = r;
        }
        if (q < unsigned(U) && seg0 + q < nseg) {
            if constexpr (std::is_same<O, A>::value) out[seg0 + q] = mine;
            else                                      out[seg0 + q] = C::narrow(mine);
        }
    }
}

// ---------------------------------------------------------------------------
// Scan.  Lane vectors are taken in plain order: warp tile = U*32 consecutive
// lane vectors, results stored in place of the inputs' positions.
// MODE 0: reference full-DPP association (rows of 16 + carries), fp32/fp64;
// MODE 1: fast (any association), integers;
// MODE 2: Kogge-Stone over the whole 64 in fp32, 16-bit inputs;
// EXCL : shift the inclusive result right by one (exclusive sum).
// ---------------------------------------------------------------------------
template <typename S, typename Op, int BYTES, int U, int MODE, bool EXCL>
__global__ void __launch_bounds__(kThreads)
segscan_kernel(const S* __restrict__ in, S* __restrict__ out, size_t nvec) {
    using C = Codec<S>;
    using A = typename C::acc_t;
    constexpr int VEC = Shape<S, BYTES>::VEC, W = BYTES / 4;

    const unsigned lane = wave::lane_id();
    const size_t warp  = size_t(blockIdx.x) * kWarpsPerCta + threadIdx.x / 32;
    const size_t nwarp = size_t(gridDim.x) * kWarpsPerCta;
    const size_t ntile = (nvec + size_t(32 * U) - 1) / size_t(32 * U);
    const char* src = reinterpret_cast<const char*>(in);
    char* dst = reinterpret_cast<char*>(out);
    const Op op{};
    const A ident = Op::template identity<A>();

    for (size_t tile = warp; tile < ntile; tile += nwarp) {
        const size_t v0 = tile * size_t(32 * U) + lane;
        uint32_t w[U][W];
        #pragma unroll
        for (int j = 0; j < U; ++j) {
            if (v0 + size_t(j) * 32 < nvec) VecIO<BYTES>::load(src + (v0 + size_t(j) * 32) * BYTES, w[j]);
        }
        #pragma unroll
        for (int j = 0; j < U; ++j) {
            const bool live = v0 + size_t(j) * 32 < nvec;   // whole segments are live or not
            A v[VEC];
            if (live) {
                C::unpack(w[j], v);
            } else {
                #pragma unroll
                for (int i = 0; i < VEC; ++i) v[i] = ident;
            }
            if constexpr (MODE == 0)      wave::segment_scan_dpp_order<VEC>(v, op, ident);
            else if constexpr (MODE == 1) wave::segment_scan_fast<VEC>(v, op, ident);
            else                          wave::row_scan_kogge_stone<VEC, 64>(v, op, ident);
            if constexpr (EXCL) wave::segment_shift_right<VEC>(v, A(0));
            if (live) {
                uint32_t r[W];
                C::pack(v, r);
                VecIO<BYTES>::store(dst + (v0 + size_t(j) * 32) * BYTES, r);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Packed fp32 pairs.  sm_100a adds two independent fp32 lanes with one instruction
// (add.rn.f32x2, each half rounded to nearest exactly like a scalar add), which
// halves the issue slots of the in-register trees below for sums.
// ---------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
// Inclusive Kogge-Stone sum scan of 64 floats held by one lane, bit for bit wave::lane_scan_kogge_stone<64>:
// the offset-1 step on scalars, the offsets 2 .. 32 on pairs (v[i], v[i+1]) += (v[i-o], v[i-o+1]).
__device__ __forceinline__ void lane_scan64_sum_packed(float (&v)[64]) {
    #pragma unroll
    for (int i = 63; i >= 1; --i) v[i] = v[i] + v[i - 1];
    unsigned long long p[32];
    #pragma unroll
    for (int k = 0; k < 32; ++k) p[k] = pack_f32x2(v[2 * k], v[2 * k + 1]);
    #pragma unroll
    for (int o = 1; o < 32; o <<= 1) {                       // o pairs = 2 o elements
        #pragma unroll
        for (int k = 31; k >= o; --k) p[k] = add_f32x2(p[k], p[k - o]);
    }
    #pragma unroll
    for (int k = 0; k < 32; ++k) unpack_f32x2(p[k], v[2 * k], v[2 * k + 1]);
}
// The reference's portable reduction tree (elements i and i + 32 first, ...) over 64 floats held by one lane,
// bit for bit wave::lane_reduce_shfl_down_order<64>: five packed levels, then two scalar adds.
__device__ __forceinline__ float lane_reduce64_sum_packed(const float (&v)[64]) {
    unsigned long long p[32];
    #pragma unroll
    for (int k = 0; k < 32; ++k) p[k] = pack_f32x2(v[2 * k], v[2 * k + 1]);
    #pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {                      // element offsets 32, 16, 8, 4, 2
        #pragma unroll
        for (int k = 0; k < o; ++k) p[k] = add_f32x2(p[k], p[k + o]);
    }
    float lo, hi;
    unpack_f32x2(p[0], lo, hi);
    return lo + hi;                                          // element offset 1
}

// ---------------------------------------------------------------------------
// Scan of 16-bit inputs, one whole segment per lane.  The fp32 Kogge-Stone order
// the 16-bit overloads prescribe costs 47 shuffles per 32 bytes when a segment is
// spread over four lanes, which makes that form issue-bound; a lane that holds all
// 64 values of its segment (128 bytes, four 32-byte or eight 16-byte vectors) runs
// the same dataflow with no cross-lane traffic.  Lanes of a warp read adjacent
// 128-byte lines, every sector exactly once.
// ---------------------------------------------------------------------------
template <typename S, typename Op, int BYTES>
__global__ void __launch_bounds__(kThreads)
segscan_lane_kernel(const S* __restrict__ in, S* __restrict__ out, size_t nseg) {
    using C = Codec<S>;
    static_assert(sizeof(S) == 2, "16-bit storage");
    constexpr int W = BYTES / 4, NV = 128 / BYTES, EPV = BYTES / 2;
    const char* src = reinterpret_cast<const char*>(in);
    char* dst = reinterpret_cast<char*>(out);
    const Op op{};
    const size_t stride = size_t(gridDim.x) * kThreads;
    for (size_t seg = size_t(blockIdx.x) * kThreads + threadIdx.x; seg < nseg; seg += stride) {
        uint32_t w[NV][W];
        #pragma unroll
        for (int j = 0; j < NV; ++j) VecIO<BYTES>::load(src + seg * 128 + size_t(j) * BYTES, w[j]);
        float v[64];
        #pragma unroll
        for (int j = 0; j < NV; ++j) {
            float t[EPV];
            C::unpack(w[j], t);
            #pragma unroll
            for (int i = 0; i < EPV; ++i) v[j * EPV + i] = t[i];
        }
        if constexpr (std::is_same<Op, wave::SumOp>::value) lane_scan64_sum_packed(v);
        else                                                wave::lane_scan_kogge_stone<64>(v, op);
        #pragma unroll
        for (int j = 0; j < NV; ++j) {
            float t[EPV];
            #pragma unroll
            for (int i = 0; i < EPV; ++i) t[i] = v[j * EPV + i];
            uint32_t r[W];
            C::pack(t, r);
            VecIO<BYTES>::store(dst + seg * 128 + size_t(j) * BYTES, r);
        }
    }
}

// ---------------------------------------------------------------------------
// Sum of 16-bit inputs, one whole segment per lane, in the association the
// reference's 16-bit overloads prescribe: fp32, elements (i, i + 32) first, then
// (i, i + 16), ... (the shfl_down loop of wave_reduce.hpp:48-63).  With the
// segment in one lane's registers that tree costs 63 adds and no shuffle, so the
// result agrees with the reference bit for bit at streaming speed.  A warp reads
// 32 adjacent 128-byte lines and writes 32 adjacent results.
// ---------------------------------------------------------------------------
template <typename S, typename O, typename Op, int BYTES>
__global__ void __launch_bounds__(kThreads)
segreduce_lane_kernel(const S* __restrict__ in, O* __restrict__ out, size_t nseg) {
    using C = Codec<S>;
    static_assert(sizeof(S) == 2, "16-bit storage");
    constexpr int W = BYTES / 4, NV = 128 / BYTES, EPV = BYTES / 2;
    const char* src = reinterpret_cast<const char*>(in);
    const Op op{};
    const size_t stride = size_t(gridDim.x) * kThreads;
    for (size_t seg = size_t(blockIdx.x) * kThreads + threadIdx.x; seg < nseg; seg += stride) {
        uint32_t w[NV][W];
        #pragma unroll
        for (int j = 0; j < NV; ++j) VecIO<BYTES>::load(src + seg * 128 + size_t(j) * BYTES, w[j]);
        float v[64];
        #pragma unroll
        for (int j = 0; j < NV; ++j) {
            float t[EPV];
            C::unpack(w[j], t);
            #pragma unroll
            for (int i = 0; i < EPV; ++i) v[j * EPV + i] = t[i];
        }
        float r;
        if constexpr (std::is_same<Op, wave::SumOp>::value) r = lane_reduce64_sum_packed(v);
        else                                                r = wave::lane_reduce_shfl_down_order<64>(v, op);
        if constexpr (std::is_same<O, float>::value) out[seg] = r;
        else                                          out[seg] = C::narrow(r);
    }
}

// --- single-wave probe through the public pair-per-lane API ----------------------
template <typename T>
__global__ void wave_probe_kernel(int fn, int op, const T* in, T* out, int nwaves) {
    const int wave_i = int(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32;
    if (wave_i >= nwaves) return;                              // whole warps leave together
    in += size_t(wave_i) * 64; out += size_t(wave_i) * 64;
    const unsigned l = threadIdx.x % 32;
    T a = in[2 * l], b = in[2 * l + 1];
    if (fn == 0) {
        T r;
        if (op == B200P_SUM)      r = wave::dpp::reduce_sum_bcast(a, b);
        else if (op == B200P_MAX) r = wave::dpp::reduce_max_bcast(a, b);
        else                      r = wave::dpp::reduce_min_bcast(a, b);
        out[2 * l] = r; out[2 * l + 1] = r;
    } else {
        if (fn == 2)              wave::dpp::scan_exclusive_sum(a, b);
        else if (op == B200P_SUM) wave::dpp::scan_inclusive_sum(a, b);
        else if (op == B200P_MAX) wave::dpp::scan_inclusive_max(a, b);
        else                      wave::dpp::scan_inclusive_min(a, b);
        out[2 * l] = a; out[2 * l + 1] = b;
    }
}
template <typename N>
__global__ void wave_probe_narrow_kernel(int fn, int op, const N* in, N* out, int nwaves) {
    const int wave_i = int(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32;
    if (wave_i >= nwaves) return;
    in += size_t(wave_i) * 64; out += size_t(wave_i) * 64;
    const unsigned l = threadIdx.x % 32;
    N a = in[2 * l], b = in[2 * l + 1];
    if (fn == 0) {
        N r;
        if (op == B200P_SUM)      r = wave::reduce_sum(a, b);
        else if (op == B200P_MAX) r = wave::reduce_max(a, b);
        else                      r = wave::reduce_min(a, b);
        out[2 * l] = r; out[2 * l + 1] = r;
    } else {
        wave::scan_inclusive_sum(a, b);
        out[2 * l] = a; out[2 * l + 1] = b;
    }
}
// Vote / bitwise wrappers on one wave: in[64] ints -> out[0..7] (see b200p_wave_vote_probe).
__global__ void wave_vote_probe_kernel(const int* in, unsigned long long* out) {
    const unsigned l = threadIdx.x % 32;
    const int a = in[2 * l], b = in[2 * l + 1];
    const unsigned long long bal = wave::ballot(a > 0, b > 0);
    const int any_ = wave::any(a > 0, b > 0), all_ = wave::all(a > 0, b > 0), pc = wave::popcount(a > 0, b > 0);
    const unsigned ra = wave::reduce_and(unsigned(a), unsigned(b)), ro = wave::reduce_or(unsigned(a), unsigned(b));
    const unsigned long long b32 = wave::ballot(a > 0);
    if (l == 5) {
        out[0] = bal; out[1] = (unsigned long long)any_; out[2] = (unsigned long long)all_; out[3] = (unsigned long long)pc;
        out[4] = ra; out[5] = ro; out[6] = b32; out[7] = wave::lane_mask_lt();
    }
}

// --- launch helpers ------------------------------------------------------------
int grid_for(size_t ntile_warps) {
    const int sms = sm_count();
    const int per_sm = tuning(KNOB_SEG_CTAS_PER_SM, 1 << 20);   // measured: one tile per warp beats a resident grid
    size_t ctas = (ntile_warps + kWarpsPerCta - 1) / kWarpsPerCta;
    size_t cap = size_t(sms) * size_t(per_sm);
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    return int(ctas);
}

template <typename S, typename O, typename Op, int BYTES>
int launch_reduce(const void* in, void* out, size_t n, cudaStream_t st) {
    constexpr int U = 4;
    using Sh = Shape<S, BYTES>;
    const size_t nseg = n / 64;
    const size_t ntile = (nseg + size_t(Sh::G * U) - 1) / size_t(Sh::G * U);
    segreduce_kernel<S, O, Op, BYTES, U><<<grid_for(ntile), kThreads, 0, st>>>(
        static_cast<const S*>(in), static_cast<O*>(out), nseg);
    return launched();
}
template <typename S, typename O, int BYTES>
int reduce_op(int op, const void* in, void* out, size_t n, cudaStream_t st) {
    switch (op) {
        case B200P_SUM: return launch_reduce<S, O, wave::SumOp, BYTES>(in, out, n, st);
        case B200P_MAX: return launch_reduce<S, O, wave::MaxOp, BYTES>(in, out, n, st);
        case B200P_MIN: return launch_reduce<S, O, wave::MinOp, BYTES>(in, out, n, st);
    }
    return B200P_E_OP;
}
template <typename S, typename O>
int reduce_bytes(int op, const void* in, void* out, size_t n, cudaStream_t st) {
    const bool wide = tuning(KNOB_SEG_VEC_BYTES, 32) == 32 && aligned(in, 32);
    if constexpr (sizeof(S) == 2) {
        // 16-bit sum: the reference's fp32 shfl_down association, a whole segment per lane
        if (op == B200P_SUM) {
            const size_t nseg = n / 64;
            const int grid = grid_for((nseg + 31) / 32);
            if (wide) segreduce_lane_kernel<S, O, wave::SumOp, 32><<<grid, kThreads, 0, st>>>(static_cast<const S*>(in), static_cast<O*>(out), nseg);
            else      segreduce_lane_kernel<S, O, wave::SumOp, 16><<<grid, kThreads, 0, st>>>(static_cast<const S*>(in), static_cast<O*>(out), nseg);
            return launched();
        }
    }
    return wide ? reduce_op<S, O, 32>(op, in, out, n, st) : reduce_op<S, O, 16>(op, in, out, n, st);
}

template <typename S, typename Op, int BYTES, int MODE, bool EXCL>
int launch_scan(const void* in, void* out, size_t n, cudaStream_t st) {
    constexpr int U = (BYTES == 32) ? 2 : 4;
    const size_t nvec = n * sizeof(S) / BYTES;
    const size_t ntile = (nvec + size_t(32 * U) - 1) / size_t(32 * U);
    segscan_kernel<S, Op, BYTES, U, MODE, EXCL><<<grid_for(ntile), kThreads, 0, st>>>(
        static_cast<const S*>(in), static_cast<S*>(out), nvec);
    return launched();
}
template <typename S, int BYTES, int MODE, bool EXCL>
int scan_op(int op, const void* in, void* out, size_t n, cudaStream_t st) {
    switch (op) {
        case B200P_SUM: return launch_scan<S, wave::SumOp, BYTES, MODE, EXCL>(in, out, n, st);
        case B200P_MAX: if constexpr (!EXCL) return launch_scan<S, wave::MaxOp, BYTES, MODE, false>(in, out, n, st); else break;
        case B200P_MIN: if constexpr (!EXCL) return launch_scan<S, wave::MinOp, BYTES, MODE, false>(in, out, n, st); else break;
    }
    return B200P_E_OP;
}
template <typename S, typename Op>
int launch_scan_lane(const void* in, void* out, size_t n, cudaStream_t st) {
    const size_t nseg = n / 64;
    const bool wide = tuning(KNOB_SEG_VEC_BYTES, 32) == 32 && aligned(in, 32) && aligned(out, 32);
    const int grid = grid_for((nseg + 31) / 32);
    if (wide) segscan_lane_kernel<S, Op, 32><<<grid, kThreads, 0, st>>>(static_cast<const S*>(in), static_cast<S*>(out), nseg);
    else      segscan_lane_kernel<S, Op, 16><<<grid, kThreads, 0, st>>>(static_cast<const S*>(in), static_cast<S*>(out), nseg);
    return launched();
}
template <typename S, int MODE, bool EXCL>
int scan_bytes(int op, const void* in, void* out, size_t n, cudaStream_t st) {
    const bool wide = tuning(KNOB_SEG_VEC_BYTES, 32) == 32 && aligned(in, 32) && aligned(out, 32);
    return wide ? scan_op<S, 32, MODE, EXCL>(op, in, out, n, st) : scan_op<S, 16, MODE, EXCL>(op, in, out, n, st);
}
// 16-bit inclusive scans: one segment per lane (knob scan16_lane = 0 selects the
// four-lanes-per-segment shuffle form).
template <typename S>
int scan_narrow(int op, const void* in, void* out, size_t n, cudaStream_t st) {
    if (tuning(KNOB_SCAN16_LANE, 1) == 0) return scan_bytes<S, 2, false>(op, in, out, n, st);
    switch (op) {
        case B200P_SUM: return launch_scan_lane<S, wave::SumOp>(in, out, n, st);
        case B200P_MAX: return launch_scan_lane<S, wave::MaxOp>(in, out, n, st);
        case B200P_MIN: return launch_scan_lane<S, wave::MinOp>(in, out, n, st);
    }
    return B200P_E_OP;
}

template <typename S, bool EXCL>
int scan_fp(int op, const void* in, void* out, size_t n, cudaStream_t st) {
    return tuning(KNOB_SCAN_FP_EXACT, 1) ? scan_bytes<S, 0, EXCL>(op, in, out, n, st)
                                         : scan_bytes<S, 1, EXCL>(op, in, out, n, st);
}

int check_args(const void* in, const void* out, size_t n, int op) {
    if (op < B200P_SUM || op > B200P_MIN) return B200P_E_OP;
    if (n % 64 != 0) return B200P_E_LENGTH;
    if (n == 0) return B200P_OK;
    if (!in || !out) return B200P_E_NULL;
    if (!aligned(in, 16) || !aligned(out, 4)) return B200P_E_ALIGN;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    return B200P_OK;
}

} // namespace
} // namespace b200p

using namespace b200p;

extern "C" int b200p_segreduce(int op, int dtype, const void* in, void* out, size_t n, b200p_stream_t stream) {
    if (dtype < B200P_F32 || dtype > B200P_BF16) return B200P_E_DTYPE;
    if (int e = check_args(in, out, n, op)) return e;
    if (n == 0) return B200P_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case B200P_F32:  return reduce_bytes<float, float>(op, in, out, n, st);
        case B200P_F64:  return reduce_bytes<double, double>(op, in, out, n, st);
        case B200P_I32:  return reduce_bytes<int, int>(op, in, out, n, st);
        case B200P_I64:  return reduce_bytes<long long, long long>(op, in, out, n, st);
        case B200P_F16:  return reduce_bytes<__half, float>(op, in, out, n, st);
        case B200P_BF16: return reduce_bytes<__nv_bfloat16, float>(op, in, out, n, st);
    }
    return B200P_E_DTYPE;
}

extern "C" int b200p_segreduce_narrow(int op, int dtype, const void* in, void* out, size_t n, b200p_stream_t stream) {
    if (dtype != B200P_F16 && dtype != B200P_BF16) return B200P_E_DTYPE;
    if (int e = check_args(in, out, n, op)) return e;
    if (n == 0) return B200P_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == B200P_F16 ? reduce_bytes<__half, __half>(op, in, out, n, st)
                              : reduce_bytes<__nv_bfloat16, __nv_bfloat16>(op, in, out, n, st);
}

extern "C" int b200p_segscan_inclusive(int op, int dtype, const void* in, void* out, size_t n, b200p_stream_t stream) {
    if (dtype < B200P_F32 || dtype > B200P_BF16) return B200P_E_DTYPE;
    if (int e = check_args(in, out, n, op)) return e;
    if (n == 0) return B200P_OK;
    if (!aligned(out, 16)) return B200P_E_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case B200P_F32:  return scan_fp<float, false>(op, in, out, n, st);
        case B200P_F64:  return scan_fp<double, false>(op, in, out, n, st);
        case B200P_I32:  return scan_bytes<int, 1, false>(op, in, out, n, st);
        case B200P_I64:  return scan_bytes<long long, 1, false>(op, in, out, n, st);
        case B200P_F16:  return scan_narrow<__half>(op, in, out, n, st);
        case B200P_BF16: return scan_narrow<__nv_bfloat16>(op, in, out, n, st);
    }
    return B200P_E_DTYPE;
}

extern "C" int b200p_segscan_exclusive_sum(int dtype, const void* in, void* out, size_t n, b200p_stream_t stream) {
    if (dtype < B200P_F32 || dtype > B200P_I64) return B200P_E_DTYPE;
    if (int e = check_args(in, out, n, B200P_SUM)) return e;
    if (n == 0) return B200P_OK;
    if (!aligned(out, 16)) return B200P_E_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case B200P_F32:  return scan_fp<float, true>(B200P_SUM, in, out, n, st);
        case B200P_F64:  return scan_fp<double, true>(B200P_SUM, in, out, n, st);
        case B200P_I32:  return scan_bytes<int, 1, true>(B200P_SUM, in, out, n, st);
        case B200P_I64:  return scan_bytes<long long, 1, true>(B200P_SUM, in, out, n, st);
    }
    return B200P_E_DTYPE;
}

extern "C" int b200p_wave_probe_n(int fn, int op, int dtype, const void* in, void* out, int n_waves, b200p_stream_t stream) {
    if (fn < 0 || fn > 2) return B200P_E_OP;
    if (op < B200P_SUM || op > B200P_MIN) return B200P_E_OP;
    if (dtype < B200P_F32 || dtype > B200P_BF16) return B200P_E_DTYPE;
    if (n_waves < 0) return B200P_E_LENGTH;
    if (n_waves == 0) return B200P_OK;
    if (!in || !out) return B200P_E_NULL;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    const bool narrow = dtype == B200P_F16 || dtype == B200P_BF16;
    if (narrow && (fn == 2 || (fn == 1 && op != B200P_SUM))) return B200P_E_OP;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int wpb = 4, grid = (n_waves + wpb - 1) / wpb, tpb = (n_waves < wpb ? n_waves : wpb) * 32;
    switch (dtype) {
        case B200P_F32:  wave_probe_kernel<float><<<grid, tpb, 0, st>>>(fn, op, (const float*)in, (float*)out, n_waves); break;
        case B200P_F64:  wave_probe_kernel<double><<<grid, tpb, 0, st>>>(fn, op, (const double*)in, (double*)out, n_waves); break;
        case B200P_I32:  wave_probe_kernel<int><<<grid, tpb, 0, st>>>(fn, op, (const int*)in, (int*)out, n_waves); break;
        case B200P_I64:  wave_probe_kernel<long long><<<grid, tpb, 0, st>>>(fn, op, (const long long*)in, (long long*)out, n_waves); break;
        case B200P_F16:  wave_probe_narrow_kernel<__half><<<grid, tpb, 0, st>>>(fn, op, (const __half*)in, (__half*)out, n_waves); break;
        case B200P_BF16: wave_probe_narrow_kernel<__nv_bfloat16><<<grid, tpb, 0, st>>>(fn, op, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, n_waves); break;
    }
    return launched();
}

extern "C" int b200p_wave_probe(int fn, int op, int dtype, const void* in, void* out, b200p_stream_t stream) {
    return b200p_wave_probe_n(fn, op, dtype, in, out, 1, stream);
}

extern "C" int b200p_wave_vote_probe(const int* in64, unsigned long long* out8, b200p_stream_t stream) {
    if (!in64 || !out8) return B200P_E_NULL;
    if (sm_count() <= 0) return B200P_E_NO_DEVICE;
    wave_vote_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(in64, out8);
    return launched();
}
