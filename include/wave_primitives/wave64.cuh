// ---------------------------------------------------------------------------
// wave_primitives/wave64.cuh -- wave64 cross-lane primitives for sm_100a.
//
// Drop-in for the device API of the reference's wave-primitives headers
//   research/wave-primitives/include/wave_primitives/wave_reduce_dpp.hpp:106-113
//   research/wave-primitives/include/wave_primitives/wave_scan_dpp.hpp:70-87
//   research/wave-primitives/include/wave_primitives/wave_reduce.hpp:48-119
//   research/wave-primitives/include/wave_primitives/wave_scan.hpp:52-74
// with the same names (wave::dpp::reduce_sum / reduce_max / reduce_min,
// *_bcast, scan_inclusive_{sum,max,min}, scan_exclusive_sum) and the same
// per-64-element segment semantics, on a 32-lane warp.
//
// A 64-element "wave" is held by ONE warp: every lane owns a run of VEC
// consecutive elements of the segment (VEC = 2 for a whole-warp segment: lane
// l holds elements 2l and 2l+1).  Wider runs (VEC = 4, 8, 16) put several
// independent segments in one warp (64/VEC lanes each) and exist so that a
// streaming kernel can issue one 16- or 32-byte load per lane.
//
// Everything is shuffle / redux.sync only: no shared memory is touched.
//
// Summation order.  The reference's dpp_reduce builds a balanced tree over
// ADJACENT pairs: in each 16-lane row offsets 1,2,4,8 give
// ((x15+x14)+(x13+x12))+..., then row_bcast15 / row_bcast31 give
// (r3+r2)+(r1+r0) on lane 63.  A local balanced tree over the lane's run
// followed by an xor butterfly (masks 1,2,4,...) builds exactly that tree, and
// IEEE addition is commutative, so float/double sums are bit-identical to the
// reference's order; every lane ends with the result, so reduce_x and
// reduce_x_bcast coincide.
//
// The scans reproduce the reference's association as well: Kogge-Stone inside
// each 16-element row (offsets 1,2,4,8, out-of-row reads give the identity,
// which is still combined), then the row carries t0, t1+t0, (t2+t1)+t0
// (wave_scan_dpp.hpp:51-68).  Integer scans use the cheaper "local prefix +
// warp scan of run totals" form, which is exact for wrapping integers.
//
// max/min use a>b?a:b / a<b?a:b like the reference.  The operand order inside
// the butterfly is not the reference's, so inputs that compare equal but differ
// in bits (+0/-0) or NaNs may select a different bit pattern.
// ---------------------------------------------------------------------------
#pragma once
#ifdef WAVE64_HOST_EMULATION
// Tests only: a host shim (named by the macro) supplies a 32-thread lockstep
// stand-in for %laneid, the *_sync intrinsics and redux.sync, so that the
// cross-lane logic below can be checked on a machine without a GPU.
#include WAVE64_HOST_EMULATION
#else
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#endif
#include <cstdint>
#include <limits>
#include <type_traits>

// redux.sync over a sub-warp member mask is issued once per distinct mask, so for the
// short lane groups of wide vectors a shuffle butterfly is cheaper; groups of at
// least this many lanes use redux.sync.
#ifndef WAVE64_REDUX_MIN_LANES
#define WAVE64_REDUX_MIN_LANES 32
#endif

namespace wave {

constexpr unsigned kFullMask = 0xffffffffu;
constexpr int kSegment = 64;   // elements per wave64 segment

#ifndef WAVE64_HOST_EMULATION
__device__ __forceinline__ unsigned lane_id() {
    unsigned id;
    asm("mov.u32 %0, %%laneid;" : "=r"(id));
    return id;
}
// The lane index read afresh at every call (volatile: never hoisted out of a caller's loop).  The scans select on
// the lane index; when that index is loop-invariant the compiler may unswitch the caller's loop on it and give
// lane 0 a loop body of its own -- legal, but the full-mask shuffles of the two bodies then meet from different
// program counters and take ~300 cycles each (a 32-bit pair scan in a loop: 1900 cycles instead of 250).
__device__ __forceinline__ unsigned lane_id_here() {
    unsigned id;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(id));
    return id;
}
namespace detail {
__device__ __forceinline__ float redux_max_f32(unsigned m, float v) { float r; asm volatile("redux.sync.max.f32 %0, %1, %2;" : "=f"(r) : "f"(v), "r"(m)); return r; }
__device__ __forceinline__ float redux_min_f32(unsigned m, float v) { float r; asm volatile("redux.sync.min.f32 %0, %1, %2;" : "=f"(r) : "f"(v), "r"(m)); return r; }
} // namespace detail
#endif

// --- op functors (same comparison forms as wave_reduce_dpp.hpp:101-103) -----
struct SumOp {
    template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a + b; }
    template <typename T> static __device__ __forceinline__ T identity() { return T(0); }
};
struct MaxOp {
    template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a > b ? a : b; }
    template <typename T> static __device__ __forceinline__ T identity() { return std::numeric_limits<T>::lowest(); }
};
struct MinOp {
    template <typename T> __device__ __forceinline__ T operator()(T a, T b) const { return a < b ? a : b; }
    template <typename T> static __device__ __forceinline__ T identity() { return std::numeric_limits<T>::max(); }
};

namespace detail {

template <typename T> __device__ __forceinline__ T shfl_xor(T v, int m)         { return __shfl_xor_sync(kFullMask, v, m); }
template <typename T> __device__ __forceinline__ T shfl_up(T v, unsigned d)     { return __shfl_up_sync(kFullMask, v, d); }
template <typename T> __device__ __forceinline__ T shfl_idx(T v, int src)       { return __shfl_sync(kFullMask, v, src); }

// Mask of the lanes that hold the same segment as this lane (LPS lanes/segment).
template <int LPS> __device__ __forceinline__ unsigned segment_mask() {
    if constexpr (LPS == 32) return kFullMask;
    else {
        const unsigned base = lane_id() & ~unsigned(LPS - 1);
        return ((1u << LPS) - 1u) << base;
    }
}

// redux.sync: one instruction for a whole lane group.  Integer forms are in
// the CUDA headers; the f32 max/min forms exist on sm_100a as PTX only.
template <typename Op> struct Redux;
template <> struct Redux<SumOp> {
    static __device__ __forceinline__ int      run(unsigned m, int v)      { return __reduce_add_sync(m, v); }
};
template <> struct Redux<MaxOp> {
    static __device__ __forceinline__ int      run(unsigned m, int v)      { return __reduce_max_sync(m, v); }
    static __device__ __forceinline__ float    run(unsigned m, float v)    { return redux_max_f32(m, v); }
};
template <> struct Redux<MinOp> {
    static __device__ __forceinline__ int      run(unsigned m, int v)      { return __reduce_min_sync(m, v); }
    static __device__ __forceinline__ float    run(unsigned m, float v)    { return redux_min_f32(m, v); }
};

template <typename T, typename Op> struct has_redux : std::false_type {};
template <typename Op>             struct has_redux<int, Op> : std::true_type {};
template <>                        struct has_redux<float, MaxOp> : std::true_type {};
template <>                        struct has_redux<float, MinOp> : std::true_type {};

} // namespace detail

// ---------------------------------------------------------------------------
// segment_reduce<VEC>: reduce the 64-element segment this lane belongs to.
// v[0..VEC) are the lane's consecutive elements; 64/VEC lanes share a segment.
// Returns the segment result on EVERY lane of the segment.
// ---------------------------------------------------------------------------
template <int VEC, typename T, typename Op>
__device__ __forceinline__ T segment_reduce(const T (&v)[VEC], Op op) {
    static_assert(VEC == 2 || VEC == 4 || VEC == 8 || VEC == 16, "run length");
    constexpr int LPS = kSegment / VEC;
    T t[VEC];
    #pragma unroll
    for (int i = 0; i < VEC; ++i) t[i] = v[i];
    // local balanced tree over adjacent pairs
    #pragma unroll
    for (int s = 1; s < VEC; s <<= 1) {
        #pragma unroll
        for (int i = 0; i < VEC; i += 2 * s) t[i] = op(t[i + s], t[i]);
    }
    T r = t[0];
    if constexpr (detail::has_redux<T, Op>::value && LPS >= WAVE64_REDUX_MIN_LANES) {
        r = detail::Redux<Op>::run(detail::segment_mask<LPS>(), r);
    } else {
        #pragma unroll
        for (int m = 1; m < LPS; m <<= 1) r = op(r, detail::shfl_xor(r, m));
    }
    return r;
}

// ---------------------------------------------------------------------------
// lane_group_reduce<LANES>: xor-butterfly reduction over aligned groups of
// LANES lanes (2, 4, 8, 16 or 32); every lane of a group gets the result.
// The attention kernels use it for online-softmax row max / row sum where a
// score row is spread over a lane group (4 lanes in the MMA accumulator
// layout, 8 lanes in the vector decode kernel).
// ---------------------------------------------------------------------------
template <int LANES, typename T, typename Op>
__device__ __forceinline__ T lane_group_reduce(T v, Op op) {
    static_assert(LANES >= 1 && LANES <= 32 && (LANES & (LANES - 1)) == 0, "power of two");
    #pragma unroll
    for (int m = 1; m < LANES; m <<= 1) v = op(v, detail::shfl_xor(v, m));
    return v;
}

// ---------------------------------------------------------------------------
// The reference's PORTABLE reduction order (wave_reduce.hpp:40-63): six steps
// v[i] = op(v[i], v[i + o]) with o = 32, 16, ..., 1, result on element 0, i.e.
// elements (i, i + 32) meet first.  Its 16-bit overloads prescribe this order
// in fp32, so the 16-bit sums use it to agree bit for bit.
//
// lane_reduce_shfl_down_order<64>: ONE lane holds the whole segment; the tree
// runs in registers with no cross-lane traffic.
// pair_reduce_shfl_down_order: the segment is a pair per lane (elements 2l,
// 2l+1).  Elements i and i + 32 sit in lanes l and l + 16, then l and l + 8, ...
// so the first five levels are xor butterflies (masks 16, 8, 4, 2, 1) on both
// elements and the last level is a (op) b inside the lane; op is commutative, so
// both partners compute the same bits and every lane ends with the result.
// ---------------------------------------------------------------------------
template <int N, typename T, typename Op>
__device__ __forceinline__ T lane_reduce_shfl_down_order(T (&v)[N], Op op) {
    #pragma unroll
    for (int o = N / 2; o > 0; o >>= 1) {
        #pragma unroll
        for (int i = 0; i < o; ++i) v[i] = op(v[i], v[i + o]);
    }
    return v[0];
}
template <typename T, typename Op>
__device__ __forceinline__ T pair_reduce_shfl_down_order(T a, T b, Op op) {
    #pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        a = op(a, detail::shfl_xor(a, m));
        b = op(b, detail::shfl_xor(b, m));
    }
    return op(a, b);
}

// ---------------------------------------------------------------------------
// Kogge-Stone inclusive scan over rows of ROW consecutive elements, VEC per
// lane.  Step with offset o: x[i] = op(x[i], i-o inside the row ? x[i-o] : id).
// This is the association of the reference's row_shr cascade (ROW = 16,
// wave_scan_dpp.hpp:55-58) and of its portable Hillis-Steele loop (ROW = 64,
// wave_scan.hpp:40-48).
// ---------------------------------------------------------------------------
template <int VEC, int ROW, typename T, typename Op>
__device__ __forceinline__ void row_scan_kogge_stone(T (&v)[VEC], Op op, T identity) {
    constexpr int LPR = ROW / VEC;                 // lanes per row
    static_assert(LPR >= 1 && LPR <= 32, "row must fit a warp");
    const unsigned q = lane_id_here() & unsigned(LPR - 1);   // lane position inside its row
    #pragma unroll
    for (int o = 1; o < ROW; o <<= 1) {
        T old[VEC];
        #pragma unroll
        for (int j = 0; j < VEC; ++j) old[j] = v[j];
        if (o < VEC) {
            // the first o elements read from the previous lane's tail
            #pragma unroll
            for (int j = 0; j < VEC; ++j) {
                T src;
                if (j >= o) {
                    src = old[j - o];
                } else {
                    T up = detail::shfl_up(old[VEC - o + j], 1);
                    src = (q >= 1u) ? up : identity;
                }
                v[j] = op(old[j], src);
            }
        } else {
            const unsigned dl = unsigned(o / VEC);   // whole lanes
            #pragma unroll
            for (int j = 0; j < VEC; ++j) {
                T up = detail::shfl_up(old[j], dl);
                T src = (q >= dl) ? up : identity;
                v[j] = op(old[j], src);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// lane_scan_kogge_stone<N>: the same Kogge-Stone dataflow over N values that ONE
// lane holds (no cross-lane traffic at all): after the step with offset o,
// v[i] = v[i] (op) v[i - o] for i >= o.  Bitwise the result of
// row_scan_kogge_stone over a row of N one-element lanes.  Descending i lets the
// update run in place.
// ---------------------------------------------------------------------------
template <int N, typename T, typename Op>
__device__ __forceinline__ void lane_scan_kogge_stone(T (&v)[N], Op op) {
    #pragma unroll
    for (int o = 1; o < N; o <<= 1) {
        #pragma unroll
        for (int i = N - 1; i >= o; --i) v[i] = op(v[i], v[i - o]);
    }
}

// ---------------------------------------------------------------------------
// segment_scan_dpp_order<VEC>: inclusive scan of the lane's 64-element segment
// with the reference's full-DPP association (rows of 16 + cascaded carries).
// ---------------------------------------------------------------------------
template <int VEC, typename T, typename Op>
__device__ __forceinline__ void segment_scan_dpp_order(T (&v)[VEC], Op op, T identity) {
    static_assert(VEC == 2 || VEC == 4 || VEC == 8 || VEC == 16, "run length");
    constexpr int LPS = kSegment / VEC;            // lanes per segment
    constexpr int LPR = 16 / VEC;                  // lanes per 16-element row
    row_scan_kogge_stone<VEC, 16>(v, op, identity);
    const unsigned lane = lane_id_here();
    const unsigned seg0 = lane & ~unsigned(LPS - 1);
    const unsigned row  = (lane & unsigned(LPS - 1)) / unsigned(LPR);
    // Row totals sit on the last element of the last lane of each row.
    const T t0 = detail::shfl_idx(v[VEC - 1], int(seg0 + 1 * LPR - 1));
    const T t1 = detail::shfl_idx(v[VEC - 1], int(seg0 + 2 * LPR - 1));
    const T t2 = detail::shfl_idx(v[VEC - 1], int(seg0 + 3 * LPR - 1));
    // c1 / c1b / c1c of the reference: the totals of the 1st, 2nd, 3rd row
    // below this one, combined nearest-first.
    const T c2 = op(t1, t0), c3 = op(op(t2, t1), t0);
    const T carry = row == 1u ? t0 : row == 2u ? c2 : c3;
    #pragma unroll
    for (int j = 0; j < VEC; ++j) {
        const T w = op(v[j], carry);
        v[j] = row >= 1u ? w : v[j];
    }
    (void)identity;
}

// ---------------------------------------------------------------------------
// segment_scan_fast<VEC>: local prefix + warp scan of the run totals.  Any
// association; used for integers (exact) and available for floating point
// where bitwise agreement with the reference order is not needed.
// ---------------------------------------------------------------------------
template <int VEC, typename T, typename Op>
__device__ __forceinline__ void segment_scan_fast(T (&v)[VEC], Op op, T identity) {
    constexpr int LPS = kSegment / VEC;
    #pragma unroll
    for (int j = 1; j < VEC; ++j) v[j] = op(v[j], v[j - 1]);
    const unsigned q = lane_id_here() & unsigned(LPS - 1);
    T tot = v[VEC - 1];
    // every lane runs the same instructions: lanes a step does not apply to keep their value through a select
    #pragma unroll
    for (int d = 1; d < LPS; d <<= 1) {
        const T up = detail::shfl_up(tot, unsigned(d));
        const T sum = op(tot, up);
        tot = q >= unsigned(d) ? sum : tot;
    }
    if constexpr (std::is_same<Op, SumOp>::value && std::is_integral<T>::value) {
        // wrapping integer sums have an inverse: the exclusive prefix is the inclusive one minus the lane's own total
        const T excl = tot - v[VEC - 1];
        #pragma unroll
        for (int j = 0; j < VEC; ++j) v[j] = v[j] + excl;
    } else {
        const T excl = detail::shfl_up(tot, 1);
        #pragma unroll
        for (int j = 0; j < VEC; ++j) {
            const T w = op(v[j], excl);
            v[j] = q != 0u ? w : v[j];
        }
    }
    (void)identity;
}

// Shift an inclusive scan right by one element inside the segment (element 0
// receives `first`): the reference's scan_exclusive_sum (wave_scan_dpp.hpp:74-87).
template <int VEC, typename T>
__device__ __forceinline__ void segment_shift_right(T (&v)[VEC], T first) {
    constexpr int LPS = kSegment / VEC;
    const unsigned q = lane_id_here() & unsigned(LPS - 1);
    T prev = detail::shfl_up(v[VEC - 1], 1);
    if (q == 0u) prev = first;
    #pragma unroll
    for (int j = VEC - 1; j >= 1; --j) v[j] = v[j - 1];
    v[0] = prev;
}

// ===========================================================================
// Public API, reference names.
// ===========================================================================
namespace dpp {

// ---- wave64: the lane passes its adjacent pair (elements 2l, 2l+1) ---------
template <typename T> __device__ __forceinline__ T reduce_sum(T a, T b) { T v[2] = {a, b}; return segment_reduce<2>(v, SumOp{}); }
template <typename T> __device__ __forceinline__ T reduce_max(T a, T b) { T v[2] = {a, b}; return segment_reduce<2>(v, MaxOp{}); }
template <typename T> __device__ __forceinline__ T reduce_min(T a, T b) { T v[2] = {a, b}; return segment_reduce<2>(v, MinOp{}); }
// The butterfly leaves the result on every lane, so the broadcast forms are aliases.
template <typename T> __device__ __forceinline__ T reduce_sum_bcast(T a, T b) { return reduce_sum(a, b); }
template <typename T> __device__ __forceinline__ T reduce_max_bcast(T a, T b) { return reduce_max(a, b); }
template <typename T> __device__ __forceinline__ T reduce_min_bcast(T a, T b) { return reduce_min(a, b); }

template <typename T, typename Op>
__device__ __forceinline__ void scan_inclusive(T& a, T& b, Op op) {
    T v[2] = {a, b};
    if constexpr (std::is_integral<T>::value) segment_scan_fast<2>(v, op, Op::template identity<T>());
    else                                      segment_scan_dpp_order<2>(v, op, Op::template identity<T>());
    a = v[0]; b = v[1];
}
template <typename T> __device__ __forceinline__ void scan_inclusive_sum(T& a, T& b) { scan_inclusive(a, b, SumOp{}); }
template <typename T> __device__ __forceinline__ void scan_inclusive_max(T& a, T& b) { scan_inclusive(a, b, MaxOp{}); }
template <typename T> __device__ __forceinline__ void scan_inclusive_min(T& a, T& b) { scan_inclusive(a, b, MinOp{}); }
template <typename T> __device__ __forceinline__ void scan_exclusive_sum(T& a, T& b) {
    scan_inclusive_sum(a, b);
    T v[2] = {a, b};
    segment_shift_right<2>(v, T(0));
    a = v[0]; b = v[1];
}

// ---- 32-lane forms: the meaning the reference gives these names on a 32-wide
// machine (wave_reduce_dpp.hpp:115-128, wave_scan_dpp.hpp:89-106): one value
// per lane, reduce over the warp.  Here every lane gets the result.
template <typename T, typename Op>
__device__ __forceinline__ T warp_reduce(T v, Op op) {
    if constexpr (detail::has_redux<T, Op>::value) {
        return detail::Redux<Op>::run(kFullMask, v);
    } else {
        #pragma unroll
        for (int m = 1; m < 32; m <<= 1) v = op(v, detail::shfl_xor(v, m));
        return v;
    }
}
template <typename T> __device__ __forceinline__ T reduce_sum(T v) { return warp_reduce(v, SumOp{}); }
template <typename T> __device__ __forceinline__ T reduce_max(T v) { return warp_reduce(v, MaxOp{}); }
template <typename T> __device__ __forceinline__ T reduce_min(T v) { return warp_reduce(v, MinOp{}); }
template <typename T> __device__ __forceinline__ T reduce_sum_bcast(T v) { return reduce_sum(v); }
template <typename T> __device__ __forceinline__ T reduce_max_bcast(T v) { return reduce_max(v); }
template <typename T> __device__ __forceinline__ T reduce_min_bcast(T v) { return reduce_min(v); }

template <typename T, typename Op>
__device__ __forceinline__ T warp_scan_inclusive(T v, Op op) {
    const unsigned l = lane_id_here();
    #pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T u = detail::shfl_up(v, unsigned(o));
        const T w = op(v, u);
        v = l >= unsigned(o) ? w : v;
    }
    return v;
}
template <typename T> __device__ __forceinline__ T scan_inclusive_sum(T v) { return warp_scan_inclusive(v, SumOp{}); }
template <typename T> __device__ __forceinline__ T scan_inclusive_max(T v) { return warp_scan_inclusive(v, MaxOp{}); }
template <typename T> __device__ __forceinline__ T scan_inclusive_min(T v) { return warp_scan_inclusive(v, MinOp{}); }
template <typename T> __device__ __forceinline__ T scan_exclusive_sum(T v) {
    T inc = scan_inclusive_sum(v);
    T ex = detail::shfl_up(inc, 1);
    return lane_id_here() == 0u ? T(0) : ex;
}

} // namespace dpp

#ifndef WAVE64_HOST_EMULATION
// ===========================================================================
// Vote / predicate operations and bitwise reductions (wave_ballot.hpp:23-75,
// wave_reduce.hpp reduce_and / reduce_or).  A wave64 ballot is 64 bits: with a
// pair per lane, bit 2l is lane l's first predicate and bit 2l+1 its second.
// The one-argument forms are the 32-lane meaning (upper 32 bits zero), as the
// reference defines them on a 32-wide machine.
// ===========================================================================
using mask_t = unsigned long long;
__device__ __forceinline__ mask_t activemask() { return mask_t(__activemask()); }
__device__ __forceinline__ mask_t ballot(int predicate) { return mask_t(__ballot_sync(kFullMask, predicate)); }
__device__ __forceinline__ mask_t ballot(int pa, int pb) {
    const unsigned ea = __ballot_sync(kFullMask, pa), eb = __ballot_sync(kFullMask, pb);
    // interleave: bit l of ea -> bit 2l, bit l of eb -> bit 2l + 1
    auto spread = [](unsigned x) {
        mask_t v = x;
        v = (v | (v << 16)) & 0x0000ffff0000ffffull;
        v = (v | (v << 8))  & 0x00ff00ff00ff00ffull;
        v = (v | (v << 4))  & 0x0f0f0f0f0f0f0f0full;
        v = (v | (v << 2))  & 0x3333333333333333ull;
        v = (v | (v << 1))  & 0x5555555555555555ull;
        return v;
    };
    return spread(ea) | (spread(eb) << 1);
}
__device__ __forceinline__ int any(int predicate) { return __any_sync(kFullMask, predicate); }
__device__ __forceinline__ int all(int predicate) { return __all_sync(kFullMask, predicate); }
__device__ __forceinline__ int any(int pa, int pb) { return __any_sync(kFullMask, pa || pb); }
__device__ __forceinline__ int all(int pa, int pb) { return __all_sync(kFullMask, pa && pb); }
__device__ __forceinline__ int popcount(int predicate) { return __popc(__ballot_sync(kFullMask, predicate)); }
__device__ __forceinline__ int popcount(int pa, int pb) { return __popc(__ballot_sync(kFullMask, pa)) + __popc(__ballot_sync(kFullMask, pb)); }
// bits of the elements before this lane's first element (wave64: 2 * lane of them)
__device__ __forceinline__ mask_t lane_mask_lt() { const unsigned l = lane_id(); return l == 0 ? 0ull : ((1ull << l) - 1ull); }
__device__ __forceinline__ mask_t lane_mask_le() { const unsigned l = lane_id(); return (l >= 63u) ? ~0ull : ((1ull << (l + 1)) - 1ull); }
// bitwise reductions over the wave (redux.sync), result on every lane
__device__ __forceinline__ unsigned reduce_and(unsigned v) { return __reduce_and_sync(kFullMask, v); }
__device__ __forceinline__ unsigned reduce_or(unsigned v)  { return __reduce_or_sync(kFullMask, v); }
__device__ __forceinline__ unsigned reduce_and(unsigned a, unsigned b) { return __reduce_and_sync(kFullMask, a & b); }
__device__ __forceinline__ unsigned reduce_or(unsigned a, unsigned b)  { return __reduce_or_sync(kFullMask, a | b); }
#endif

#ifndef WAVE64_HOST_EMULATION
// ===========================================================================
// 16-bit inputs with fp32 accumulation (wave_reduce.hpp:48-63, wave_scan.hpp:52-74).
// The reference converts each lane's value to float, combines in float and
// converts back; these overloads take the lane's adjacent pair and return the
// float result (`*_f32`) or the value rounded to the input type.
// ===========================================================================
__device__ __forceinline__ float to_f32(__half h)        { return __half2float(h); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 h) { return __bfloat162float(h); }
template <typename N> __device__ __forceinline__ N from_f32(float f);
template <> __device__ __forceinline__ __half        from_f32<__half>(float f)        { return __float2half_rn(f); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float f) { return __float2bfloat16_rn(f); }

// sum: the portable order (i, i + 32 first) the reference's 16-bit overloads use; max / min do not depend on the order
template <typename N> __device__ __forceinline__ float reduce_sum_f32(N a, N b) { return pair_reduce_shfl_down_order(to_f32(a), to_f32(b), SumOp{}); }
template <typename N> __device__ __forceinline__ float reduce_max_f32(N a, N b) { return dpp::reduce_max(to_f32(a), to_f32(b)); }
template <typename N> __device__ __forceinline__ float reduce_min_f32(N a, N b) { return dpp::reduce_min(to_f32(a), to_f32(b)); }

__device__ __forceinline__ __half        reduce_sum(__half a, __half b)               { return from_f32<__half>(reduce_sum_f32(a, b)); }
__device__ __forceinline__ __half        reduce_max(__half a, __half b)               { return from_f32<__half>(reduce_max_f32(a, b)); }
__device__ __forceinline__ __half        reduce_min(__half a, __half b)               { return from_f32<__half>(reduce_min_f32(a, b)); }
__device__ __forceinline__ __nv_bfloat16 reduce_sum(__nv_bfloat16 a, __nv_bfloat16 b) { return from_f32<__nv_bfloat16>(reduce_sum_f32(a, b)); }
__device__ __forceinline__ __nv_bfloat16 reduce_max(__nv_bfloat16 a, __nv_bfloat16 b) { return from_f32<__nv_bfloat16>(reduce_max_f32(a, b)); }
__device__ __forceinline__ __nv_bfloat16 reduce_min(__nv_bfloat16 a, __nv_bfloat16 b) { return from_f32<__nv_bfloat16>(reduce_min_f32(a, b)); }

// Inclusive sum scan of a 16-bit pair: float Kogge-Stone over the whole 64
// (the reference's Hillis-Steele association), rounded once at the end.
template <typename N>
__device__ __forceinline__ void scan_inclusive_sum_narrow(N& a, N& b) {
    float v[2] = {to_f32(a), to_f32(b)};
    row_scan_kogge_stone<2, 64>(v, SumOp{}, 0.0f);
    a = from_f32<N>(v[0]); b = from_f32<N>(v[1]);
}
__device__ __forceinline__ void scan_inclusive_sum(__half& a, __half& b)               { scan_inclusive_sum_narrow(a, b); }
__device__ __forceinline__ void scan_inclusive_sum(__nv_bfloat16& a, __nv_bfloat16& b) { scan_inclusive_sum_narrow(a, b); }
#endif // !WAVE64_HOST_EMULATION

} // namespace wave
