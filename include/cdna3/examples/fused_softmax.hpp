// ---------------------------------------------------------------------------
// cdna3/examples/fused_softmax.hpp -- row softmax building blocks on the wave
// primitives: cdna3::ex::row_softmax_lane and cdna3::ex::online_softmax_step of
// the reference (cdna3-prims/examples/fused_softmax.hpp:26-48).
//
// A 64-score row is held by one warp as an adjacent pair per lane (scores 2l and
// 2l+1), the shape the pair overloads of wave64.cuh reduce.  The one-score forms
// keep the reference's signatures for a 32-wide row (one score per lane).
// ---------------------------------------------------------------------------
#pragma once
#include "../cdna3.hpp"

namespace cdna3 {
namespace ex {

// Softmax of a row held one score per lane (32-wide row): this lane's probability.
__device__ __forceinline__ float row_softmax_lane(float score) {
    const float m = wave::dpp::reduce_max_bcast(score);
    const float e = __expf(score - m);
    const float s = wave::dpp::reduce_sum_bcast(e);
    return s > 0.f ? e / s : 0.f;
}
// Softmax of a 64-wide row, pair per lane: p0, p1 receive this lane's two probabilities.
__device__ __forceinline__ void row_softmax_lane(float s0, float s1, float& p0, float& p1) {
    const float m = wave::dpp::reduce_max_bcast(s0, s1);
    const float e0 = __expf(s0 - m), e1 = __expf(s1 - m);
    const float s = wave::dpp::reduce_sum_bcast(e0, e1);
    const float inv = s > 0.f ? 1.f / s : 0.f;
    p0 = e0 * inv; p1 = e1 * inv;
}

// One step of the online softmax over a stream of row tiles:
//   m_new = max(m_run, rowmax);  p = exp(score - m_new);  l_run = exp(m_run - m_new) * l_run + rowsum(p)
// Returns the factor by which the caller rescales its accumulator O before adding p . V.
__device__ __forceinline__ float online_softmax_step(float score, float& m_run, float& l_run, float& p_out) {
    const float m_new = fmaxf(m_run, wave::dpp::reduce_max_bcast(score));
    const float p = __expf(score - m_new);
    const float resc = __expf(m_run - m_new);
    l_run = resc * l_run + wave::dpp::reduce_sum_bcast(p);
    m_run = m_new;
    p_out = p;
    return resc;
}
// 64-wide tile, pair per lane.
__device__ __forceinline__ float online_softmax_step(float s0, float s1, float& m_run, float& l_run, float& p0, float& p1) {
    const float m_new = fmaxf(m_run, wave::dpp::reduce_max_bcast(s0, s1));
    p0 = __expf(s0 - m_new); p1 = __expf(s1 - m_new);
    const float resc = __expf(m_run - m_new);
    l_run = resc * l_run + wave::dpp::reduce_sum_bcast(p0, p1);
    m_run = m_new;
    return resc;
}

} // namespace ex
} // namespace cdna3
